// Dense batch allocator: pinned staging + asynchronous host-to-device copies on side streams, ordered against
// the compute stream by events.  Takes over BatchAllocator's dense path (source/batchAllocator.cpp:101-251
// init, 253-274 buffers, 340-366 first batch, 399-425 staging memcpy, 759-777 + 843-847 async copies,
// 977-994 + 1036-1053 swap and wrap-around).
//
// Differences from the reference, none visible in the results: the swap does not block the host
// (cudaStreamWaitEvent instead of cudaStreamSynchronize), the device buffers are sized once for a full batch so
// the short last batch needs no cudaFree / cudaMalloc, and the next copy is ordered after the transposes that
// read the previous one.
//
// Options of cn_batch_create_ex (flags):
//   CN_BATCH_KEEP_ROW_MAJOR  the row-major device copy of the CURRENT batch stays valid until the next swap (two
//                            row-major buffers that alternate), so that a product can read the batch as a transposed
//                            operand (cn_tdotmpi_f32 / cn_gemm_f32 with transA) without the col-major detour;
//   CN_BATCH_NO_COL_MAJOR    X is not transposed into col-major at the swap at all (implies the former);
//   CN_BATCH_SHARDED_UPLOAD  every rank of the communicator holds the data set (the reference's Matrix* form of init,
//                            source/batchAllocator.cpp:411-440, where the rank-0 guard around the staging memcpy is
//                            commented out): rank r copies only rows [r*floor(B/G), ...) of the batch over its own
//                            PCIe link and pushes that block into every peer's buffer over NVLink (copy engine, peer
//                            addresses of a symmetric buffer), framed by two bounded cross-GPU flag exchanges on the
//                            copy stream ("your buffer may be overwritten" / "my block has arrived").  One link no
//                            longer carries the whole batch.
//   CN_BATCH_PUSH_BY_KERNEL  the push of the sharded upload by one kernel's stores instead of the copy engines;
//   CN_BATCH_LOOKAHEAD       three row-major buffers and two copies in flight: the copy of the batch after next starts
//                            as soon as its buffer is free, so one copy's chain of waits has two steps to finish in.
#include <string.h>
#include "cn_internal.h"

struct cn_batch {
    cn_context *ctx = nullptr;
    const float *h_X = nullptr, *h_y = nullptr;   // caller's row-major data set (not owned)
    int64_t rows = 0, cols_X = 0, cols_y = 0, batch = 0;
    int skip_last = 0;
    int64_t total_batches = 0;
    int64_t next_batch = 0;      // m_next_batch_number
    int64_t next_rows = 0;       // rows of the batch now in the "next" buffers
    int64_t cur_rows = 0;
    bool copy_pending = false;
    bool direct = false;         // the data set itself is pinned: copy from it, no staging memcpy
    float *p_X = nullptr, *p_y = nullptr;     // pinned staging
    float *dn_y = nullptr;                    // device, next batch's labels, row-major
    // options (cn_batch_create_ex)
    int flags = 0;
    // Row-major X buffers form a ring: one (plain: transposed into dc_X at the swap), two (the current batch stays valid
    // while the next one is copied) or three (CN_BATCH_LOOKAHEAD: two copies in flight).  `fill` is where the next copy
    // goes, `ready` what the next swap takes, `in_flight` how many copies lie between them.
    int nb = 1, depth = 1;
    float *xb[3] = {nullptr, nullptr, nullptr};
    bool xb_sym = false;                      // xb[] came from cn_sym_alloc
    float *peer_xb[3][8] = {};                // peer addresses of xb[i]
    cudaEvent_t e_Xb[3] = {};                 // "buffer i holds its batch"
    int64_t rows_in[3] = {0, 0, 0}, idx_in[3] = {-1, -1, -1};
    int fill = 0, ready = 0, in_flight = 0;
    int staged_from = -1;                     // the buffer whose copy last read the staging memory
    int64_t x_next_idx = 0;                   // batch number of the next X copy to start
    float *cur_rm = nullptr;                  // row-major copy of the current batch
    int G = 1, rank = 0, slot = 0;
    unsigned int epoch = 0;
    // optional timing of the copy stream's phases (cn_batch_profile): start, after the "buffer free" exchange, after the
    // host-to-device copy, after the push to the peers, after the "arrived" exchange
    bool profile = false;
    cudaEvent_t e_prof[5] = {};
    float *dc_X = nullptr, *dc_y = nullptr;   // device, current batch, column-major
    cudaStream_t s_X = nullptr, s_y = nullptr;
    cudaEvent_t e_y = nullptr, e_consumed = nullptr;
};

// Sharded upload: this rank's block of the batch, already in its own buffer, goes to the same place in every peer's
// buffer with 16-byte stores to the peers' mapped memory (a warp writes 512 contiguous bytes per destination): one
// launch instead of one copy call per peer, chosen with CN_BATCH_PUSH_BY_KERNEL.  The default is the copy engines, which
// need no SM: beside a product whose CTAs fill the register files this kernel only runs in the gaps between launches.
// Plain stores, no multicast.
struct PushParams {
    float *dst[8];
    int ndst;
};
__global__ void __launch_bounds__(512)
cn_push_block_kernel(const float *__restrict__ src, int64_t n, const PushParams pp)
{
    const int64_t n4 = n >> 2, stride = (int64_t)gridDim.x * blockDim.x;
    const float4 *s4 = reinterpret_cast<const float4 *>(src);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 v = s4[i];
#pragma unroll 1
        for (int d = 0; d < pp.ndst; ++d) reinterpret_cast<float4 *>(pp.dst[d])[i] = v;
    }
    if (blockIdx.x == 0)
        for (int64_t i = (n4 << 2) + threadIdx.x; i < n; i += blockDim.x)
            for (int d = 0; d < pp.ndst; ++d) pp.dst[d][i] = src[i];
}

static int64_t rows_of_batch(const cn_batch *b, int64_t idx)
{
    // the batch that would run past the end of the training rows is the short one (source/batchAllocator.cpp:404-410)
    if (b->batch * (idx + 1) > b->rows) return b->rows % b->batch;
    return b->batch;
}

extern "C" int cn_batch_destroy(cn_batch *b)
{
    if (!b) return CN_OK;
    if (b->s_X) cudaStreamSynchronize(b->s_X);
    if (b->s_y) cudaStreamSynchronize(b->s_y);
    cudaFreeHost(b->p_X); cudaFreeHost(b->p_y);
    for (int i = 0; i < 3; ++i) {
        if (!b->xb[i]) continue;
        if (b->xb_sym) cn_sym_free(b->ctx, b->xb[i]); else cudaFree(b->xb[i]);
    }
    cudaFree(b->dn_y); cudaFree(b->dc_X); cudaFree(b->dc_y);
    if (b->s_X) cudaStreamDestroy(b->s_X);
    if (b->s_y) cudaStreamDestroy(b->s_y);
    for (cudaEvent_t e : b->e_Xb) if (e) cudaEventDestroy(e);
    if (b->e_y) cudaEventDestroy(b->e_y);
    if (b->e_consumed) cudaEventDestroy(b->e_consumed);
    for (cudaEvent_t e : b->e_prof) if (e) cudaEventDestroy(e);
    delete b;
    return CN_OK;
}

extern "C" int cn_batch_create(cn_context *ctx, const float *h_X, const float *h_y, int64_t rows, int64_t cols_X, int64_t cols_y,
                               int64_t batch_size, int skip_last_batch, cn_batch **out)
{
    return cn_batch_create_ex(ctx, h_X, h_y, rows, cols_X, cols_y, batch_size, skip_last_batch, 0, out);
}

extern "C" int cn_batch_create_ex(cn_context *ctx, const float *h_X, const float *h_y, int64_t rows, int64_t cols_X, int64_t cols_y,
                                  int64_t batch_size, int skip_last_batch, int flags, cn_batch **out)
{
    CN_REQUIRE(ctx && h_X && h_y && out, CN_ERR_ARG, "cn_batch_create: null argument");
    CN_REQUIRE((flags & ~(CN_BATCH_KEEP_ROW_MAJOR | CN_BATCH_NO_COL_MAJOR | CN_BATCH_SHARDED_UPLOAD | CN_BATCH_PUSH_BY_KERNEL |
                          CN_BATCH_LOOKAHEAD)) == 0, CN_ERR_ARG, "cn_batch_create_ex: unknown flag bits 0x%x", flags);
    if (flags & (CN_BATCH_NO_COL_MAJOR | CN_BATCH_LOOKAHEAD)) flags |= CN_BATCH_KEEP_ROW_MAJOR;
    const int G = cn_comm_size(ctx);
    if (G == 1) flags &= ~CN_BATCH_SHARDED_UPLOAD;   // nothing to share the upload with
    if (flags & CN_BATCH_SHARDED_UPLOAD) flags |= CN_BATCH_KEEP_ROW_MAJOR;
    CN_REQUIRE(G <= 8, CN_ERR_UNSUPPORTED, "cn_batch_create_ex: at most 8 ranks");
    CN_REQUIRE(rows > 0 && cols_X > 0 && cols_y > 0 && batch_size > 0, CN_ERR_ARG, "cn_batch_create: non-positive size");
    // "ERROR: Batch size must be smaller than the training set." (source/batchAllocator.cpp:135-139)
    CN_REQUIRE(batch_size <= rows, CN_ERR_SHAPE, "Batch size must be smaller than the training set.");
    *out = nullptr;
    cn_batch *b = new cn_batch();
    b->ctx = ctx;
    b->h_X = h_X; b->h_y = h_y;
    b->rows = rows; b->cols_X = cols_X; b->cols_y = cols_y; b->batch = batch_size;
    b->skip_last = skip_last_batch;
    b->flags = flags;
    b->G = G;
    b->rank = cn_comm_rank(ctx);
    b->total_batches = (rows + batch_size - 1) / batch_size;
    b->nb = (flags & CN_BATCH_LOOKAHEAD) ? 3 : (flags & CN_BATCH_KEEP_ROW_MAJOR) ? 2 : 1;
    b->depth = (flags & CN_BATCH_LOOKAHEAD) ? 2 : 1;
    const size_t bx = (size_t)batch_size * cols_X * sizeof(float), by = (size_t)batch_size * cols_y * sizeof(float);
    cudaError_t e;
    // The copy streams get the highest priority: their work is a few copies and, with the sharded upload, two one-warp flag
    // kernels, which must not queue behind the thousands of CTAs of a product that runs on the compute stream meanwhile.
    int prio_low = 0, prio_high = 0;
    cudaDeviceGetStreamPriorityRange(&prio_low, &prio_high);
    {   // the reference keeps the whole data set in pinned memory (empty_pinned); if the caller did the same, the
        // batch rows (contiguous in the row-major set) are copied straight from it
        cudaPointerAttributes ax, ay;
        const bool px = cudaPointerGetAttributes(&ax, h_X) == cudaSuccess && ax.type == cudaMemoryTypeHost;
        const bool py = cudaPointerGetAttributes(&ay, h_y) == cudaSuccess && ay.type == cudaMemoryTypeHost;
        cudaGetLastError();
        b->direct = px && py;
    }
    if ((!b->direct && (e = cudaHostAlloc(&b->p_X, bx, cudaHostAllocPortable)) != cudaSuccess) ||
        (!b->direct && (e = cudaHostAlloc(&b->p_y, by, cudaHostAllocPortable)) != cudaSuccess) ||
        (e = cudaMalloc(&b->dn_y, by)) != cudaSuccess ||
        (!(flags & CN_BATCH_NO_COL_MAJOR) && (e = cudaMalloc(&b->dc_X, bx)) != cudaSuccess) ||
        (e = cudaMalloc(&b->dc_y, by)) != cudaSuccess ||
        (e = cudaStreamCreateWithPriority(&b->s_X, cudaStreamNonBlocking, prio_high)) != cudaSuccess ||
        (e = cudaStreamCreateWithPriority(&b->s_y, cudaStreamNonBlocking, prio_high)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&b->e_Xb[0], cudaEventDisableTiming)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&b->e_Xb[1], cudaEventDisableTiming)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&b->e_Xb[2], cudaEventDisableTiming)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&b->e_y, cudaEventDisableTiming)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&b->e_consumed, cudaEventDisableTiming)) != cudaSuccess) {
        cn_batch_destroy(b);
        return cn_cuda_fail(e, "cn_batch_create");
    }
    for (int i = 0; i < b->nb; ++i) {
        int st2;
        if (flags & CN_BATCH_SHARDED_UPLOAD) {
            void *p = nullptr;
            st2 = cn_sym_alloc(ctx, bx, &p);   // collective: every rank creates its allocator at the same point
            b->xb[i] = (float *)p;
            b->xb_sym = true;
            void *peers[8] = {};
            if (st2 == CN_OK && !cn_comm_sym_peers(ctx, p, bx, peers)) {
                cn_set_error("cn_batch_create_ex: symmetric buffer not found");
                st2 = CN_ERR_CUDA;
            }
            for (int r = 0; r < G; ++r) b->peer_xb[i][r] = (float *)peers[r];
        } else {
            st2 = cudaMalloc(&b->xb[i], bx) == cudaSuccess ? CN_OK : cn_cuda_fail(cudaGetLastError(), "cn_batch_create_ex");
        }
        if (st2 != CN_OK) { cn_batch_destroy(b); return st2; }
    }
    if (flags & CN_BATCH_SHARDED_UPLOAD) {
        int st2 = cn_comm_flag_slots(ctx, 2, &b->slot);
        if (st2 != CN_OK) { cn_batch_destroy(b); return st2; }
    }
    // first batch: staged, copied and transposed before returning, as BatchAllocator::init does
    b->next_batch = 0;
    b->x_next_idx = 0;
    int st = cn_batch_copy_next_async(b);
    float *dx, *dy;
    int64_t r;
    if (st == CN_OK) st = cn_batch_swap(b, nullptr, &dx, &dy, &r);
    if (st == CN_OK && cudaStreamSynchronize(nullptr) != cudaSuccess) st = cn_cuda_fail(cudaGetLastError(), "cn_batch_create");
    if (st == CN_OK && (flags & CN_BATCH_SHARDED_UPLOAD)) {
        unsigned int *d_status = nullptr;   // the first exchange must not have timed out
        unsigned int h = 0;
        st = cn_status_block(ctx, &d_status);
        if (st == CN_OK && cudaMemcpy(&h, d_status, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) st = cn_cuda_fail(cudaGetLastError(), "cn_batch_create_ex");
        if (st == CN_OK && h != 0) {
            cn_set_error("cn_batch_create_ex: a peer did not take part in the first batch exchange (status %u)", h);
            st = CN_ERR_TIMEOUT;
        }
    }
    if (st != CN_OK) { cn_batch_destroy(b); return st; }
    *out = b;
    return CN_OK;
}

// the batch that follows batch idx: counter and wrap-around exactly as replace_current_batch_with_next
// (source/batchAllocator.cpp:1036-1052)
static int64_t batch_after(const cn_batch *b, int64_t idx)
{
    int64_t n = idx + 1;
    if ((n + 1) == b->total_batches && b->skip_last) n = 0;
    if (n >= b->total_batches) n = 0;
    return n;
}

extern "C" int cn_batch_set_skip_last(cn_batch *b, int skip)
{
    CN_REQUIRE(b, CN_ERR_ARG, "cn_batch_set_skip_last: null handle");
    b->skip_last = skip ? 1 : 0;
    // X copies already under way were chosen with the old setting: keep those that still lie on the new sequence, forget
    // the rest (their buffers are simply filled again; the copy stream keeps the order)
    int64_t expected = b->next_batch;
    int kept = 0;
    for (; kept < b->in_flight; ++kept) {
        if (b->idx_in[(b->ready + kept) % b->nb] != expected) break;
        expected = batch_after(b, expected);
    }
    b->in_flight = kept;
    b->fill = (b->ready + kept) % b->nb;
    b->x_next_idx = expected;
    return CN_OK;
}

extern "C" int64_t cn_batch_total_batches(const cn_batch *b) { return b ? b->total_batches : 0; }

extern "C" int cn_batch_current(const cn_batch *b, float **d_X, float **d_y, int64_t *batch_rows)
{
    CN_REQUIRE(b, CN_ERR_ARG, "cn_batch_current: null handle");
    if (d_X) *d_X = b->dc_X;
    if (d_y) *d_y = b->dc_y;
    if (batch_rows) *batch_rows = b->cur_rows;
    return CN_OK;
}

extern "C" int cn_batch_current_row_major(const cn_batch *b, float **d_X_row_major, int64_t *batch_rows)
{
    CN_REQUIRE(b, CN_ERR_ARG, "cn_batch_current_row_major: null handle");
    CN_REQUIRE(b->flags & CN_BATCH_KEEP_ROW_MAJOR, CN_ERR_ARG, "cn_batch_current_row_major: the allocator was created without CN_BATCH_KEEP_ROW_MAJOR");
    if (d_X_row_major) *d_X_row_major = b->cur_rm;
    if (batch_rows) *batch_rows = b->cur_rows;
    return CN_OK;
}

extern "C" int cn_batch_next_row_major(cn_batch *b, void *stream, float **d_X_row_major, int64_t *batch_rows)
{
    CN_REQUIRE(b, CN_ERR_ARG, "cn_batch_next_row_major: null handle");
    CN_REQUIRE(b->flags & CN_BATCH_KEEP_ROW_MAJOR, CN_ERR_ARG, "cn_batch_next_row_major: the allocator was created without CN_BATCH_KEEP_ROW_MAJOR");
    CN_REQUIRE(b->in_flight > 0, CN_ERR_ARG, "cn_batch_next_row_major: no copy under way (call cn_batch_copy_next_async first)");
    const int buf = b->ready;
    CN_CUDA(cudaStreamWaitEvent(cn_stream(stream), b->e_Xb[buf], 0));
    if (d_X_row_major) *d_X_row_major = b->xb[buf];
    if (batch_rows) *batch_rows = b->rows_in[buf];
    return CN_OK;
}

// Timing of the last sharded upload's phases on the copy stream, in milliseconds: [0] wait for the peers' "buffer free"
// flags, [1] host-to-device copy of the own block, [2] push to the peers, [3] wait for the peers' "arrived" flags.
// enable != 0 switches the recording on for the following copies; the call then returns the last recorded copy (zeros
// when there is none yet) after waiting for it.
extern "C" int cn_batch_profile(cn_batch *b, int enable, float *ms4)
{
    CN_REQUIRE(b, CN_ERR_ARG, "cn_batch_profile: null handle");
    if (ms4) ms4[0] = ms4[1] = ms4[2] = ms4[3] = 0.0f;
    if (b->profile && (b->flags & CN_BATCH_SHARDED_UPLOAD) && ms4 && b->epoch > 0) {
        if (cudaEventSynchronize(b->e_prof[4]) == cudaSuccess)
            for (int i = 0; i < 4; ++i) cudaEventElapsedTime(&ms4[i], b->e_prof[i], b->e_prof[i + 1]);
        cudaGetLastError();
    }
    if (enable && !b->e_prof[0])
        for (cudaEvent_t &e : b->e_prof) CN_CUDA(cudaEventCreate(&e));
    b->profile = enable != 0;
    return CN_OK;
}

// Start the copy of batch b->x_next_idx into the ring buffer b->fill.
static int start_x_copy(cn_batch *b)
{
    const int64_t idx = b->x_next_idx, r = rows_of_batch(b, idx);
    const int buf = b->fill;
    float *dst = b->xb[buf];
    const float *src_X = b->h_X + (size_t)idx * b->batch * b->cols_X;
    // rows of the batch this rank uploads itself: all of them, or its block of floor(r / G) rows (last rank: + remainder)
    int64_t row0 = 0, nrows = r;
    if (b->flags & CN_BATCH_SHARDED_UPLOAD) {
        const int64_t split = r / b->G;
        row0 = split * b->rank;
        nrows = (b->rank == b->G - 1) ? r - row0 : split;
    }
    const size_t off_X = (size_t)row0 * b->cols_X, bytes_X = (size_t)nrows * b->cols_X * sizeof(float);
    if (!b->direct) {
        // the staging buffer is free once the last copy out of it has finished
        if (b->staged_from >= 0) CN_CUDA(cudaEventSynchronize(b->e_Xb[b->staged_from]));
        memcpy(b->p_X + off_X, src_X + off_X, bytes_X);
        src_X = b->p_X;
        b->staged_from = buf;
    }
    // do not overwrite a buffer while the work that read it may still run: its last reader is the batch before the current
    // one (or, with one buffer, the last swap's transpose), and e_consumed, recorded at the last swap, follows both
    CN_CUDA(cudaStreamWaitEvent(b->s_X, b->e_consumed, 0));
    if (b->flags & CN_BATCH_SHARDED_UPLOAD) {
        // (1) every peer's buffer of this index must be free, and each rank says so only after its own e_consumed (waited
        //     for above); (2) own block over this rank's PCIe link; (3) the block into every peer's buffer over NVLink;
        //     (4) "my block has arrived everywhere"
        const unsigned int epoch = ++b->epoch;
        if (b->profile) CN_CUDA(cudaEventRecord(b->e_prof[0], b->s_X));
        int st = cn_comm_flag_barrier(b->ctx, b->slot, epoch, b->s_X);
        if (st != CN_OK) return st;
        if (b->profile) CN_CUDA(cudaEventRecord(b->e_prof[1], b->s_X));
        if (bytes_X) CN_CUDA(cudaMemcpyAsync(dst + off_X, src_X + off_X, bytes_X, cudaMemcpyHostToDevice, b->s_X));
        if (b->profile) CN_CUDA(cudaEventRecord(b->e_prof[2], b->s_X));
        if (bytes_X) {
            const bool aligned = (off_X % 4 == 0) && ((uintptr_t)dst % 16 == 0);   // 16-byte stores need it; buffers are 256-byte aligned
            if (aligned && (b->flags & CN_BATCH_PUSH_BY_KERNEL)) {
                PushParams pp;
                pp.ndst = 0;
                for (int p = 1; p < b->G; ++p) pp.dst[pp.ndst++] = b->peer_xb[buf][(b->rank + p) % b->G] + off_X;   // staggered by rank
                cn_push_block_kernel<<<32, 512, 0, b->s_X>>>(dst + off_X, (int64_t)(bytes_X / sizeof(float)), pp);
                CN_CUDA(cudaGetLastError());
                cn_count_launch();
            } else {
                for (int p = 1; p < b->G; ++p) {
                    const int peer = (b->rank + p) % b->G;
                    CN_CUDA(cudaMemcpyAsync(b->peer_xb[buf][peer] + off_X, dst + off_X, bytes_X, cudaMemcpyDeviceToDevice, b->s_X));
                }
            }
        }
        if (b->profile) CN_CUDA(cudaEventRecord(b->e_prof[3], b->s_X));
        if ((st = cn_comm_flag_barrier(b->ctx, b->slot + 1, epoch, b->s_X)) != CN_OK) return st;
        if (b->profile) CN_CUDA(cudaEventRecord(b->e_prof[4], b->s_X));
    } else {
        CN_CUDA(cudaMemcpyAsync(dst, src_X, (size_t)r * b->cols_X * sizeof(float), cudaMemcpyHostToDevice, b->s_X));
    }
    CN_CUDA(cudaEventRecord(b->e_Xb[buf], b->s_X));
    b->rows_in[buf] = r;
    b->idx_in[buf] = idx;
    b->fill = (buf + 1) % b->nb;
    b->in_flight += 1;
    b->x_next_idx = batch_after(b, idx);
    return CN_OK;
}

extern "C" int cn_batch_copy_next_async(cn_batch *b)
{
    CN_REQUIRE(b, CN_ERR_ARG, "cn_batch_copy_next_async: null handle");
    // labels: always one batch ahead
    const int64_t idx = b->next_batch, r = rows_of_batch(b, idx);
    const float *src_y = b->h_y + (size_t)idx * b->batch * b->cols_y;
    if (!b->direct) {
        CN_CUDA(cudaEventSynchronize(b->e_y));   // the staging buffer is free once the last copy out of it has finished
        memcpy(b->p_y, src_y, (size_t)r * b->cols_y * sizeof(float));
        src_y = b->p_y;
    }
    CN_CUDA(cudaStreamWaitEvent(b->s_y, b->e_consumed, 0));
    CN_CUDA(cudaMemcpyAsync(b->dn_y, src_y, (size_t)r * b->cols_y * sizeof(float), cudaMemcpyHostToDevice, b->s_y));
    CN_CUDA(cudaEventRecord(b->e_y, b->s_y));
    // X: one copy in flight, or two with CN_BATCH_LOOKAHEAD (the first call then starts two)
    while (b->in_flight < b->depth) {
        int st = start_x_copy(b);
        if (st != CN_OK) return st;
    }
    b->next_rows = r;
    b->copy_pending = true;
    return CN_OK;
}

extern "C" int cn_batch_swap(cn_batch *b, void *stream, float **d_X, float **d_y, int64_t *batch_rows)
{
    CN_REQUIRE(b, CN_ERR_ARG, "cn_batch_swap: null handle");
    CN_REQUIRE(b->copy_pending && b->in_flight > 0, CN_ERR_ARG, "cn_batch_swap: no batch was copied (call cn_batch_copy_next_async first)");
    const int buf = b->ready;
    CN_REQUIRE(b->idx_in[buf] == b->next_batch && b->rows_in[buf] == b->next_rows, CN_ERR_ARG,
               "cn_batch_swap: the copied batch (%lld) is not the next one (%lld)", (long long)b->idx_in[buf], (long long)b->next_batch);
    cudaStream_t s = cn_stream(stream);
    CN_CUDA(cudaStreamWaitEvent(s, b->e_Xb[buf], 0));
    CN_CUDA(cudaStreamWaitEvent(s, b->e_y, 0));
    int st = CN_OK;
    if (!(b->flags & CN_BATCH_NO_COL_MAJOR)) st = cn_to_col_major(b->ctx, b->xb[buf], b->dc_X, b->next_rows, b->cols_X, stream);
    if (st == CN_OK) st = cn_to_col_major(b->ctx, b->dn_y, b->dc_y, b->next_rows, b->cols_y, stream);
    if (st != CN_OK) return st;
    // everything queued on the compute stream so far - the transposes above and the caller's work on the batch that was
    // current until now - precedes this event; the next copy waits for it before it overwrites a buffer
    CN_CUDA(cudaEventRecord(b->e_consumed, s));
    b->cur_rows = b->next_rows;
    if (b->flags & CN_BATCH_KEEP_ROW_MAJOR) b->cur_rm = b->xb[buf];   // stays valid until the next swap
    b->ready = (buf + 1) % b->nb;
    b->in_flight -= 1;
    b->copy_pending = false;
    b->next_batch = batch_after(b, b->next_batch);
    if (d_X) *d_X = b->dc_X;
    if (d_y) *d_y = b->dc_y;
    if (batch_rows) *batch_rows = b->cur_rows;
    return CN_OK;
}
