// Dense batch allocator: pinned staging + asynchronous host-to-device copies on side streams, ordered against
// the compute stream by events.  Takes over BatchAllocator's dense path (source/batchAllocator.cpp:101-251
// init, 253-274 buffers, 340-366 first batch, 399-425 staging memcpy, 759-777 + 843-847 async copies,
// 977-994 + 1036-1053 swap and wrap-around).
//
// Differences from the reference, none visible in the results: the swap does not block the host
// (cudaStreamWaitEvent instead of cudaStreamSynchronize), the device buffers are sized once for a full batch so
// the short last batch needs no cudaFree / cudaMalloc, and the next copy is ordered after the transposes that
// read the previous one.
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
    float *dn_X = nullptr, *dn_y = nullptr;   // device, next batch, row-major
    float *dc_X = nullptr, *dc_y = nullptr;   // device, current batch, column-major
    cudaStream_t s_X = nullptr, s_y = nullptr;
    cudaEvent_t e_X = nullptr, e_y = nullptr, e_consumed = nullptr;
};

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
    cudaFree(b->dn_X); cudaFree(b->dn_y); cudaFree(b->dc_X); cudaFree(b->dc_y);
    if (b->s_X) cudaStreamDestroy(b->s_X);
    if (b->s_y) cudaStreamDestroy(b->s_y);
    if (b->e_X) cudaEventDestroy(b->e_X);
    if (b->e_y) cudaEventDestroy(b->e_y);
    if (b->e_consumed) cudaEventDestroy(b->e_consumed);
    delete b;
    return CN_OK;
}

extern "C" int cn_batch_create(cn_context *ctx, const float *h_X, const float *h_y, int64_t rows, int64_t cols_X, int64_t cols_y,
                               int64_t batch_size, int skip_last_batch, cn_batch **out)
{
    CN_REQUIRE(ctx && h_X && h_y && out, CN_ERR_ARG, "cn_batch_create: null argument");
    CN_REQUIRE(rows > 0 && cols_X > 0 && cols_y > 0 && batch_size > 0, CN_ERR_ARG, "cn_batch_create: non-positive size");
    // "ERROR: Batch size must be smaller than the training set." (source/batchAllocator.cpp:135-139)
    CN_REQUIRE(batch_size <= rows, CN_ERR_SHAPE, "Batch size must be smaller than the training set.");
    *out = nullptr;
    cn_batch *b = new cn_batch();
    b->ctx = ctx;
    b->h_X = h_X; b->h_y = h_y;
    b->rows = rows; b->cols_X = cols_X; b->cols_y = cols_y; b->batch = batch_size;
    b->skip_last = skip_last_batch;
    b->total_batches = (rows + batch_size - 1) / batch_size;
    const size_t bx = (size_t)batch_size * cols_X * sizeof(float), by = (size_t)batch_size * cols_y * sizeof(float);
    cudaError_t e;
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
        (e = cudaMalloc(&b->dn_X, bx)) != cudaSuccess || (e = cudaMalloc(&b->dn_y, by)) != cudaSuccess ||
        (e = cudaMalloc(&b->dc_X, bx)) != cudaSuccess || (e = cudaMalloc(&b->dc_y, by)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&b->s_X, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&b->s_y, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&b->e_X, cudaEventDisableTiming)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&b->e_y, cudaEventDisableTiming)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&b->e_consumed, cudaEventDisableTiming)) != cudaSuccess) {
        cn_batch_destroy(b);
        return cn_cuda_fail(e, "cn_batch_create");
    }
    // first batch: staged, copied and transposed before returning, as BatchAllocator::init does
    b->next_batch = 0;
    int st = cn_batch_copy_next_async(b);
    float *dx, *dy;
    int64_t r;
    if (st == CN_OK) st = cn_batch_swap(b, nullptr, &dx, &dy, &r);
    if (st == CN_OK && cudaStreamSynchronize(nullptr) != cudaSuccess) st = cn_cuda_fail(cudaGetLastError(), "cn_batch_create");
    if (st != CN_OK) { cn_batch_destroy(b); return st; }
    *out = b;
    return CN_OK;
}

extern "C" int cn_batch_set_skip_last(cn_batch *b, int skip)
{
    CN_REQUIRE(b, CN_ERR_ARG, "cn_batch_set_skip_last: null handle");
    b->skip_last = skip ? 1 : 0;
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

extern "C" int cn_batch_copy_next_async(cn_batch *b)
{
    CN_REQUIRE(b, CN_ERR_ARG, "cn_batch_copy_next_async: null handle");
    const int64_t idx = b->next_batch, r = rows_of_batch(b, idx);
    const float *src_X = b->h_X + (size_t)idx * b->batch * b->cols_X, *src_y = b->h_y + (size_t)idx * b->batch * b->cols_y;
    if (!b->direct) {
        // the staging buffers are free once the previous copy out of them has finished
        if (b->copy_pending) {
            CN_CUDA(cudaEventSynchronize(b->e_X));
            CN_CUDA(cudaEventSynchronize(b->e_y));
        }
        memcpy(b->p_X, src_X, (size_t)r * b->cols_X * sizeof(float));
        memcpy(b->p_y, src_y, (size_t)r * b->cols_y * sizeof(float));
        src_X = b->p_X;
        src_y = b->p_y;
    }
    // do not overwrite the device "next" buffers while the last swap's transposes may still read them
    CN_CUDA(cudaStreamWaitEvent(b->s_X, b->e_consumed, 0));
    CN_CUDA(cudaStreamWaitEvent(b->s_y, b->e_consumed, 0));
    CN_CUDA(cudaMemcpyAsync(b->dn_X, src_X, (size_t)r * b->cols_X * sizeof(float), cudaMemcpyHostToDevice, b->s_X));
    CN_CUDA(cudaMemcpyAsync(b->dn_y, src_y, (size_t)r * b->cols_y * sizeof(float), cudaMemcpyHostToDevice, b->s_y));
    CN_CUDA(cudaEventRecord(b->e_X, b->s_X));
    CN_CUDA(cudaEventRecord(b->e_y, b->s_y));
    b->next_rows = r;
    b->copy_pending = true;
    return CN_OK;
}

extern "C" int cn_batch_swap(cn_batch *b, void *stream, float **d_X, float **d_y, int64_t *batch_rows)
{
    CN_REQUIRE(b, CN_ERR_ARG, "cn_batch_swap: null handle");
    CN_REQUIRE(b->copy_pending, CN_ERR_ARG, "cn_batch_swap: no batch was copied (call cn_batch_copy_next_async first)");
    cudaStream_t s = cn_stream(stream);
    CN_CUDA(cudaStreamWaitEvent(s, b->e_X, 0));
    CN_CUDA(cudaStreamWaitEvent(s, b->e_y, 0));
    int st = cn_to_col_major(b->ctx, b->dn_X, b->dc_X, b->next_rows, b->cols_X, stream);
    if (st == CN_OK) st = cn_to_col_major(b->ctx, b->dn_y, b->dc_y, b->next_rows, b->cols_y, stream);
    if (st != CN_OK) return st;
    CN_CUDA(cudaEventRecord(b->e_consumed, s));
    b->cur_rows = b->next_rows;
    // counter and wrap-around exactly as replace_current_batch_with_next (source/batchAllocator.cpp:1036-1052)
    b->next_batch += 1;
    if ((b->next_batch + 1) == b->total_batches && b->skip_last) b->next_batch = 0;
    if (b->next_batch >= b->total_batches) b->next_batch = 0;
    if (d_X) *d_X = b->dc_X;
    if (d_y) *d_y = b->dc_y;
    if (batch_rows) *batch_rows = b->cur_rows;
    return CN_OK;
}
