// Communicator and the sharded product.  One process per GPU; NCCL (over NVLink / NVSwitch) takes the place of
// the reference's CUDA-aware MPI: ClusterNet::init_MPI / shutdown_MPI (source/clusterNet.cpp:148-183,223-228)
// and the barrier + ring all-gather + hStackN tail of dotMPI (source/clusterNet.cpp:663-694).
//
// NCCL is loaded at run time (dlopen of libnccl.so.2) so that the library has no link-time dependency on it and
// single-GPU users never touch it; if the host program has already loaded an NCCL (torch does), that copy is used.
//
// Data placement of a column-sharded matrix is the reference's (source/clusterNet.cpp:515-516,926-931): rank r owns
// columns [r*floor(N/G), (r+1)*floor(N/G)), the last rank also the remainder.  In the column-major layout each
// shard is one contiguous block of the full matrix, so the local GEMM writes its slice in place and the all-gather
// needs no packing or concatenation kernel (the reference's slice_cols / hStackN copies disappear).
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>
#include <time.h>
#include <unistd.h>
#include <vector>
#include "cn_gemm.h"

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t *, int, const int *) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*Broadcast)(const void *, void *, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;   // optional: used by cn_comm_sync only
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
};

static NcclApi g_nccl;

static int nccl_load()
{
    if (g_nccl.handle) return CN_OK;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    CN_REQUIRE(h, CN_ERR_NCCL, "cannot load libnccl.so.2: %s", dlerror());
#define CN_SYM(field, name)                                                          \
    *(void **)(&g_nccl.field) = dlsym(h, name);                                      \
    CN_REQUIRE(g_nccl.field, CN_ERR_NCCL, "libnccl.so.2 has no symbol %s", name)
    CN_SYM(GetUniqueId, "ncclGetUniqueId");
    CN_SYM(CommInitRank, "ncclCommInitRank");
    CN_SYM(CommInitAll, "ncclCommInitAll");
    CN_SYM(CommDestroy, "ncclCommDestroy");
    CN_SYM(Broadcast, "ncclBroadcast");
    CN_SYM(AllGather, "ncclAllGather");
    CN_SYM(AllReduce, "ncclAllReduce");
    CN_SYM(GroupStart, "ncclGroupStart");
    CN_SYM(GroupEnd, "ncclGroupEnd");
    CN_SYM(GetErrorString, "ncclGetErrorString");
#undef CN_SYM
    *(void **)(&g_nccl.CommGetAsyncError) = dlsym(h, "ncclCommGetAsyncError");
    *(void **)(&g_nccl.CommAbort) = dlsym(h, "ncclCommAbort");
    g_nccl.handle = h;
    return CN_OK;
}

#define CN_NCCL(call)                                                                              \
    do {                                                                                           \
        ncclResult_t r__ = (call);                                                                 \
        if (r__ != ncclSuccess) {                                                                  \
            cn_set_error("NCCL error %d (%s) in %s", (int)r__, g_nccl.GetErrorString(r__), #call); \
            return CN_ERR_NCCL;                                                                    \
        }                                                                                          \
    } while (0)

// A buffer that exists with the same size on every rank and that every rank has mapped from every peer
// (cudaIpc handles exchanged once through the communicator).
struct cn_sym_buf {
    void *base = nullptr;
    size_t bytes = 0;
    std::vector<void *> peer;   // [nranks]; peer[rank] == base
};

struct cn_comm_state {
    ncclComm_t comm = nullptr;
    int rank = 0, nranks = 1;
    float *d_scales = nullptr;   // one codec scale per rank
    std::vector<cn_sym_buf> sym;
    // cross-GPU flags (a symmetric buffer of its own): slot 0 = "my copy may be written", slot 1 = "my stores are done";
    // entry [slot * nranks + r] on a GPU is written by rank r
    unsigned int *flags = nullptr;
    std::vector<unsigned int *> peer_flags;
    unsigned int **d_peer_flags = nullptr;   // device copy of peer_flags
    unsigned int epoch = 0;
    int next_flag_slot = 2;   // slots 0 and 1 frame the fused gather; the batch allocators reserve theirs from here
    // Pushed block exchange (cn_comm_push_area / cn_comm_push_blocks): one symmetric area of nranks blocks; every rank
    // writes its block into the same place of every peer's area.  The epoch lives in device memory so that a recorded
    // launch (CUDA graph) can be replayed.
    uint8_t *xchg = nullptr;
    size_t xchg_bytes = 0;
    void *xchg_peer[8] = {};
    int xchg_slot = -1;                  // two flag slots: "my area may be written", "my block has arrived"
    unsigned int *d_xchg_state = nullptr;   // [0] epoch of the last finished exchange, [1] ticket
    int push_exchange = 1;               // cn_comm_set_push_exchange
    bool aborted = false;   // cn_comm_sync gave up on a collective: only cn_comm_destroy is accepted from here on
    bool in_process = false;   // made by cn_comm_init_all: the peers are contexts of this process (no CUDA IPC between them)
};

// Refuses work on a communicator that cn_comm_sync has aborted; a context without communicator passes (single rank).
#define CN_COMM_ALIVE(ctx)                                                                                             \
    CN_REQUIRE(!((ctx)->comm && (ctx)->comm->aborted), CN_ERR_NCCL,                                                    \
               "the communicator was aborted after a failed or timed-out collective: call cn_comm_destroy, then cn_comm_init_rank again")

static void sym_release(cn_comm_state *c, cn_sym_buf &b)
{
    for (int r = 0; r < (int)b.peer.size(); ++r)
        if (r != c->rank && b.peer[r]) cudaIpcCloseMemHandle(b.peer[r]);
    cudaFree(b.base);
    b.base = nullptr;
}

void cn_comm_state_free(cn_context *ctx)
{
    if (!ctx->comm) return;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(ctx->device);   // several contexts may live in one process (cn_comm_init_all)
    cudaDeviceSynchronize();
    for (auto &b : ctx->comm->sym) sym_release(ctx->comm, b);
    cudaFree(ctx->comm->d_peer_flags);
    cudaFree(ctx->comm->d_xchg_state);
    if (ctx->comm->comm && !ctx->comm->aborted && g_nccl.CommDestroy) g_nccl.CommDestroy(ctx->comm->comm);
    cudaFree(ctx->comm->d_scales);
    delete ctx->comm;
    ctx->comm = nullptr;
    if (prev >= 0) cudaSetDevice(prev);
}

extern "C" int cn_comm_get_unique_id(void *id128)
{
    CN_REQUIRE(id128, CN_ERR_ARG, "cn_comm_get_unique_id: null buffer");
    int st = nccl_load();
    if (st != CN_OK) return st;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is expected to be 128 bytes");
    ncclUniqueId id;
    CN_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(id128, &id, sizeof(id));
    return CN_OK;
}

extern "C" int cn_comm_init_rank(cn_context *ctx, const void *id128, int rank, int nranks)
{
    CN_REQUIRE(ctx && id128, CN_ERR_ARG, "cn_comm_init_rank: null argument");
    CN_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, CN_ERR_ARG, "cn_comm_init_rank: rank %d of %d", rank, nranks);
    CN_REQUIRE(!ctx->comm, CN_ERR_ARG, "cn_comm_init_rank: communicator already initialised");
    int st = nccl_load();
    if (st != CN_OK) return st;
    CN_CUDA(cudaSetDevice(ctx->device));
    cn_comm_state *c = new cn_comm_state();
    c->rank = rank;
    c->nranks = nranks;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    ncclResult_t r = g_nccl.CommInitRank(&c->comm, nranks, id, rank);
    if (r != ncclSuccess) {
        cn_set_error("NCCL error %d (%s) in ncclCommInitRank", (int)r, g_nccl.GetErrorString(r));
        delete c;
        return CN_ERR_NCCL;
    }
    cudaError_t e = cudaMalloc(&c->d_scales, sizeof(float) * (size_t)nranks);
    if (e != cudaSuccess) {
        g_nccl.CommDestroy(c->comm);
        delete c;
        return cn_cuda_fail(e, "cn_comm_init_rank");
    }
    ctx->comm = c;
    return CN_OK;
}

// Single-process form (ncclCommInitAll): contexts of this process, one per device, become ranks 0 .. n-1 of one
// communicator.  Each rank is then driven by its own host thread, or one thread drives all of them and brackets the
// per-rank calls of one collective with cn_group_start / cn_group_end.
extern "C" int cn_comm_init_all(cn_context **ctxs, int n)
{
    CN_REQUIRE(ctxs && n >= 1 && n <= CN_MAX_PEERS + 1, CN_ERR_ARG, "cn_comm_init_all: 1 .. %d contexts", CN_MAX_PEERS + 1);
    std::vector<int> devs(n);
    for (int i = 0; i < n; ++i) {
        CN_REQUIRE(ctxs[i] && !ctxs[i]->comm, CN_ERR_ARG, "cn_comm_init_all: context %d is null or already has a communicator", i);
        devs[i] = ctxs[i]->device;
        for (int j = 0; j < i; ++j) CN_REQUIRE(devs[j] != devs[i], CN_ERR_ARG, "cn_comm_init_all: two contexts on device %d", devs[i]);
    }
    int st = nccl_load();
    if (st != CN_OK) return st;
    int prev = 0;
    CN_CUDA(cudaGetDevice(&prev));
    std::vector<ncclComm_t> comms(n, nullptr);
    ncclResult_t r = g_nccl.CommInitAll(comms.data(), n, devs.data());
    if (r != ncclSuccess) {
        cn_set_error("NCCL error %d (%s) in ncclCommInitAll", (int)r, g_nccl.GetErrorString(r));
        cudaSetDevice(prev);
        return CN_ERR_NCCL;
    }
    for (int i = 0; i < n; ++i) {
        cn_comm_state *c = new cn_comm_state();
        c->comm = comms[i];
        c->rank = i;
        c->nranks = n;
        c->in_process = true;
        cudaError_t e = cudaSetDevice(devs[i]);
        if (e == cudaSuccess) e = cudaMalloc(&c->d_scales, sizeof(float) * (size_t)n);
        if (e != cudaSuccess) {
            delete c;
            for (int j = 0; j < n; ++j) {
                if (j < i) cn_comm_state_free(ctxs[j]); else g_nccl.CommDestroy(comms[j]);
            }
            cudaSetDevice(prev);
            return cn_cuda_fail(e, "cn_comm_init_all");
        }
        ctxs[i]->comm = c;
    }
    CN_CUDA(cudaSetDevice(prev));
    return CN_OK;
}

extern "C" int cn_group_start(void)
{
    int st = nccl_load();
    if (st != CN_OK) return st;
    CN_NCCL(g_nccl.GroupStart());
    return CN_OK;
}

extern "C" int cn_group_end(void)
{
    int st = nccl_load();
    if (st != CN_OK) return st;
    CN_NCCL(g_nccl.GroupEnd());
    return CN_OK;
}

extern "C" int cn_context_make_current(const cn_context *ctx)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_context_make_current: null context");
    CN_CUDA(cudaSetDevice(ctx->device));
    return CN_OK;
}

extern "C" int cn_comm_destroy(cn_context *ctx)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_comm_destroy: null context");
    cn_comm_state_free(ctx);
    return CN_OK;
}

// Bounded host-side wait for the work queued on `stream`, for loops in which a peer may have left: polls the stream and
// the communicator's asynchronous error state; on an NCCL error, or when timeout_ms passes with the stream still busy,
// the communicator is aborted (ncclCommAbort ends NCCL kernels that wait for a peer), the status says which, and every
// later collective call on this context fails until the communicator is destroyed and created again.  The reference
// blocks forever in MPI_Barrier / MPI_Wait in that situation (source/clusterNet.cpp:663-690).
extern "C" int cn_comm_sync(cn_context *ctx, void *stream, int timeout_ms)
{
    CN_REQUIRE(ctx && timeout_ms > 0, CN_ERR_ARG, "cn_comm_sync: bad argument");
    cudaStream_t s = cn_stream(stream);
    cn_comm_state *c = ctx->comm;
    timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (;;) {
        cudaError_t q = cudaStreamQuery(s);
        if (q == cudaSuccess) return CN_OK;
        if (q != cudaErrorNotReady) return cn_cuda_fail(q, "cn_comm_sync");
        ncclResult_t async = ncclSuccess;
        if (c && c->comm && !c->aborted && g_nccl.CommGetAsyncError) {
            if (g_nccl.CommGetAsyncError(c->comm, &async) != ncclSuccess) async = ncclSystemError;
            if (async == ncclInProgress) async = ncclSuccess;
        }
        timespec t1;
        clock_gettime(CLOCK_MONOTONIC, &t1);
        const double ms = (t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) * 1e-6;
        const bool timed_out = ms > (double)timeout_ms;
        if (async != ncclSuccess || timed_out) {
            bool did_abort = false;
            if (c && c->comm && !c->aborted) {
                if (g_nccl.CommAbort) g_nccl.CommAbort(c->comm);
                c->aborted = true;
                did_abort = true;
            }
            if (async != ncclSuccess) {
                cn_set_error("cn_comm_sync: NCCL reported asynchronous error %d (%s)%s", (int)async, g_nccl.GetErrorString(async),
                             did_abort ? "; communicator aborted" : "");
                return CN_ERR_NCCL;
            }
            cn_set_error("cn_comm_sync: stream still busy after %d ms%s", timeout_ms, did_abort ? "; communicator aborted" : "");
            return CN_ERR_TIMEOUT;
        }
        usleep(50);
    }
}

extern "C" int cn_comm_rank(const cn_context *ctx) { return (ctx && ctx->comm) ? ctx->comm->rank : 0; }
extern "C" int cn_comm_size(const cn_context *ctx) { return (ctx && ctx->comm) ? ctx->comm->nranks : 1; }

extern "C" int cn_shard_cols(int64_t n_total, int rank, int nranks, int64_t *col_start, int64_t *col_count)
{
    CN_REQUIRE(n_total >= 0 && nranks >= 1 && rank >= 0 && rank < nranks, CN_ERR_ARG, "cn_shard_cols: bad argument");
    const int64_t split = n_total / nranks;
    if (col_start) *col_start = split * rank;
    if (col_count) *col_count = (rank == nranks - 1) ? n_total - split * (nranks - 1) : split;
    return CN_OK;
}

extern "C" int cn_bcast_f32(cn_context *ctx, float *d_buf, int64_t n, int root, void *stream)
{
    CN_REQUIRE(ctx && n >= 0 && (n == 0 || d_buf), CN_ERR_ARG, "cn_bcast_f32: bad argument");
    if (!ctx->comm || ctx->comm->nranks == 1 || n == 0) return CN_OK;
    CN_COMM_ALIVE(ctx);
    CN_REQUIRE(root >= 0 && root < ctx->comm->nranks, CN_ERR_ARG, "cn_bcast_f32: root %d", root);
    CN_NCCL(g_nccl.Broadcast(d_buf, d_buf, (size_t)n, ncclFloat, root, ctx->comm->comm, cn_stream(stream)));
    return CN_OK;
}

// All-gather of contiguous per-rank blocks of `elem_size`-byte elements; blocks are equal except possibly the last.
static int allgather_blocks(cn_context *ctx, void *base, int64_t M, int64_t n_total, ncclDataType_t dt, size_t elem_size, cudaStream_t s)
{
    cn_comm_state *c = ctx->comm;
    if (!c || c->nranks == 1) return CN_OK;
    CN_COMM_ALIVE(ctx);
    const int G = c->nranks;
    const int64_t split = n_total / G;
    if (n_total % G == 0) {
        const size_t count = (size_t)M * split;
        if (count == 0) return CN_OK;
        CN_NCCL(g_nccl.AllGather((const uint8_t *)base + (size_t)c->rank * count * elem_size, base, count, dt, c->comm, s));
        return CN_OK;
    }
    // uneven shards: one broadcast per owner, fused into a single NCCL group
    CN_NCCL(g_nccl.GroupStart());
    for (int r = 0; r < G; ++r) {
        int64_t start, cnt;
        cn_shard_cols(n_total, r, G, &start, &cnt);
        if (cnt == 0) continue;
        void *blk = (uint8_t *)base + (size_t)M * start * elem_size;
        ncclResult_t res = g_nccl.Broadcast(blk, blk, (size_t)M * cnt, dt, r, c->comm, s);
        if (res != ncclSuccess) {
            g_nccl.GroupEnd();
            cn_set_error("NCCL error %d (%s) in ncclBroadcast", (int)res, g_nccl.GetErrorString(res));
            return CN_ERR_NCCL;
        }
    }
    CN_NCCL(g_nccl.GroupEnd());
    return CN_OK;
}

extern "C" int cn_allgather_cols_f32(cn_context *ctx, float *d_C, int64_t M, int64_t n_total, void *stream)
{
    CN_REQUIRE(ctx && M >= 0 && n_total >= 0 && (M * n_total == 0 || d_C), CN_ERR_ARG, "cn_allgather_cols_f32: bad argument");
    return allgather_blocks(ctx, d_C, M, n_total, ncclFloat, sizeof(float), cn_stream(stream));
}

extern "C" int cn_allgather_cols_u8(cn_context *ctx, uint8_t *d_codes, int64_t M, int64_t n_total, void *stream)
{
    CN_REQUIRE(ctx && M >= 0 && n_total >= 0 && (M * n_total == 0 || d_codes), CN_ERR_ARG, "cn_allgather_cols_u8: bad argument");
    return allgather_blocks(ctx, d_codes, M, n_total, ncclUint8, 1, cn_stream(stream));
}

extern "C" int cn_allgather_scalar_f32(cn_context *ctx, float *d_vals, void *stream)
{
    CN_REQUIRE(ctx && d_vals, CN_ERR_ARG, "cn_allgather_scalar_f32: bad argument");
    if (!ctx->comm || ctx->comm->nranks == 1) return CN_OK;
    CN_COMM_ALIVE(ctx);
    CN_NCCL(g_nccl.AllGather(d_vals + ctx->comm->rank, d_vals, 1, ncclFloat, ctx->comm->comm, cn_stream(stream)));
    return CN_OK;
}

extern "C" int cn_allreduce_sum_f32(cn_context *ctx, float *d_buf, int64_t n, void *stream)
{
    CN_REQUIRE(ctx && n >= 0 && (n == 0 || d_buf), CN_ERR_ARG, "cn_allreduce_sum_f32: bad argument");
    if (!ctx->comm || ctx->comm->nranks == 1 || n == 0) return CN_OK;
    CN_COMM_ALIVE(ctx);
    CN_NCCL(g_nccl.AllReduce(d_buf, d_buf, (size_t)n, ncclFloat, ncclSum, ctx->comm->comm, cn_stream(stream)));
    return CN_OK;
}

// ------------------------------------------------------------------------------------------------
// Symmetric buffers and the flag barrier used by the fused GEMM -> all-gather path.
// ------------------------------------------------------------------------------------------------
static int sym_alloc_impl(cn_context *ctx, size_t bytes, cn_sym_buf *out)
{
    cn_comm_state *c = ctx->comm;
    CN_COMM_ALIVE(ctx);
    const int G = c->nranks;
    cn_sym_buf b;
    b.bytes = bytes;
    CN_CUDA(cudaMalloc(&b.base, bytes ? bytes : 256));
    b.peer.assign(G, nullptr);
    b.peer[c->rank] = b.base;
    // exchange the IPC handles: every rank contributes 64 bytes
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "cudaIpcMemHandle_t is expected to be 64 bytes");
    cudaIpcMemHandle_t mine;
    unsigned char *d_h = nullptr;
    cudaError_t e = cudaIpcGetMemHandle(&mine, b.base);
    if (e == cudaSuccess) e = cudaMalloc(&d_h, 64 * (size_t)G);
    if (e == cudaSuccess) e = cudaMemcpy(d_h + 64 * c->rank, &mine, 64, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        cudaFree(d_h);
        cudaFree(b.base);
        return cn_cuda_fail(e, "cn_sym_alloc");
    }
    ncclResult_t r = g_nccl.AllGather(d_h + 64 * c->rank, d_h, 64, ncclUint8, c->comm, nullptr);
    std::vector<cudaIpcMemHandle_t> all(G);
    e = cudaMemcpy(all.data(), d_h, 64 * (size_t)G, cudaMemcpyDeviceToHost);   // synchronises the default stream
    cudaFree(d_h);
    if (r != ncclSuccess || e != cudaSuccess) {
        cudaFree(b.base);
        cn_set_error("cn_sym_alloc: exchange of the memory handles failed (nccl %d, cuda %d)", (int)r, (int)e);
        return CN_ERR_NCCL;
    }
    for (int p = 0; p < G; ++p) {
        if (p == c->rank) continue;
        e = cudaIpcOpenMemHandle(&b.peer[p], all[p], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            sym_release(c, b);
            return cn_cuda_fail(e, "cudaIpcOpenMemHandle");
        }
    }
    *out = b;
    return CN_OK;
}

extern "C" int cn_sym_alloc(cn_context *ctx, size_t bytes, void **ptr)
{
    CN_REQUIRE(ctx && ptr, CN_ERR_ARG, "cn_sym_alloc: null argument");
    *ptr = nullptr;
    CN_CUDA(cudaSetDevice(ctx->device));
    if (!ctx->comm || ctx->comm->nranks == 1) {   // nothing to map: an ordinary allocation
        CN_CUDA(cudaMalloc(ptr, bytes ? bytes : 256));
        return CN_OK;
    }
    cn_comm_state *c = ctx->comm;
    CN_REQUIRE(c->nranks - 1 <= CN_MAX_PEERS, CN_ERR_UNSUPPORTED, "cn_sym_alloc: at most %d ranks", CN_MAX_PEERS + 1);
    CN_REQUIRE(!c->in_process, CN_ERR_UNSUPPORTED,
               "cn_sym_alloc: symmetric buffers are CUDA-IPC mappings between processes; a communicator made by cn_comm_init_all gathers with NCCL "
               "(pass an ordinary buffer)");
    int st;
    if (!c->flags) {   // first use: the flag words, zeroed, and the device table of their peer addresses
        // Everything is built in locals and published (c->flags, c->d_peer_flags) only after every step, the closing
        // barrier included, has succeeded: a failed set-up leaves the context without flags, so the fused path stays off.
        cn_sym_buf f;
        if ((st = sym_alloc_impl(ctx, 4096, &f)) != CN_OK) return st;
        unsigned int **d_tab = nullptr;
        float *d_tmp = nullptr;
        std::vector<unsigned int *> tab;
        for (void *q : f.peer) tab.push_back((unsigned int *)q);
        cudaError_t e = cudaMemset(f.base, 0, 4096);
        if (e == cudaSuccess) e = cudaMalloc(&d_tab, sizeof(unsigned int *) * c->nranks);
        if (e == cudaSuccess) e = cudaMemcpy(d_tab, tab.data(), sizeof(unsigned int *) * c->nranks, cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMalloc(&d_tmp, 4);
        if (e == cudaSuccess) e = cudaMemset(d_tmp, 0, 4);
        // nobody may signal into flags that a slower rank has not zeroed yet
        ncclResult_t r = e == cudaSuccess ? g_nccl.AllReduce(d_tmp, d_tmp, 1, ncclFloat, ncclSum, c->comm, nullptr) : ncclSuccess;
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        cudaFree(d_tmp);
        if (e != cudaSuccess || r != ncclSuccess) {
            cudaFree(d_tab);
            sym_release(c, f);
            cudaGetLastError();
            cn_set_error("cn_sym_alloc: set-up of the cross-GPU flags failed (cuda %d, nccl %d)", (int)e, (int)r);
            return e != cudaSuccess ? CN_ERR_CUDA : CN_ERR_NCCL;
        }
        c->sym.push_back(f);
        c->peer_flags = tab;
        c->d_peer_flags = d_tab;
        c->flags = (unsigned int *)f.base;
    }
    cn_sym_buf b;
    if ((st = sym_alloc_impl(ctx, bytes, &b)) != CN_OK) return st;
    c->sym.push_back(b);
    *ptr = b.base;
    return CN_OK;
}

extern "C" int cn_sym_free(cn_context *ctx, void *ptr)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_sym_free: null context");
    if (!ptr) return CN_OK;
    if (ctx->comm) {
        auto &v = ctx->comm->sym;
        for (size_t i = 0; i < v.size(); ++i) {
            if (v[i].base == ptr) {
                CN_CUDA(cudaDeviceSynchronize());
                sym_release(ctx->comm, v[i]);
                v.erase(v.begin() + i);
                return CN_OK;
            }
        }
    }
    CN_CUDA(cudaFree(ptr));
    return CN_OK;
}

// Raise the flag, then wait (bounded) until every peer has raised its own for this epoch.
__global__ void cn_flag_barrier_kernel(unsigned int *const *peer_flags, const unsigned int *local_flags, int nranks, int my_rank,
                                       int slot, unsigned int epoch, unsigned int *status)
{
    const int r = threadIdx.x;
    if (r < nranks && r != my_rank) {
        __threadfence_system();
        volatile unsigned int *f = peer_flags[r] + slot * nranks + my_rank;
        *f = epoch;
        const volatile unsigned int *mine = local_flags + slot * nranks + r;
        const long long t0 = clock64();
        while ((int)(*mine - epoch) < 0) {
            if (clock64() - t0 > 6000000000LL) { atomicMax(status, 10u); break; }
            __nanosleep(200);
        }
        __threadfence_system();
    }
}

// Is [p, p + bytes) inside a symmetric buffer?  Fills the peer addresses of p.
static bool sym_lookup(cn_comm_state *c, const void *p, size_t bytes, float **peers_out)
{
    for (auto &b : c->sym) {
        const char *lo = (const char *)b.base;
        if ((const char *)p >= lo && (const char *)p + bytes <= lo + b.bytes) {
            const size_t off = (const char *)p - lo;
            int k = 0;
            for (int r = 0; r < c->nranks; ++r)
                if (r != c->rank) peers_out[k++] = (float *)((char *)b.peer[r] + off);
            return true;
        }
    }
    return false;
}

// transA = 0: A stored M x K (leading dimension lda >= M); transA = 1: A stored K x M (lda >= K), the product uses its
// transpose (TdotMPI, source/clusterNet.cpp:510).
static int dotmpi_impl(cn_context *ctx, int transA, int64_t M, int64_t K, int64_t n_total, const float *d_A, int64_t lda,
                       const float *d_Wshard, float *d_C, const cn_epilogue *epi, int mode, int exchange, void *stream)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_dotmpi_f32: null context");
    CN_REQUIRE(M >= 0 && K >= 0 && n_total >= 0, CN_ERR_SHAPE, "cn_dotmpi_f32: negative dimension");
    CN_REQUIRE(exchange == 0 || exchange == 1, CN_ERR_ARG, "cn_dotmpi_f32: exchange must be 0 (fp32) or 1 (8-bit)");
    CN_REQUIRE(!epi || epi->maxout_level <= 1, CN_ERR_UNSUPPORTED, "cn_dotmpi_f32: maxout is not available on the sharded product");
    CN_COMM_ALIVE(ctx);
    const int G = ctx->comm ? ctx->comm->nranks : 1, rank = ctx->comm ? ctx->comm->rank : 0;
    int64_t start, cnt;
    cn_shard_cols(n_total, rank, G, &start, &cnt);
    // local product straight into this rank's window of the full C
    cn_epilogue local;
    local.bias = (epi && epi->bias) ? epi->bias + start : nullptr;
    local.activation = epi ? epi->activation : CN_ACT_LINEAR;
    local.maxout_level = 0;
    local.argmax_out = nullptr;
    float *slice = d_C + (size_t)M * start;
    int st;
    // Fused form: when C lives in a symmetric buffer, the GEMM's epilogue stores every finished tile into all peers'
    // copies of C as well (bulk copies over NVLink), framed by two flag exchanges: "my copy may be written", raised by
    // the GEMM kernel when it starts, and "my stores are complete", a one-block kernel after it.  No gather kernel runs.
    cn_peer_out po;
    // Whether to push is decided from values that are equal on every rank (shapes, mode), so that all ranks take the
    // same branch: the narrowest shard must still be a shape the tensor-core kernel takes.
    const bool shape_ok = mode != CN_GEMM_FP32_SIMT && (n_total / G) >= 16 && K >= 32 && (K & 3) == 0 && M >= 1;
    if (G > 1 && exchange == 0 && shape_ok && ctx->comm->flags && ctx->comm->d_peer_flags &&
        sym_lookup(ctx->comm, d_C, (size_t)M * n_total * sizeof(float), po.C)) {
        cn_comm_state *c = ctx->comm;
        cudaStream_t s = cn_stream(stream);
        const unsigned int epoch = ++c->epoch;
        for (int i = 0; i < G - 1; ++i) po.C[i] += (size_t)M * start;   // the window this rank writes
        po.npeers = G - 1;
        po.ready = c->flags;   // slot 0
        po.nranks = G;
        po.my_rank = rank;
        po.epoch = epoch;
        po.peer_flags = c->d_peer_flags;   // the GEMM kernel raises this rank's "ready" flag itself when it starts
        bool pushed = false;
        st = cn_gemm_dispatch(ctx, transA, 0, M, cnt, K, d_A, lda, d_Wshard, K, slice, M, &local, mode, stream, &po, &pushed);
        if (st != CN_OK) return st;
        // a rank whose operands the tensor-core kernel refused (a misaligned shard pointer) cannot fall back on its own:
        // the peers are already past the point of calling a collective
        CN_REQUIRE(pushed, CN_ERR_UNSUPPORTED, "cn_dotmpi_f32: this rank's shard cannot take the fused path (16-byte alignment of W)");
        cn_flag_barrier_kernel<<<1, 32, 0, s>>>(c->d_peer_flags, c->flags, G, rank, 1, epoch, ctx->gemm->d_status);
        CN_CUDA(cudaGetLastError());
        cn_count_launch();
        return CN_OK;
    }
    st = cn_gemm_f32(ctx, transA, 0, M, cnt, K, d_A, lda, d_Wshard, K, slice, M, &local, mode, stream);
    if (st != CN_OK || G == 1) return st;
    if (exchange == 0) return cn_allgather_cols_f32(ctx, d_C, M, n_total, stream);

    // 8-bit exchange: scale = absmax of the own slice, codes gathered next to the per-rank scales, peers' slices
    // decoded on arrival; the own slice keeps its fp32 values (as the reference's cache[MYRANK] does).
    void *buf = nullptr;
    st = cn_gemm_scratch(ctx, CN_GEMM_SLOT_EXCHANGE, (size_t)M * n_total, &buf);
    if (st != CN_OK) return st;
    uint8_t *codes = (uint8_t *)buf;
    float *scales = ctx->comm->d_scales;
    if ((st = cn_absmax_compress_8bit(ctx, slice, M * cnt, scales + rank, codes + (size_t)M * start, stream)) != CN_OK) return st;
    if ((st = cn_allgather_scalar_f32(ctx, scales, stream)) != CN_OK) return st;
    if ((st = cn_allgather_cols_u8(ctx, codes, M, n_total, stream)) != CN_OK) return st;
    for (int r = 0; r < G; ++r) {
        if (r == rank) continue;
        int64_t s0, c0;
        cn_shard_cols(n_total, r, G, &s0, &c0);
        if ((st = cn_decompress_8bit_dp(ctx, codes + (size_t)M * s0, scales + r, M * c0, d_C + (size_t)M * s0, stream)) != CN_OK) return st;
    }
    return CN_OK;
}

bool cn_comm_sym_peers(cn_context *ctx, const void *local, size_t bytes, void **peers_out)
{
    cn_comm_state *c = ctx->comm;
    if (!c) return false;
    for (auto &b : c->sym) {
        const char *lo = (const char *)b.base;
        if ((const char *)local >= lo && (const char *)local + bytes <= lo + b.bytes) {
            const size_t off = (const char *)local - lo;
            for (int r = 0; r < c->nranks; ++r) peers_out[r] = (char *)b.peer[r] + off;
            return true;
        }
    }
    return false;
}

int cn_comm_flag_slots(cn_context *ctx, int count, int *first_slot)
{
    cn_comm_state *c = ctx->comm;
    CN_REQUIRE(c && c->flags, CN_ERR_ARG, "flag slots need a communicator with symmetric buffers (cn_sym_alloc)");
    CN_REQUIRE((c->next_flag_slot + count) * c->nranks <= 1024, CN_ERR_UNSUPPORTED, "out of cross-GPU flag slots");
    *first_slot = c->next_flag_slot;
    c->next_flag_slot += count;
    return CN_OK;
}

int cn_comm_flag_barrier(cn_context *ctx, int slot, unsigned int epoch, cudaStream_t s)
{
    cn_comm_state *c = ctx->comm;
    CN_REQUIRE(c && c->flags && c->d_peer_flags, CN_ERR_ARG, "flag barrier needs a communicator with symmetric buffers");
    CN_COMM_ALIVE(ctx);
    unsigned int *d_status = nullptr;
    int st = cn_status_block(ctx, &d_status);
    if (st != CN_OK) return st;
    cn_flag_barrier_kernel<<<1, 32, 0, s>>>(c->d_peer_flags, c->flags, c->nranks, c->rank, slot, epoch, d_status);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

extern "C" int cn_dotmpi_f32(cn_context *ctx, int64_t M, int64_t K, int64_t n_total, const float *d_A, const float *d_Wshard,
                             float *d_C, const cn_epilogue *epi, int mode, int exchange, void *stream)
{
    return dotmpi_impl(ctx, 0, M, K, n_total, d_A, M, d_Wshard, d_C, epi, mode, exchange, stream);
}

extern "C" int cn_tdotmpi_f32(cn_context *ctx, int64_t M, int64_t K, int64_t n_total, const float *d_At, int64_t lda,
                              const float *d_Wshard, float *d_C, const cn_epilogue *epi, int mode, int exchange, void *stream)
{
    CN_REQUIRE(lda >= K, CN_ERR_SHAPE, "cn_tdotmpi_f32: leading dimension smaller than K");
    return dotmpi_impl(ctx, 1, M, K, n_total, d_At, lda, d_Wshard, d_C, epi, mode, exchange, stream);
}

extern "C" int cn_dottmpi_f32(cn_context *ctx, int64_t M, int64_t n_total, int64_t R, const float *d_A, const float *d_Bshard,
                              float *d_out, int mode, void *stream)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_dottmpi_f32: null context");
    CN_REQUIRE(M >= 0 && n_total >= 0 && R >= 0, CN_ERR_SHAPE, "cn_dottmpi_f32: negative dimension");
    const int G = ctx->comm ? ctx->comm->nranks : 1, rank = ctx->comm ? ctx->comm->rank : 0;
    int64_t start, cnt;
    cn_shard_cols(n_total, rank, G, &start, &cnt);
    // A1 = columns [start, start + cnt) of A: a contiguous block in column-major, no slice copy
    const float *A1 = d_A + (size_t)M * start;
    int st;
    if (cnt > 0) {
        st = cn_gemm_f32(ctx, 0, 1, M, R, cnt, A1, M, d_Bshard, R, d_out, M, nullptr, mode, stream);
    } else {
        st = cn_fill_f32(ctx, d_out, M * R, 0.0f, stream);
    }
    if (st != CN_OK || G == 1) return st;
    return cn_allreduce_sum_f32(ctx, d_out, M * R, stream);
}

extern "C" int cn_dot_sharded_out_f32(cn_context *ctx, int transA, int64_t M, int64_t K, int64_t n_total, const float *d_A,
                                      const float *d_B, float *d_out_shard, int mode, void *stream)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_dot_sharded_out_f32: null context");
    CN_REQUIRE(M >= 0 && K >= 0 && n_total >= 0, CN_ERR_SHAPE, "cn_dot_sharded_out_f32: negative dimension");
    const int G = ctx->comm ? ctx->comm->nranks : 1, rank = ctx->comm ? ctx->comm->rank : 0;
    int64_t start, cnt;
    cn_shard_cols(n_total, rank, G, &start, &cnt);
    if (cnt == 0) return CN_OK;
    const float *B1 = d_B + (size_t)K * start;   // columns of B owned by this rank
    return cn_gemm_f32(ctx, transA, 0, M, cnt, K, d_A, transA ? K : M, B1, K, d_out_shard, M, nullptr, mode, stream);
}

// ---- helpers for the gradient exchange in cn_train.cu
int cn_comm_info(cn_context *ctx, int *rank, int *nranks, float **d_scales)
{
    *rank = ctx->comm ? ctx->comm->rank : 0;
    *nranks = ctx->comm ? ctx->comm->nranks : 1;
    *d_scales = ctx->comm ? ctx->comm->d_scales : nullptr;
    return CN_OK;
}

// blocks: nranks blocks of block_bytes bytes, block [rank] filled
int cn_comm_gather_blocks(cn_context *ctx, uint8_t *d_blocks, size_t block_bytes, void *stream)
{
    cn_comm_state *c = ctx->comm;
    if (!c || c->nranks == 1) return CN_OK;
    CN_COMM_ALIVE(ctx);
    CN_NCCL(g_nccl.AllGather(d_blocks + (size_t)c->rank * block_bytes, d_blocks, block_bytes, ncclUint8, c->comm, cn_stream(stream)));
    return CN_OK;
}

// ---- pushed block exchange: an all-gather of one block per rank without a library collective
//
// Every rank holds an area of nranks blocks in symmetric memory.  One kernel per exchange: (1) tell the peers "my area
// may be written" (everything this rank queued before, the decode of the last exchange included, has finished) and wait
// for theirs; (2) copy the own block to the same place in every peer's area with 16-byte stores over NVLink; (3) the CTA
// that finishes last tells the peers "my block has arrived" and waits for theirs.  One NVLink hop instead of the nranks-1
// steps of a ring, and no second launch.  Every wait is clock-bounded (status 10, reported by cn_gemm_check_status as
// CN_ERR_TIMEOUT); a rank whose first wait ran out does not write into its peers.  The epoch is read from and advanced in
// device memory, so the launch has the same arguments every time.
struct XchgPeers {
    uint8_t *dst[8];
    int ndst;
};

__device__ __forceinline__ bool xchg_wait_flags(const unsigned int *local_flags, int slot, int nranks, int my_rank, unsigned int epoch,
                                                unsigned int *status)
{
    // threads 0..nranks-1 each watch one peer's flag
    bool ok = true;
    const int r = threadIdx.x;
    if (r < nranks && r != my_rank) {
        const volatile unsigned int *f = local_flags + slot * nranks + r;
        const long long t0 = clock64();
        while ((int)(*f - epoch) < 0) {
            if (clock64() - t0 > 6000000000LL) { atomicMax(status, 10u); ok = false; break; }
            __nanosleep(100);
        }
        __threadfence_system();
    }
    return __syncthreads_and(ok);
}

__global__ void __launch_bounds__(512)
cn_push_exchange_kernel(const uint8_t *__restrict__ src, size_t nbytes, const XchgPeers pp, unsigned int *const *peer_flags,
                        const unsigned int *local_flags, int nranks, int my_rank, int slot, unsigned int *state, unsigned int *status)
{
    __shared__ int s_last;
    const unsigned int epoch = *reinterpret_cast<volatile unsigned int *>(state) + 1u;   // advanced by the last CTA, after every CTA has read it
    const int r = threadIdx.x;
    if (blockIdx.x == 0 && r < nranks && r != my_rank) {
        __threadfence_system();
        *reinterpret_cast<volatile unsigned int *>(peer_flags[r] + slot * nranks + my_rank) = epoch;
    }
    const bool may_write = xchg_wait_flags(local_flags, slot, nranks, my_rank, epoch, status);
    if (may_write) {
        const size_t n16 = nbytes >> 4, stride = (size_t)gridDim.x * blockDim.x;
        const uint4 *s16 = reinterpret_cast<const uint4 *>(src);
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
            const uint4 v = s16[i];
#pragma unroll 1
            for (int d = 0; d < pp.ndst; ++d) reinterpret_cast<uint4 *>(pp.dst[d])[i] = v;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(state + 1, 1u) == gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (!s_last) return;
    __threadfence_system();
    if (may_write && r < nranks && r != my_rank)
        *reinterpret_cast<volatile unsigned int *>(peer_flags[r] + (slot + 1) * nranks + my_rank) = epoch;
    if (may_write) xchg_wait_flags(local_flags, slot + 1, nranks, my_rank, epoch, status);
    __syncthreads();
    if (threadIdx.x == 0) {
        state[1] = 0u;
        state[0] = epoch;
        __threadfence();
    }
}

extern "C" int cn_comm_set_push_exchange(cn_context *ctx, int on)
{
    CN_REQUIRE(ctx && ctx->comm, CN_ERR_ARG, "cn_comm_set_push_exchange: no communicator");
    ctx->comm->push_exchange = on ? 1 : 0;
    return CN_OK;
}

// An area of nranks blocks of block_bytes (a multiple of 16) in symmetric memory, or *blocks = nullptr when this
// communicator cannot push (one rank, all ranks in one process, switched off).  Collective: every rank calls it with the
// same size at the same point; the area grows (rarely) by a collective reallocation.
int cn_comm_push_area(cn_context *ctx, size_t block_bytes, void *stream, uint8_t **blocks)
{
    *blocks = nullptr;
    cn_comm_state *c = ctx->comm;
    if (!c || c->nranks == 1 || c->in_process || !c->push_exchange || c->nranks - 1 > CN_MAX_PEERS || (block_bytes & 15)) return CN_OK;
    CN_COMM_ALIVE(ctx);
    const size_t need = block_bytes * c->nranks;
    if (need > c->xchg_bytes) {
        // growing allocates and synchronises, which a stream that is being recorded cannot do: gather with the library
        // then (every rank sees the same sizes, so every rank decides the same)
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(cn_stream(stream), &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
            cudaGetLastError();
            return CN_OK;
        }
        int st;
        if (c->xchg) {
            if ((st = cn_sym_free(ctx, c->xchg)) != CN_OK) return st;
            c->xchg = nullptr;
            c->xchg_bytes = 0;
        }
        size_t bytes = need + need / 4;                    // head room, so that slightly larger tensors do not reallocate
        bytes = (bytes + 65535) & ~(size_t)65535;
        void *p = nullptr;
        if ((st = cn_sym_alloc(ctx, bytes, &p)) != CN_OK) return st;
        void *peers[8] = {};
        if (!cn_comm_sym_peers(ctx, p, bytes, peers)) {
            cn_set_error("cn_comm_push_area: symmetric buffer not found");
            return CN_ERR_CUDA;
        }
        if (c->xchg_slot < 0 && (st = cn_comm_flag_slots(ctx, 2, &c->xchg_slot)) != CN_OK) return st;
        if (!c->d_xchg_state) {
            CN_CUDA(cudaMalloc(&c->d_xchg_state, 256));
            CN_CUDA(cudaMemset(c->d_xchg_state, 0, 256));
        }
        for (int r = 0; r < c->nranks; ++r) c->xchg_peer[r] = peers[r];
        c->xchg = (uint8_t *)p;
        c->xchg_bytes = bytes;
    }
    *blocks = c->xchg;
    return CN_OK;
}

int cn_comm_push_params(cn_context *ctx, size_t block_bytes, size_t scale_offset, cn_codec_push *out)
{
    cn_comm_state *c = ctx->comm;
    CN_REQUIRE(c && c->xchg && block_bytes * c->nranks <= c->xchg_bytes && c->xchg_slot >= 0 && c->d_xchg_state && c->d_peer_flags, CN_ERR_ARG,
               "cn_comm_push_params: no exchange area of this size (cn_comm_push_area first)");
    CN_COMM_ALIVE(ctx);
    const size_t off = (size_t)c->rank * block_bytes;
    out->ndst = 0;
    for (int p = 1; p < c->nranks; ++p) {   // staggered by rank
        uint8_t *base = (uint8_t *)c->xchg_peer[(c->rank + p) % c->nranks] + off;
        out->codes_dst[out->ndst] = base;
        out->scale_dst[out->ndst] = reinterpret_cast<float *>(base + scale_offset);
        out->ndst += 1;
    }
    out->peer_flags = c->d_peer_flags;
    out->local_flags = c->flags;
    out->nranks = c->nranks;
    out->my_rank = c->rank;
    out->slot = c->xchg_slot;
    out->state = c->d_xchg_state;
    return CN_OK;
}

// blocks: the area cn_comm_push_area returned for this block size, block [rank] filled; on return (in stream order) every
// block is filled.
int cn_comm_push_blocks(cn_context *ctx, uint8_t *blocks, size_t block_bytes, void *stream)
{
    cn_comm_state *c = ctx->comm;
    CN_REQUIRE(c && blocks && blocks == c->xchg && block_bytes * c->nranks <= c->xchg_bytes && !(block_bytes & 15), CN_ERR_ARG,
               "cn_comm_push_blocks: not the area of cn_comm_push_area");
    CN_COMM_ALIVE(ctx);
    unsigned int *d_status = nullptr;
    int st = cn_status_block(ctx, &d_status);
    if (st != CN_OK) return st;
    XchgPeers pp;
    pp.ndst = 0;
    const size_t off = (size_t)c->rank * block_bytes;
    for (int p = 1; p < c->nranks; ++p) pp.dst[pp.ndst++] = (uint8_t *)c->xchg_peer[(c->rank + p) % c->nranks] + off;   // staggered by rank
    const size_t n16 = block_bytes >> 4;
    int grid = (int)((n16 + 4 * 512 - 1) / (4 * 512));   // four 16-byte groups per thread and destination at least
    if (grid < 1) grid = 1;
    if (grid > 64) grid = 64;
    cn_push_exchange_kernel<<<grid, 512, 0, cn_stream(stream)>>>(blocks + off, block_bytes, pp, c->d_peer_flags, c->flags, c->nranks, c->rank,
                                                                 c->xchg_slot, c->d_xchg_state, d_status);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

// ---- 8-bit exchange with the decode inside the consumer GEMM
extern "C" int cn_dotmpi_to_coded_f32(cn_context *ctx, int64_t M, int64_t K, int64_t n_total, const float *d_A, const float *d_Wshard,
                                      cn_coded *out, const cn_epilogue *epi, int mode, void *stream)
{
    CN_REQUIRE(ctx && out && out->codes && out->scales && out->own_fp32, CN_ERR_ARG, "cn_dotmpi_to_coded_f32: null argument");
    CN_REQUIRE(M >= 0 && K >= 0 && n_total >= 0, CN_ERR_SHAPE, "cn_dotmpi_to_coded_f32: negative dimension");
    CN_REQUIRE(!epi || epi->maxout_level <= 1, CN_ERR_UNSUPPORTED, "cn_dotmpi_to_coded_f32: maxout is not available on the sharded product");
    const int G = ctx->comm ? ctx->comm->nranks : 1, rank = ctx->comm ? ctx->comm->rank : 0;
    int64_t start, cnt;
    cn_shard_cols(n_total, rank, G, &start, &cnt);
    cn_epilogue local;
    local.bias = (epi && epi->bias) ? epi->bias + start : nullptr;
    local.activation = epi ? epi->activation : CN_ACT_LINEAR;
    local.maxout_level = 0;
    local.argmax_out = nullptr;
    out->rows = M;
    out->cols = n_total;
    int st = cn_gemm_f32(ctx, 0, 0, M, cnt, K, d_A, M, d_Wshard, K, out->own_fp32, M, &local, mode, stream);
    if (st != CN_OK) return st;
    if ((st = cn_absmax_compress_8bit(ctx, out->own_fp32, M * cnt, out->scales + rank, out->codes + (size_t)M * start, stream)) != CN_OK) return st;
    if (G == 1) return CN_OK;
    if ((st = cn_allgather_scalar_f32(ctx, out->scales, stream)) != CN_OK) return st;
    return cn_allgather_cols_u8(ctx, out->codes, M, n_total, stream);
}

extern "C" int cn_dotmpi_from_coded_f32(cn_context *ctx, const cn_coded *A, int64_t n_total, const float *d_Wshard, float *d_C,
                                        const cn_epilogue *epi, int mode, int exchange, void *stream)
{
    CN_REQUIRE(ctx && A && A->codes && A->scales && d_Wshard && d_C, CN_ERR_ARG, "cn_dotmpi_from_coded_f32: null argument");
    const int64_t M = A->rows, K = A->cols;
    const int G = ctx->comm ? ctx->comm->nranks : 1, rank = ctx->comm ? ctx->comm->rank : 0;
    int64_t start, cnt;
    cn_shard_cols(n_total, rank, G, &start, &cnt);
    if (mode != CN_GEMM_FP32_SIMT && cnt > 0 &&
        cn_gemm_tc_supported(ctx, 0, 0, M, cnt, K, A->own_fp32, M, d_Wshard, K, d_C, M)) {
        if (!ctx->gemm) ctx->gemm = cn_gemm_workspace_new();
        cn_coded_src src;
        src.codes = A->codes;
        src.scales = A->scales;
        src.own_fp32 = A->own_fp32;
        src.nranks = G;
        src.own_rank = rank;
        ctx->gemm->coded_src = &src;   // consumed by the launch inside the call below
        // the fp32 pointer handed down is only a placeholder: the pre-pass reads the codes
        int st = cn_dotmpi_f32(ctx, M, K, n_total, A->own_fp32 ? A->own_fp32 : reinterpret_cast<const float *>(A->codes), d_Wshard, d_C,
                               epi, mode, exchange, stream);
        ctx->gemm->coded_src = nullptr;
        return st;
    }
    // shapes the tensor-core kernel does not take: decode to fp32 scratch first
    void *buf = nullptr;
    int st = cn_gemm_scratch(ctx, CN_GEMM_SLOT_MAXOUT, (size_t)M * K * sizeof(float), &buf);
    if (st != CN_OK) return st;
    float *Af = (float *)buf;
    for (int r = 0; r < G; ++r) {
        int64_t s0, c0;
        cn_shard_cols(K, r, G, &s0, &c0);
        if (c0 == 0) continue;
        if (r == rank && A->own_fp32) {
            CN_CUDA(cudaMemcpyAsync(Af + (size_t)M * s0, A->own_fp32, (size_t)M * c0 * sizeof(float), cudaMemcpyDeviceToDevice, cn_stream(stream)));
        } else if ((st = cn_decompress_8bit_dp(ctx, A->codes + (size_t)M * s0, A->scales + r, M * c0, Af + (size_t)M * s0, stream)) != CN_OK) {
            return st;
        }
    }
    return cn_dotmpi_f32(ctx, M, K, n_total, Af, d_Wshard, d_C, epi, mode, exchange, stream);
}

// ---- activation planes made ahead of the product
extern "C" int cn_gemm_prepare_create(cn_context *ctx, int64_t M, int64_t K, int mode, cn_prepared **out)
{
    CN_REQUIRE(ctx && out, CN_ERR_ARG, "cn_gemm_prepare_create: null argument");
    CN_REQUIRE(M >= 1 && K >= 1, CN_ERR_SHAPE, "cn_gemm_prepare_create: empty operand");
    CN_REQUIRE(mode == CN_GEMM_3XTF32 || mode == CN_GEMM_TF32, CN_ERR_ARG, "cn_gemm_prepare_create: the planes exist for the tensor-core modes only");
    *out = nullptr;
    CN_CUDA(cudaSetDevice(ctx->device));
    cn_prepared *p = new cn_prepared();
    p->ctx = ctx;
    p->M = M;
    p->K = K;
    p->Kpad = (K + 31) / 32 * 32;
    p->mode = mode;
    const size_t plane = (size_t)M * p->Kpad;
    cudaError_t e = cudaMalloc(&p->hi, plane * sizeof(float) * (mode == CN_GEMM_3XTF32 ? 2 : 1));
    if (e != cudaSuccess) {
        delete p;
        return cn_cuda_fail(e, "cn_gemm_prepare_create");
    }
    p->lo = mode == CN_GEMM_3XTF32 ? p->hi + plane : nullptr;
    *out = p;
    return CN_OK;
}

extern "C" int cn_gemm_prepare_destroy(cn_prepared *p)
{
    if (!p) return CN_OK;
    cudaFree(p->hi);
    delete p;
    return CN_OK;
}

extern "C" int cn_gemm_prepare(cn_context *ctx, cn_prepared *p, int transA, const float *d_A, int64_t lda, void *stream)
{
    CN_REQUIRE(ctx && p && d_A && p->ctx == ctx, CN_ERR_ARG, "cn_gemm_prepare: null argument or a handle of another context");
    CN_REQUIRE(lda >= (transA ? p->K : p->M), CN_ERR_SHAPE, "cn_gemm_prepare: leading dimension smaller than the stored rows");
    if (!ctx->gemm) ctx->gemm = cn_gemm_workspace_new();
    int st = cn_gemm_tc_split_activations(ctx, transA, p->M, p->K, d_A, lda, p->hi, p->lo, cn_stream(stream));
    if (st == CN_OK) p->filled = true;
    return st;
}

extern "C" int cn_dotmpi_prepared_f32(cn_context *ctx, const cn_prepared *p, int64_t n_total, const float *d_Wshard, float *d_C,
                                      const cn_epilogue *epi, int exchange, void *stream)
{
    CN_REQUIRE(ctx && p && d_Wshard && d_C && p->ctx == ctx, CN_ERR_ARG, "cn_dotmpi_prepared_f32: null argument or a handle of another context");
    CN_REQUIRE(p->filled, CN_ERR_ARG, "cn_dotmpi_prepared_f32: cn_gemm_prepare has not run on this handle");
    CN_REQUIRE(!epi || epi->maxout_level <= 1, CN_ERR_UNSUPPORTED, "cn_dotmpi_prepared_f32: maxout is not available on the sharded product");
    const int G = ctx->comm ? ctx->comm->nranks : 1, rank = ctx->comm ? ctx->comm->rank : 0;
    int64_t start, cnt;
    cn_shard_cols(n_total, rank, G, &start, &cnt);
    // the planes only feed the tensor-core kernel; every rank must be able to take it (the decision is made from the
    // shapes and this rank's W pointer, like the fused gather's)
    CN_REQUIRE(cnt > 0 && cn_gemm_tc_supported(ctx, 0, 0, p->M, cnt, p->K, p->hi, p->M, d_Wshard, p->K, d_C, p->M), CN_ERR_UNSUPPORTED,
               "cn_dotmpi_prepared_f32: this shard is no shape for the tensor-core kernel (empty, or W not 16-byte aligned)");
    if (!ctx->gemm) ctx->gemm = cn_gemm_workspace_new();
    ctx->gemm->prepared = p;   // consumed by the launch inside the call below; the fp32 pointer handed down is a placeholder
    int st = dotmpi_impl(ctx, 0, p->M, p->K, n_total, p->hi, p->M, d_Wshard, d_C, epi, p->mode, exchange, stream);
    ctx->gemm->prepared = nullptr;
    return st;
}

// ---- diagnostics: the bounded wait on a cross-GPU flag, exercised without a peer.
// Waits for an epoch that nothing will ever write into this context's own probe word, with a caller-chosen cycle
// limit; when the limit runs out the kernel records status 10 and returns, exactly like cn_flag_barrier_kernel does
// when a peer never signals.  Lets a host program (and the tests) see that a missing rank surfaces as CN_ERR_TIMEOUT
// from cn_gemm_check_status instead of a hang.
__global__ void cn_wait_probe_kernel(const unsigned int *flag, unsigned int epoch, long long limit_cycles, unsigned int *status)
{
    const volatile unsigned int *f = flag;
    const long long t0 = clock64();
    while ((int)(*f - epoch) < 0) {
        if (clock64() - t0 > limit_cycles) { atomicMax(status, 10u); break; }
        __nanosleep(200);
    }
}

extern "C" int cn_diag_wait_probe(cn_context *ctx, int64_t limit_cycles, void *stream)
{
    CN_REQUIRE(ctx && limit_cycles > 0 && limit_cycles <= 4000000000LL, CN_ERR_ARG, "cn_diag_wait_probe: limit must be in 1 .. 4e9 cycles");
    unsigned int *d_status = nullptr;
    int st = cn_status_block(ctx, &d_status);
    if (st != CN_OK) return st;
    // word 8 of the status block is never written: the probe waits for it to reach 1
    cn_wait_probe_kernel<<<1, 1, 0, cn_stream(stream)>>>(d_status + 8, 1u, (long long)limit_cycles, d_status);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}
