// GEMM entry point and the fp32 SIMT kernel.
//
// cn_gemm_f32 takes over the cublasSgemm call of ClusterNet::dot (source/clusterNet.cpp:404-487): column-
// major operands, alpha = 1, beta = 0, optional transposes, shape check first.  Shapes the tensor-core
// kernel can take (see cn_gemm_tc.cu) go there; everything else — tiny matrices such as the reference's
// 2x3 . 3x2 known-answer tests, a weight pitch that is not a multiple of 4 — runs on the fp32 FMA kernel
// below, which accumulates along k in order and therefore reproduces plain fp32 dot products exactly.
#include <stdlib.h>
#include "cn_epilogue.cuh"
#include "cn_gemm.h"

#define SG_BM 64
#define SG_BN 64
#define SG_BK 16
#define SG_THREADS 256

// C tile 64x64 per CTA, 4x4 outputs per thread, operands staged through shared memory.
__global__ void __launch_bounds__(SG_THREADS)
cn_sgemm_simt_kernel(int transA, int transB, int64_t M, int64_t N, int64_t K,
                     const float *__restrict__ A, int64_t lda, const float *__restrict__ B, int64_t ldb,
                     float *__restrict__ C, int64_t ldc, const float *__restrict__ bias, int act, int64_t tiles_m)
{
    __shared__ float As[SG_BK][SG_BM + 4];
    __shared__ float Bs[SG_BK][SG_BN + 4];
    const int tid = threadIdx.x;
    const int64_t tile = blockIdx.x;
    const int64_t m0 = (tile % tiles_m) * SG_BM, n0 = (tile / tiles_m) * SG_BN;
    const int tx = tid & 15, ty = tid >> 4;   // thread -> rows tx*4.., cols ty*4..
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int64_t k0 = 0; k0 < K; k0 += SG_BK) {
        // 64 x 16 elements of each operand, 4 per thread
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * SG_THREADS;
            {   // A: walk m fastest when A is stored untransposed (m contiguous), k fastest otherwise
                const int mm = transA ? idx / SG_BK : idx % SG_BM;
                const int kk = transA ? idx % SG_BK : idx / SG_BM;
                const int64_t m = m0 + mm, k = k0 + kk;
                float v = 0.0f;
                if (m < M && k < K) v = transA ? A[k + m * lda] : A[m + k * lda];
                As[kk][mm] = v;
            }
            {   // B: k contiguous when untransposed
                const int kk = transB ? idx / SG_BN : idx % SG_BK;
                const int nn = transB ? idx % SG_BN : idx / SG_BK;
                const int64_t n = n0 + nn, k = k0 + kk;
                float v = 0.0f;
                if (n < N && k < K) v = transB ? B[n + k * ldb] : B[k + n * ldb];
                Bs[kk][nn] = v;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < SG_BK; ++kk) {
            const float4 a = *reinterpret_cast<const float4 *>(&As[kk][tx * 4]);
            const float4 b = *reinterpret_cast<const float4 *>(&Bs[kk][ty * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int64_t n = n0 + ty * 4 + j;
        if (n >= N) continue;
        const float bj = bias ? bias[n] : 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int64_t m = m0 + tx * 4 + i;
            if (m < M) {
                float v = acc[i][j];
                if (bias) v += bj;
                C[m + n * ldc] = cn_apply_activation(v, act);
            }
        }
    }
}

static int simt_launch(cn_context *ctx, int transA, int transB, int64_t M, int64_t N, int64_t K, const float *A, int64_t lda,
                       const float *B, int64_t ldb, float *C, int64_t ldc, const float *bias, int act, cudaStream_t s)
{
    const int64_t tiles_m = (M + SG_BM - 1) / SG_BM, tiles_n = (N + SG_BN - 1) / SG_BN;
    CN_REQUIRE(tiles_m * tiles_n < (1LL << 31), CN_ERR_UNSUPPORTED, "cn_gemm_f32: too many tiles for the fp32 FMA kernel");
    cn_sgemm_simt_kernel<<<(unsigned)(tiles_m * tiles_n), SG_THREADS, 0, s>>>(transA, transB, M, N, K, A, lda, B, ldb, C, ldc, bias, act, tiles_m);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    ctx->gemm_last_path = "simt_fp32";
    return CN_OK;
}

cn_gemm_workspace *cn_gemm_workspace_new()
{
    cn_gemm_workspace *w = new cn_gemm_workspace();
    if (const char *e = getenv("CN_GEMM_NT")) w->force_nt = atoi(e);
    if (const char *e = getenv("CN_GEMM_SPLITS")) w->force_splits = atoi(e);
    if (const char *e = getenv("CN_GEMM_CHAIN")) w->force_chain = atoi(e);
    return w;
}

extern "C" int cn_gemm_set_tuning(cn_context *ctx, int tiles_per_cta, int k_splits, int chain_k_blocks)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_gemm_set_tuning: null context");
    CN_REQUIRE(tiles_per_cta >= 0 && tiles_per_cta <= 2 && k_splits >= 0 && chain_k_blocks >= 0, CN_ERR_ARG,
               "cn_gemm_set_tuning: tiles_per_cta must be 0, 1 or 2, the other two non-negative");
    if (!ctx->gemm) ctx->gemm = cn_gemm_workspace_new();
    ctx->gemm->force_nt = tiles_per_cta;
    ctx->gemm->force_splits = k_splits;
    ctx->gemm->force_chain = chain_k_blocks;
    return CN_OK;
}

int cn_status_block(cn_context *ctx, unsigned int **d_status)
{
    if (!ctx->gemm) ctx->gemm = cn_gemm_workspace_new();
    cn_gemm_workspace *w = ctx->gemm;
    if (!w->d_status) {
        CN_CUDA(cudaMalloc(&w->d_status, 64 + CN_GEMM_MAX_TICKETS * sizeof(unsigned int)));
        CN_CUDA(cudaMemset(w->d_status, 0, 64 + CN_GEMM_MAX_TICKETS * sizeof(unsigned int)));
    }
    *d_status = w->d_status;
    return CN_OK;
}

int cn_gemm_scratch(cn_context *ctx, int slot, size_t bytes, void **out)
{
    if (!ctx->gemm) ctx->gemm = cn_gemm_workspace_new();
    cn_gemm_workspace *w = ctx->gemm;
    if (w->bytes[slot] < bytes) {
        // grown buffers may still be in use by kernels queued earlier: drain before freeing
        if (w->ptr[slot]) {
            CN_CUDA(cudaDeviceSynchronize());
            CN_CUDA(cudaFree(w->ptr[slot]));
            w->ptr[slot] = nullptr;
            w->bytes[slot] = 0;
        }
        size_t want = bytes + (bytes >> 3);
        cudaError_t e = cudaMalloc(&w->ptr[slot], want);
        if (e != cudaSuccess) {
            cudaGetLastError();
            cn_set_error("cn_gemm_f32: cannot allocate %zu bytes of workspace", want);
            return CN_ERR_NOMEM;
        }
        w->bytes[slot] = want;
    }
    *out = w->ptr[slot];
    return CN_OK;
}

void cn_gemm_workspace_free(cn_context *ctx)
{
    if (!ctx->gemm) return;
    for (int i = 0; i < CN_GEMM_SLOTS; ++i) cudaFree(ctx->gemm->ptr[i]);
    cudaFree(ctx->gemm->d_status);
    for (cudaEvent_t e : ctx->gemm->prof_events) cudaEventDestroy(e);
    delete ctx->gemm;
    ctx->gemm = nullptr;
}

extern "C" const char *cn_gemm_last_path(const cn_context *ctx) { return ctx ? ctx->gemm_last_path : ""; }

extern "C" int cn_gemm_f32(cn_context *ctx, int transA, int transB, int64_t M, int64_t N, int64_t K,
                           const float *d_A, int64_t lda, const float *d_B, int64_t ldb, float *d_C, int64_t ldc,
                           const cn_epilogue *epi, int mode, void *stream)
{
    return cn_gemm_dispatch(ctx, transA, transB, M, N, K, d_A, lda, d_B, ldb, d_C, ldc, epi, mode, stream, nullptr, nullptr);
}

int cn_gemm_dispatch(cn_context *ctx, int transA, int transB, int64_t M, int64_t N, int64_t K, const float *d_A, int64_t lda,
                     const float *d_B, int64_t ldb, float *d_C, int64_t ldc, const cn_epilogue *epi, int mode, void *stream,
                     const cn_peer_out *peers, bool *used_peers)
{
    if (used_peers) *used_peers = false;
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_gemm_f32: null context");
    CN_REQUIRE(M >= 0 && N >= 0 && K >= 0, CN_ERR_SHAPE, "cn_gemm_f32: negative dimension");
    CN_REQUIRE(mode >= CN_GEMM_3XTF32 && mode <= CN_GEMM_FP32_SIMT, CN_ERR_ARG, "cn_gemm_f32: unknown mode %d", mode);
    // leading dimensions must cover the stored rows (checkMatrixOperation's role, source/basicOps.cu:839-933)
    CN_REQUIRE(lda >= (transA ? K : M) && ldb >= (transB ? N : K), CN_ERR_SHAPE, "cn_gemm_f32: leading dimension smaller than the stored rows");
    const float *bias = epi ? epi->bias : nullptr;
    const int act = epi ? epi->activation : CN_ACT_LINEAR;
    const int L = (epi && epi->maxout_level > 1) ? epi->maxout_level : 1;
    float *argmax = epi ? epi->argmax_out : nullptr;
    CN_REQUIRE(act >= CN_ACT_LINEAR && act <= CN_ACT_DOUBLE_RELU, CN_ERR_ARG, "cn_gemm_f32: unknown activation %d", act);
    CN_REQUIRE(L <= 32, CN_ERR_ARG, "cn_gemm_f32: maxout level %d above 32", L);
    CN_REQUIRE(N % L == 0, CN_ERR_SHAPE, "cn_gemm_f32: N=%lld is not a multiple of the maxout level %d", (long long)N, L);
    CN_REQUIRE(ldc >= M, CN_ERR_SHAPE, "cn_gemm_f32: ldc smaller than M");
    if (M == 0 || N == 0) return CN_OK;
    CN_REQUIRE(d_C && (K == 0 || (d_A && d_B)), CN_ERR_ARG, "cn_gemm_f32: null buffer");
    cudaStream_t s = cn_stream(stream);

    // maxout that cannot be fused: full product into scratch, then the stand-alone reduction
    float *target = d_C;
    int64_t target_ld = ldc;
    bool tc_ok = mode != CN_GEMM_FP32_SIMT && cn_gemm_tc_supported(ctx, transA, transB, M, N, K, d_A, lda, d_B, ldb, d_C, ldc);
    bool fused_maxout = tc_ok && (L == 1 || cn_gemm_tc_can_fuse_maxout(L));
    if (L > 1 && !fused_maxout) {
        void *p = nullptr;
        int st = cn_gemm_scratch(ctx, CN_GEMM_SLOT_MAXOUT, (size_t)M * N * sizeof(float), &p);
        if (st != CN_OK) return st;
        target = (float *)p;
        target_ld = M;
        CN_REQUIRE(ldc == M, CN_ERR_UNSUPPORTED, "cn_gemm_f32: un-fused maxout needs ldc == M");
    }
    int st;
    if (tc_ok) {
        cn_epilogue e2;
        e2.bias = bias;
        e2.activation = act;
        e2.maxout_level = fused_maxout ? L : 1;
        e2.argmax_out = fused_maxout ? argmax : nullptr;
        const bool push = peers && peers->npeers > 0 && L == 1;
        st = cn_gemm_tc_launch(ctx, M, N, K, d_A, lda, d_B, ldb, target, target_ld, &e2, mode, s, push ? peers : nullptr, transA, transB);
        if (push && used_peers) *used_peers = true;
    } else {
        st = simt_launch(ctx, transA, transB, M, N, K, d_A, lda, d_B, ldb, target, target_ld, bias, act, s);
    }
    if (st != CN_OK) return st;
    if (L > 1 && !fused_maxout) return cn_maxout(ctx, target, d_C, argmax, M, N, L, stream);
    return CN_OK;
}
