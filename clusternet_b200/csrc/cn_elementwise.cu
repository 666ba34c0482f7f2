// Stand-alone bias/activation and maxout kernels over a column-major matrix: the un-fused forms of
// addMatrixVector + activation (source/basicOps.cu:966-974; source/clusterKernels.cu:706-718) and of
// maxout (source/basicOps.cu:1287-1299; kMaxout source/clusterKernels.cu:1432-1458).
#include "cn_epilogue.cuh"

__global__ void cn_bias_act_kernel(const float *__restrict__ A, const float *__restrict__ bias, int act,
                                   float *__restrict__ out, int64_t rows, int64_t n)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v = A[i];
        if (bias) v += bias[i / rows];   // kAddMatrixVector: one bias value per column
        out[i] = cn_apply_activation(v, act);
    }
}

// One warp per (row, output column).  The reference reduces 32 shared-memory slots (slot t = column
// g*L + t for t < L, -FLT_MAX with index -1 otherwise) with a fixed tree: at offsets 16, 8, 4, 2, 1 slot t
// takes slot t+offset when its own value is strictly smaller (reduceToMaxAndArgMax,
// source/clusterKernels.cu:563-604).  The same tree is walked here with shuffles so that ties resolve
// to the same column.
__global__ void cn_maxout_kernel(const float *__restrict__ A, float *__restrict__ out, float *__restrict__ argmax,
                                 int64_t rows, int64_t out_cols, int L)
{
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t total = rows * out_cols;
    for (int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < total; w += warps) {
        const int64_t g = w / rows, row = w % rows;
        float v = -FLT_MAX, idx = -1.0f;
        if (lane < L) {
            v = A[row + (g * L + lane) * rows];
            idx = (float)(g * L + lane);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_down_sync(0xffffffffu, v, off);
            const float oi = __shfl_down_sync(0xffffffffu, idx, off);
            if (lane < off && v < ov) { v = ov; idx = oi; }
        }
        if (lane == 0) {
            out[row + g * rows] = v;
            if (argmax) argmax[row + g * rows] = idx;
        }
    }
}

extern "C" int cn_bias_activation(cn_context *ctx, const float *d_A, const float *d_bias, int activation,
                                  float *d_out, int64_t rows, int64_t cols, void *stream)
{
    CN_REQUIRE(ctx && rows >= 0 && cols >= 0, CN_ERR_ARG, "cn_bias_activation: bad argument");
    const int64_t n = rows * cols;
    if (n == 0) return CN_OK;
    CN_REQUIRE(d_A && d_out, CN_ERR_ARG, "cn_bias_activation: null buffer");
    CN_REQUIRE(activation >= CN_ACT_LINEAR && activation <= CN_ACT_DOUBLE_RELU, CN_ERR_ARG, "cn_bias_activation: unknown activation %d", activation);
    int64_t blocks = (n + 255) / 256, cap = (int64_t)ctx->sm_count * 8;
    cn_bias_act_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, cn_stream(stream)>>>(d_A, d_bias, activation, d_out, rows, n);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

extern "C" int cn_maxout(cn_context *ctx, const float *d_A, float *d_out, float *d_argmax, int64_t rows, int64_t cols,
                         int maxout_level, void *stream)
{
    CN_REQUIRE(ctx && rows >= 0 && cols >= 0, CN_ERR_ARG, "cn_maxout: bad argument");
    // the reference asserts cols % level == 0 and level <= 64, and its 32-slot reduction covers level <= 32
    CN_REQUIRE(maxout_level >= 1 && maxout_level <= 32, CN_ERR_ARG, "cn_maxout: level %d outside 1..32", maxout_level);
    CN_REQUIRE(cols % maxout_level == 0, CN_ERR_SHAPE, "cn_maxout: %lld columns are not a multiple of level %d", (long long)cols, maxout_level);
    const int64_t out_cols = cols / maxout_level, total = rows * out_cols;
    if (total == 0) return CN_OK;
    CN_REQUIRE(d_A && d_out, CN_ERR_ARG, "cn_maxout: null buffer");
    int64_t blocks = (total + 7) / 8, cap = (int64_t)ctx->sm_count * 8;
    cn_maxout_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, cn_stream(stream)>>>(d_A, d_out, d_argmax, rows, out_cols, maxout_level);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}
