// Layout boundary and small utilities: row-major <-> column-major transposes, fill, upload/download.
// Replaces to_gpu / to_host / to_col_major / to_row_major / kTranspose (source/basicOps.cu:14-33,35-88,
// 108-127; source/clusterKernels.cu:457-482) with a 32x32 shared-memory tile transpose that uses 64-bit
// indexing (the reference's `int size` overflows at 2^31 elements).
#include "cn_internal.h"

#define TP_TILE 32
#define TP_ROWS 8

// out (C x R, row-major) = transpose of in (R x C, row-major).  One CTA per 32x32 tile, linear tile index.
__global__ void __launch_bounds__(TP_TILE *TP_ROWS)
cn_transpose_kernel(const float *__restrict__ in, float *__restrict__ out, int64_t R, int64_t C, int64_t tiles_c)
{
    __shared__ float tile[TP_TILE][TP_TILE + 1];
    const int64_t tile_id = blockIdx.x;
    const int64_t tr = tile_id / tiles_c, tc = tile_id % tiles_c;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t c = tc * TP_TILE + tx;
#pragma unroll
    for (int j = ty; j < TP_TILE; j += TP_ROWS) {
        const int64_t r = tr * TP_TILE + j;
        if (r < R && c < C) tile[j][tx] = in[r * C + c];
    }
    __syncthreads();
    const int64_t r2 = tr * TP_TILE + tx;
#pragma unroll
    for (int j = ty; j < TP_TILE; j += TP_ROWS) {
        const int64_t c2 = tc * TP_TILE + j;
        if (r2 < R && c2 < C) out[c2 * R + r2] = tile[tx][j];
    }
}

__global__ void cn_fill_kernel(float *__restrict__ A, int64_t n, float v)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) A[i] = v;
}

static int transpose_launch(const float *in, float *out, int64_t R, int64_t C, cudaStream_t s)
{
    if (R == 0 || C == 0) return CN_OK;
    const int64_t tiles_r = (R + TP_TILE - 1) / TP_TILE, tiles_c = (C + TP_TILE - 1) / TP_TILE;
    const int64_t tiles = tiles_r * tiles_c;
    CN_REQUIRE(tiles < (1LL << 31), CN_ERR_UNSUPPORTED, "transpose: %lld tiles exceed the grid limit", (long long)tiles);
    cn_transpose_kernel<<<(unsigned)tiles, TP_TILE * TP_ROWS, 0, s>>>(in, out, R, C, tiles_c);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

// A row-major rows x cols array is the transpose of the col-major array of the same logical matrix.
extern "C" int cn_to_col_major(cn_context *ctx, const float *d_src, float *d_dst, int64_t rows, int64_t cols, void *stream)
{
    CN_REQUIRE(ctx && (rows * cols == 0 || (d_src && d_dst)) && rows >= 0 && cols >= 0, CN_ERR_ARG, "cn_to_col_major: bad argument");
    CN_REQUIRE(d_src != d_dst || rows * cols == 0, CN_ERR_ARG, "cn_to_col_major: in-place transpose is not supported");
    return transpose_launch(d_src, d_dst, rows, cols, cn_stream(stream));
}

extern "C" int cn_to_row_major(cn_context *ctx, const float *d_src, float *d_dst, int64_t rows, int64_t cols, void *stream)
{
    CN_REQUIRE(ctx && (rows * cols == 0 || (d_src && d_dst)) && rows >= 0 && cols >= 0, CN_ERR_ARG, "cn_to_row_major: bad argument");
    CN_REQUIRE(d_src != d_dst || rows * cols == 0, CN_ERR_ARG, "cn_to_row_major: in-place transpose is not supported");
    return transpose_launch(d_src, d_dst, cols, rows, cn_stream(stream));
}

extern "C" int cn_upload_row_major(cn_context *ctx, const float *h_src, float *d_stage, float *d_dst, int64_t rows, int64_t cols, void *stream)
{
    CN_REQUIRE(ctx && h_src && d_stage && d_dst && rows >= 0 && cols >= 0, CN_ERR_ARG, "cn_upload_row_major: bad argument");
    CN_CUDA(cudaMemcpyAsync(d_stage, h_src, (size_t)rows * cols * sizeof(float), cudaMemcpyHostToDevice, cn_stream(stream)));
    return transpose_launch(d_stage, d_dst, rows, cols, cn_stream(stream));
}

extern "C" int cn_download_row_major(cn_context *ctx, const float *d_src, float *d_stage, float *h_dst, int64_t rows, int64_t cols, void *stream)
{
    CN_REQUIRE(ctx && h_dst && d_stage && d_src && rows >= 0 && cols >= 0, CN_ERR_ARG, "cn_download_row_major: bad argument");
    int st = transpose_launch(d_src, d_stage, cols, rows, cn_stream(stream));
    if (st != CN_OK) return st;
    CN_CUDA(cudaMemcpyAsync(h_dst, d_stage, (size_t)rows * cols * sizeof(float), cudaMemcpyDeviceToHost, cn_stream(stream)));
    return CN_OK;
}

// kArange (source/clusterKernels.cu:925-937): the column-major image of the row-major counter start, start+1, ...
__global__ void cn_arange_kernel(float *__restrict__ out, int64_t start, int64_t rows, int64_t cols, int64_t n)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = (float)((i % rows) * cols + (i / rows) + start);
}

extern "C" int cn_arange_f32(cn_context *ctx, float *d_A, int64_t start, int64_t rows, int64_t cols, void *stream)
{
    CN_REQUIRE(ctx && rows >= 0 && cols >= 0 && (rows * cols == 0 || d_A), CN_ERR_ARG, "cn_arange_f32: bad argument");
    const int64_t n = rows * cols;
    if (n == 0) return CN_OK;
    int64_t blocks = (n + 1023) / 1024;
    int64_t cap = (int64_t)ctx->sm_count * 8;
    cn_arange_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, cn_stream(stream)>>>(d_A, start, rows, cols, n);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

extern "C" int cn_fill_f32(cn_context *ctx, float *d_A, int64_t n, float value, void *stream)
{
    CN_REQUIRE(ctx && n >= 0 && (n == 0 || d_A), CN_ERR_ARG, "cn_fill_f32: bad argument");
    if (n == 0) return CN_OK;
    int64_t blocks = (n + 1023) / 1024;
    int64_t cap = (int64_t)ctx->sm_count * 8;
    cn_fill_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, cn_stream(stream)>>>(d_A, n, value);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}
