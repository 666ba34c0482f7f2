// Elementwise kernels of the data-parallel training step and the 8-bit gradient exchange.
// They take the place of the kernels the reference's Layer class strings together per step
// (source/Layer.cpp:147-178,180-200,314-339,341-437,439-471):
//   kSoftMax source/clusterKernels.cu:651-688, kCreate_t_matrix :775-790, kSub :332-339, kMul :323-330, kAdd :313-320,
//   kScalarMul, kRectifiedLinear_Derivative :813-821, kLogisticGrad, kDoubleRectifiedLinear_Derivative,
//   kRMSprop_with_weight_update :1306-1325,
// and fuse the per-peer decompression_8bit + add loop of Layer::wait_for_synchronization into one pass.
#include <float.h>
#include "cn_gemm.h"

// ---- softmax over the columns of a column-major rows x cols matrix: one thread per row, the row's maximum, sum and
// quotient taken in the reference's order with the same fast exponential, so results match it bit for bit.
__global__ void cn_softmax_kernel(const float *__restrict__ A, float *__restrict__ out, int64_t rows, int64_t cols)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; row < rows; row += stride) {
        float mx = -FLT_MAX;
        for (int64_t i = 0; i < cols; ++i) {
            const float v = A[i * rows + row];
            if (v > mx) mx = v;
        }
        float sum = 0.0f;
        for (int64_t i = 0; i < cols; ++i) sum += __expf(A[i * rows + row] - mx);
        for (int64_t i = 0; i < cols; ++i) out[i * rows + row] = __expf(A[i * rows + row] - mx) / sum;
    }
}

// softmax of each row (as cn_softmax_kernel) and, in the same pass, the output layer's error softmax - onehot(label):
// the three launches softmax / create_t_matrix / sub of the reference's step (source/Layer.cpp:163-165,318-322) in one.
__global__ void cn_softmax_error_kernel(const float *__restrict__ A, const float *__restrict__ labels, float *__restrict__ prob,
                                        float *__restrict__ err, int64_t rows, int64_t cols)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; row < rows; row += stride) {
        float mx = -FLT_MAX;
        for (int64_t i = 0; i < cols; ++i) {
            const float v = A[i * rows + row];
            if (v > mx) mx = v;
        }
        float sum = 0.0f;
        for (int64_t i = 0; i < cols; ++i) sum += __expf(A[i * rows + row] - mx);
        const int64_t hot = (int64_t)(int)labels[row];
        for (int64_t i = 0; i < cols; ++i) {
            const float pr = __expf(A[i * rows + row] - mx) / sum;
            prob[i * rows + row] = pr;
            err[i * rows + row] = pr - (i == hot ? 1.0f : 0.0f);
        }
    }
}

// err_out = err_in * f'(activation), and optionally grad_out = f'(activation) (the reference writes the derivative into
// the layer's `out` matrix and multiplies in a second kernel, source/Layer.cpp:323-329)
template <int ACT>
__global__ void cn_mul_grad_kernel(const float *__restrict__ err_in, const float *__restrict__ act, float *__restrict__ grad_out,
                                   float *__restrict__ err_out, int64_t n)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float a = act[i];
        float g;
        if (ACT == CN_ACT_RELU) g = a > 0.0f ? 1.0f : 0.0f;
        else if (ACT == CN_ACT_LOGISTIC) g = a * (1.0f - a);
        else g = (a > 0.0f && a < 1.0f) ? 1.0f : 0.0f;
        if (grad_out) grad_out[i] = g;
        err_out[i] = err_in[i] * g;
    }
}

// out = one-hot(labels): zero fill and scatter in one pass over the output
__global__ void cn_t_matrix_kernel(const float *__restrict__ labels, float *__restrict__ out, int64_t rows, int64_t n)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t row = i % rows, col = i / rows;
        out[i] = ((int64_t)(int)labels[row] == col) ? 1.0f : 0.0f;
    }
}

enum { EW_ADD = 0, EW_SUB = 1, EW_MUL = 2, EW_SCALAR_MUL = 3, EW_GRAD_RELU = 4, EW_GRAD_LOGISTIC = 5, EW_GRAD_DOUBLE_RELU = 6,
       EW_ABS = 7, EW_DIV = 8, EW_SCALAR_ADD = 9, EW_SQUARE = 10 };

template <int OP>
__global__ void cn_ew_kernel(const float *__restrict__ A, const float *__restrict__ B, float s, float *__restrict__ out, int64_t n)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float a = A[i];
        float r;
        if (OP == EW_ADD) r = a + B[i];
        else if (OP == EW_SUB) r = a - B[i];
        else if (OP == EW_MUL) r = a * B[i];
        else if (OP == EW_SCALAR_MUL) r = a * s;
        else if (OP == EW_GRAD_RELU) r = a > 0.0f ? 1.0f : 0.0f;
        else if (OP == EW_GRAD_LOGISTIC) r = a * (1.0f - a);
        else if (OP == EW_ABS) r = fabsf(a);
        else if (OP == EW_DIV) r = fdividef(a, B[i]);   // kDiv divides with fdividef (source/clusterKernels.cu:341-348)
        else if (OP == EW_SCALAR_ADD) r = a + s;
        else if (OP == EW_SQUARE) r = powf(a, 2.0f);    // kSquare (source/clusterKernels.cu:420-427)
        else r = (a > 0.0f && a < 1.0f) ? 1.0f : 0.0f;
        out[i] = r;
    }
}

// kNesterov_weight_update (source/clusterKernels.cu:1064-1077): g = lr * grad / batch_size; m = momentum * m - g; w -= g
__global__ void cn_nesterov_kernel(const float *__restrict__ grad, float *__restrict__ w, float *__restrict__ m, float lr, float batch_size,
                                   float momentum, int64_t n)
{
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float g = lr * fdividef(grad[i], batch_size);
        m[i] = (momentum * m[i]) - g;
        w[i] -= g;
    }
}

// kRMSprop_with_weight_update: RMS = m*RMS + (1-m)*g^2 ; w -= lr * g / (sqrt(RMS) + 1e-8).  The reference divides with
// fdividef and squares with powf(g, 2.0f); both are reproduced as written.
__device__ __forceinline__ void rmsprop_step(float g, float &rms, float &w, float rms_mult, float rec, float lr)
{
    const float r = (rms_mult * rms) + (powf(g, 2.0f) * rec);
    rms = r;
    w -= lr * fdividef(g, sqrtf(r) + 1.0e-08f);
}

__global__ void cn_rmsprop_kernel(float *__restrict__ RMS, const float *__restrict__ grad, float *__restrict__ w, float rms_mult, float lr, int64_t n)
{
    const float rec = 1.0f - rms_mult;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float r = RMS[i], x = w[i];
        rmsprop_step(grad[i], r, x, rms_mult, rec, lr);
        RMS[i] = r;
        w[i] = x;
    }
}

// grad[i] += sum over peers r != me of decode_r(codes_r[i]); decode tables as kDecompression_8bit builds them, one per
// rank with that rank's scale; peers are added in rank order (the order of the reference's loop).  The gradients of
// several tensors (segments) lie back to back in one buffer, each coded with its own scale per rank.  A rank's block of
// the gathered buffer is [codes of all segments][one scale per segment]; seg_end[s] is the end offset of segment s.
#define CN_SYNC_MAX_SEGMENTS 8
struct SegParams {
    int nseg;
    int64_t seg_end[CN_SYNC_MAX_SEGMENTS];
};

// UPDATE: the RMSprop step of cn_rmsprop_kernel on the summed gradient in the same pass (same arithmetic, one launch less).
// Four elements per thread where the buffers allow 16-byte accesses (vec_ok) and the four lie in one segment.
template <bool UPDATE>
__global__ void __launch_bounds__(512)
cn_decode_sum_multi_kernel(float *__restrict__ grad, const uint8_t *__restrict__ blocks, size_t block_bytes, size_t scales_off,
                           const float *__restrict__ g_tbl, int64_t n, int nranks, int my_rank, const SegParams sp,
                           float *__restrict__ RMS, float *__restrict__ w, float rms_mult, float lr, int vec_ok)
{
    extern __shared__ float lut[];   // (segment, rank) x 256
    for (int e = threadIdx.x; e < sp.nseg * nranks * 256; e += blockDim.x) {
        const int sr = e >> 8, c = e & 255, i = c & 127;
        const int seg = sr / nranks, r = sr - seg * nranks;
        const float p = reinterpret_cast<const float *>(blocks + (size_t)r * block_bytes + scales_off)[seg];
        float v;
        if (i < CN_CODEBOOK_N) {
            v = __fmul_rn(g_tbl[i], p);
            if (c >= 128) v = -v;
        } else {
            v = (c == 255) ? -p : p;
        }
        lut[e] = v;
    }
    __syncthreads();
    const float rec = 1.0f - rms_mult;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x, tid0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    auto one = [&](int64_t i) {
        int seg = 0;
        while (seg + 1 < sp.nseg && i >= sp.seg_end[seg]) ++seg;
        const float *l = lut + (size_t)seg * nranks * 256;
        float g = grad[i];
        for (int r = 0; r < nranks; ++r)
            if (r != my_rank) g += l[(r << 8) + blocks[(size_t)r * block_bytes + i]];
        grad[i] = g;
        if (UPDATE) {
            float q = RMS[i], x = w[i];
            rmsprop_step(g, q, x, rms_mult, rec, lr);
            RMS[i] = q;
            w[i] = x;
        }
    };
    const int64_t n4 = vec_ok ? (n >> 2) : 0;
    for (int64_t v = tid0; v < n4; v += stride) {
        const int64_t i = v << 2;
        int seg = 0;
        while (seg + 1 < sp.nseg && i >= sp.seg_end[seg]) ++seg;
        if (i + 3 >= sp.seg_end[seg] && seg + 1 < sp.nseg) {   // the four straddle a segment boundary
            for (int k = 0; k < 4; ++k) one(i + k);
            continue;
        }
        const float *l = lut + (size_t)seg * nranks * 256;
        float4 g = reinterpret_cast<const float4 *>(grad)[v];
        for (int r = 0; r < nranks; ++r) {
            if (r == my_rank) continue;
            const uint32_t c = *reinterpret_cast<const uint32_t *>(blocks + (size_t)r * block_bytes + i);
            const float *lr_ = l + (r << 8);
            g.x += lr_[c & 0xffu];
            g.y += lr_[(c >> 8) & 0xffu];
            g.z += lr_[(c >> 16) & 0xffu];
            g.w += lr_[c >> 24];
        }
        reinterpret_cast<float4 *>(grad)[v] = g;
        if (UPDATE) {
            float4 q = reinterpret_cast<const float4 *>(RMS)[v], x = reinterpret_cast<const float4 *>(w)[v];
            rmsprop_step(g.x, q.x, x.x, rms_mult, rec, lr);
            rmsprop_step(g.y, q.y, x.y, rms_mult, rec, lr);
            rmsprop_step(g.z, q.z, x.z, rms_mult, rec, lr);
            rmsprop_step(g.w, q.w, x.w, rms_mult, rec, lr);
            reinterpret_cast<float4 *>(RMS)[v] = q;
            reinterpret_cast<float4 *>(w)[v] = x;
        }
    }
    for (int64_t i = (n4 << 2) + tid0; i < n; i += stride) one(i);
}

static int ew_grid(const cn_context *ctx, int64_t n)
{
    int64_t blocks = (n + 255) / 256, cap = (int64_t)ctx->sm_count * 8;
    if (blocks < 1) blocks = 1;
    return (int)(blocks < cap ? blocks : cap);
}

extern "C" int cn_softmax(cn_context *ctx, const float *d_A, float *d_out, int64_t rows, int64_t cols, void *stream)
{
    CN_REQUIRE(ctx && rows >= 0 && cols >= 0 && (rows * cols == 0 || (d_A && d_out)), CN_ERR_ARG, "cn_softmax: bad argument");
    if (rows * cols == 0) return CN_OK;
    cn_softmax_kernel<<<(unsigned)((rows + 127) / 128 < 1024 ? (rows + 127) / 128 : 1024), 128, 0, cn_stream(stream)>>>(d_A, d_out, rows, cols);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

extern "C" int cn_softmax_error(cn_context *ctx, const float *d_A, const float *d_labels, float *d_softmax_out, float *d_error_out,
                                int64_t rows, int64_t cols, void *stream)
{
    CN_REQUIRE(ctx && rows >= 0 && cols >= 0 && (rows * cols == 0 || (d_A && d_labels && d_softmax_out && d_error_out)), CN_ERR_ARG,
               "cn_softmax_error: bad argument");
    if (rows * cols == 0) return CN_OK;
    cn_softmax_error_kernel<<<(unsigned)((rows + 127) / 128 < 1024 ? (rows + 127) / 128 : 1024), 128, 0, cn_stream(stream)>>>(
        d_A, d_labels, d_softmax_out, d_error_out, rows, cols);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

extern "C" int cn_create_t_matrix(cn_context *ctx, const float *d_labels, float *d_out, int64_t rows, int64_t cols, void *stream)
{
    CN_REQUIRE(ctx && rows >= 0 && cols >= 0 && (rows * cols == 0 || (d_labels && d_out)), CN_ERR_ARG, "cn_create_t_matrix: bad argument");
    if (rows * cols == 0) return CN_OK;
    cn_t_matrix_kernel<<<ew_grid(ctx, rows * cols), 256, 0, cn_stream(stream)>>>(d_labels, d_out, rows, rows * cols);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

template <int OP>
static int ew_launch(cn_context *ctx, const float *A, const float *B, float s, float *out, int64_t n, void *stream, bool needs_b)
{
    CN_REQUIRE(ctx && n >= 0 && (n == 0 || (A && out && (!needs_b || B))), CN_ERR_ARG, "elementwise op: bad argument");
    if (n == 0) return CN_OK;
    cn_ew_kernel<OP><<<ew_grid(ctx, n), 256, 0, cn_stream(stream)>>>(A, B, s, out, n);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

extern "C" int cn_add(cn_context *ctx, const float *a, const float *b, float *out, int64_t n, void *stream) { return ew_launch<EW_ADD>(ctx, a, b, 0.f, out, n, stream, true); }
extern "C" int cn_sub(cn_context *ctx, const float *a, const float *b, float *out, int64_t n, void *stream) { return ew_launch<EW_SUB>(ctx, a, b, 0.f, out, n, stream, true); }
extern "C" int cn_mul(cn_context *ctx, const float *a, const float *b, float *out, int64_t n, void *stream) { return ew_launch<EW_MUL>(ctx, a, b, 0.f, out, n, stream, true); }
extern "C" int cn_scalar_mul(cn_context *ctx, const float *a, float s, float *out, int64_t n, void *stream) { return ew_launch<EW_SCALAR_MUL>(ctx, a, nullptr, s, out, n, stream, false); }

extern "C" int cn_div(cn_context *ctx, const float *a, const float *b, float *out, int64_t n, void *stream) { return ew_launch<EW_DIV>(ctx, a, b, 0.f, out, n, stream, true); }
extern "C" int cn_scalar_add(cn_context *ctx, const float *a, float s, float *out, int64_t n, void *stream) { return ew_launch<EW_SCALAR_ADD>(ctx, a, nullptr, s, out, n, stream, false); }
extern "C" int cn_abs(cn_context *ctx, const float *a, float *out, int64_t n, void *stream) { return ew_launch<EW_ABS>(ctx, a, nullptr, 0.f, out, n, stream, false); }
extern "C" int cn_square(cn_context *ctx, const float *a, float *out, int64_t n, void *stream) { return ew_launch<EW_SQUARE>(ctx, a, nullptr, 0.f, out, n, stream, false); }

extern "C" int cn_nesterov_update(cn_context *ctx, const float *d_grad, float *d_w, float *d_m, float learning_rate, int64_t batch_size,
                                  float momentum, int64_t n, void *stream)
{
    CN_REQUIRE(ctx && n >= 0 && batch_size > 0 && (n == 0 || (d_grad && d_w && d_m)), CN_ERR_ARG, "cn_nesterov_update: bad argument");
    if (n == 0) return CN_OK;
    cn_nesterov_kernel<<<ew_grid(ctx, n), 256, 0, cn_stream(stream)>>>(d_grad, d_w, d_m, learning_rate, (float)batch_size, momentum, n);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

extern "C" int cn_activation_gradient(cn_context *ctx, const float *d_activation, int activation, float *d_out, int64_t n, void *stream)
{
    switch (activation) {
        case CN_ACT_RELU: return ew_launch<EW_GRAD_RELU>(ctx, d_activation, nullptr, 0.f, d_out, n, stream, false);
        case CN_ACT_LOGISTIC: return ew_launch<EW_GRAD_LOGISTIC>(ctx, d_activation, nullptr, 0.f, d_out, n, stream, false);
        case CN_ACT_DOUBLE_RELU: return ew_launch<EW_GRAD_DOUBLE_RELU>(ctx, d_activation, nullptr, 0.f, d_out, n, stream, false);
    }
    cn_set_error("cn_activation_gradient: no derivative for activation %d (the reference throws 'Unknown unit')", activation);
    return CN_ERR_ARG;
}

extern "C" int cn_mul_activation_gradient(cn_context *ctx, const float *d_error_in, const float *d_activation, int activation,
                                          float *d_gradient_out, float *d_error_out, int64_t n, void *stream)
{
    CN_REQUIRE(ctx && n >= 0 && (n == 0 || (d_error_in && d_activation && d_error_out)), CN_ERR_ARG, "cn_mul_activation_gradient: bad argument");
    if (n == 0) return CN_OK;
    const int grid = ew_grid(ctx, n);
    switch (activation) {
        case CN_ACT_RELU: cn_mul_grad_kernel<CN_ACT_RELU><<<grid, 256, 0, cn_stream(stream)>>>(d_error_in, d_activation, d_gradient_out, d_error_out, n); break;
        case CN_ACT_LOGISTIC: cn_mul_grad_kernel<CN_ACT_LOGISTIC><<<grid, 256, 0, cn_stream(stream)>>>(d_error_in, d_activation, d_gradient_out, d_error_out, n); break;
        case CN_ACT_DOUBLE_RELU: cn_mul_grad_kernel<CN_ACT_DOUBLE_RELU><<<grid, 256, 0, cn_stream(stream)>>>(d_error_in, d_activation, d_gradient_out, d_error_out, n); break;
        default:
            cn_set_error("cn_mul_activation_gradient: no derivative for activation %d (the reference throws 'Unknown unit')", activation);
            return CN_ERR_ARG;
    }
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

extern "C" int cn_rmsprop_update(cn_context *ctx, float *d_rms, const float *d_grad, float *d_w, float rms_multiplier, float learning_rate,
                                 int64_t n, void *stream)
{
    CN_REQUIRE(ctx && n >= 0 && (n == 0 || (d_rms && d_grad && d_w)), CN_ERR_ARG, "cn_rmsprop_update: bad argument");
    if (n == 0) return CN_OK;
    cn_rmsprop_kernel<<<ew_grid(ctx, n), 256, 0, cn_stream(stream)>>>(d_rms, d_grad, d_w, rms_multiplier, learning_rate, n);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

// comm-side pieces live in cn_comm.cu
int cn_comm_info(cn_context *ctx, int *rank, int *nranks, float **d_scales);

int cn_comm_gather_blocks(cn_context *ctx, uint8_t *d_blocks, size_t block_bytes, void *stream);
int cn_comm_push_area(cn_context *ctx, size_t block_bytes, void *stream, uint8_t **blocks);
int cn_comm_push_blocks(cn_context *ctx, uint8_t *blocks, size_t block_bytes, void *stream);

// Several tensors that lie back to back in one buffer (the gradients of all layers of a step), each coded with its own
// scale exactly as cn_grad_sync_8bit would code it alone, but exchanged with ONE all-gather and summed in ONE pass.
extern "C" int cn_grad_sync_8bit(cn_context *ctx, float *d_grad, int64_t n, float fixed_precision, void *stream);

static int grad_sync_multi_impl(cn_context *ctx, float *d_grad, const int64_t *segment_sizes, int num_segments, float fixed_precision,
                                float *d_rms, float *d_w, float rms_multiplier, float learning_rate, void *stream)
{
    const bool update = d_rms != nullptr;
    CN_REQUIRE(ctx && segment_sizes && num_segments >= 1, CN_ERR_ARG, "cn_grad_sync_8bit_multi: bad argument");
    int rank = 0, G = 1;
    float *unused = nullptr;
    cn_comm_info(ctx, &rank, &G, &unused);
    int64_t n = 0;
    for (int s = 0; s < num_segments; ++s) {
        CN_REQUIRE(segment_sizes[s] >= 0, CN_ERR_ARG, "cn_grad_sync_8bit_multi: negative segment size");
        n += segment_sizes[s];
    }
    if (n == 0) return CN_OK;
    CN_REQUIRE(d_grad, CN_ERR_ARG, "cn_grad_sync_8bit_multi: null buffer");
    if (G == 1) return update ? cn_rmsprop_update(ctx, d_rms, d_grad, d_w, rms_multiplier, learning_rate, n, stream) : CN_OK;
    if (num_segments > CN_SYNC_MAX_SEGMENTS || (size_t)num_segments * G * 1024 > 48 * 1024) {
        // too many tables for one pass: segment by segment
        int64_t off = 0;
        for (int s = 0; s < num_segments; ++s) {
            int st = cn_grad_sync_8bit(ctx, d_grad + off, segment_sizes[s], fixed_precision, stream);
            if (st != CN_OK) return st;
            off += segment_sizes[s];
        }
        return update ? cn_rmsprop_update(ctx, d_rms, d_grad, d_w, rms_multiplier, learning_rate, n, stream) : CN_OK;
    }
    const size_t scales_off = ((size_t)n + 15) & ~(size_t)15;
    const size_t block_bytes = scales_off + (((size_t)num_segments * sizeof(float) + 15) & ~(size_t)15);
    // the blocks travel by direct stores into the peers' memory where the communicator can do that (one process per
    // GPU), else through the library's all-gather
    uint8_t *blocks = nullptr;
    int st = cn_comm_push_area(ctx, block_bytes, stream, &blocks);
    if (st != CN_OK) return st;
    const bool pushed = blocks != nullptr;
    if (!pushed) {
        void *buf = nullptr;
        if ((st = cn_gemm_scratch(ctx, CN_GEMM_SLOT_EXCHANGE, (size_t)G * block_bytes, &buf)) != CN_OK) return st;
        blocks = (uint8_t *)buf;
    }
    uint8_t *mine = blocks + (size_t)rank * block_bytes;
    float *my_scales = reinterpret_cast<float *>(mine + scales_off);
    SegParams sp;
    sp.nseg = num_segments;
    int64_t off = 0;
    bool exchanged = false;
    if (pushed && num_segments == 1 && fixed_precision <= 0.0f) {
        // one tensor, scale = its absmax: code and push in ONE launch where the tensor is small enough for that form
        cn_codec_push cp;
        if ((st = cn_comm_push_params(ctx, block_bytes, scales_off, &cp)) != CN_OK) return st;
        int done = 0;
        if ((st = cn_absmax_compress_push(ctx, d_grad, n, my_scales, mine, &cp, stream, &done)) != CN_OK) return st;
        exchanged = done != 0;
    }
    for (int s = 0; s < num_segments; ++s) {
        const int64_t sz = segment_sizes[s];
        if (exchanged) {
            // done above
        } else if (fixed_precision > 0.0f) {
            st = cn_fill_f32(ctx, my_scales + s, 1, fixed_precision, stream);
            if (st == CN_OK && sz > 0) st = cn_compress_8bit_dp(ctx, d_grad + off, my_scales + s, sz, mine + off, stream);
        } else {
            st = cn_absmax_compress_8bit(ctx, d_grad + off, sz, my_scales + s, mine + off, stream);   // one launch per tensor
        }
        if (st != CN_OK) return st;
        off += sz;
        sp.seg_end[s] = off;
    }
    for (int s = num_segments; s < CN_SYNC_MAX_SEGMENTS; ++s) sp.seg_end[s] = off;
    if (!exchanged) {
        st = pushed ? cn_comm_push_blocks(ctx, blocks, block_bytes, stream) : cn_comm_gather_blocks(ctx, blocks, block_bytes, stream);
        if (st != CN_OK) return st;
    }
    const int vec_ok = ((uintptr_t)d_grad % 16 == 0) && ((uintptr_t)blocks % 16 == 0) &&
                       (!update || ((uintptr_t)d_rms % 16 == 0 && (uintptr_t)d_w % 16 == 0));
    const int64_t work = vec_ok ? (n + 3) / 4 : n;
    int64_t nblocks = (work + 511) / 512, cap = (int64_t)ctx->sm_count * 4;
    const unsigned grid = (unsigned)(nblocks < cap ? nblocks : cap);
    const size_t smem = (size_t)num_segments * G * 256 * sizeof(float);
    if (update)
        cn_decode_sum_multi_kernel<true><<<grid, 512, smem, cn_stream(stream)>>>(d_grad, blocks, block_bytes, scales_off, ctx->d_tbl, n, G, rank, sp,
                                                                                 d_rms, d_w, rms_multiplier, learning_rate, vec_ok);
    else
        cn_decode_sum_multi_kernel<false><<<grid, 512, smem, cn_stream(stream)>>>(d_grad, blocks, block_bytes, scales_off, ctx->d_tbl, n, G, rank, sp,
                                                                                  nullptr, nullptr, 0.f, 0.f, vec_ok);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

extern "C" int cn_grad_sync_8bit(cn_context *ctx, float *d_grad, int64_t n, float fixed_precision, void *stream)
{
    CN_REQUIRE(ctx && n >= 0 && (n == 0 || d_grad), CN_ERR_ARG, "cn_grad_sync_8bit: bad argument");
    return grad_sync_multi_impl(ctx, d_grad, &n, 1, fixed_precision, nullptr, nullptr, 0.f, 0.f, stream);
}

extern "C" int cn_grad_sync_8bit_multi(cn_context *ctx, float *d_grad, const int64_t *segment_sizes, int num_segments,
                                       float fixed_precision, void *stream)
{
    return grad_sync_multi_impl(ctx, d_grad, segment_sizes, num_segments, fixed_precision, nullptr, nullptr, 0.f, 0.f, stream);
}

// cn_grad_sync_8bit_multi followed by cn_rmsprop_update over the same elements, with the update done in the pass that sums
// the decoded gradients: the results (gradient, RMS state, weights) are those of the two calls bit for bit.
extern "C" int cn_grad_sync_8bit_rmsprop(cn_context *ctx, float *d_grad, const int64_t *segment_sizes, int num_segments,
                                         float fixed_precision, float *d_rms, float *d_w, float rms_multiplier, float learning_rate,
                                         void *stream)
{
    CN_REQUIRE(d_rms && d_w, CN_ERR_ARG, "cn_grad_sync_8bit_rmsprop: null state or weight buffer");
    return grad_sync_multi_impl(ctx, d_grad, segment_sizes, num_segments, fixed_precision, d_rms, d_w, rms_multiplier, learning_rate, stream);
}
