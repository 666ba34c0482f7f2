// 8-bit dynamic-float codec for sm_100a: absmax, compress, decompress.
//
// All three kernels are HBM-bound byte/float streams (4, 5 and 5 algorithmic bytes per element), so the
// design is: persistent grid sized from the SM count, 16-byte loads, 4/16-byte stores, several
// independent loads in flight per thread, and every per-call table built once per CTA in shared memory.
//
// Compressor.  The reference (source/clusterKernels.cu:1163-1232) divides by `precision`, then runs a
// six-step search over a 126-entry table and a nearest-of-two pick.  code(|x/precision|) is a
// non-decreasing step function with 127 steps (cn_codec_build_thresholds), and fl(|x|/|precision|) is
// non-decreasing in |x|, so for one launch the code is a step function of |x| itself.  Each CTA
// therefore (1) finds, with IEEE divisions, the smallest fp32 |x| that reaches each of the 127 steps,
// (2) spreads those 127 boundaries over a table indexed by the top 16 bits of |x| (exponent + 7 mantissa
// bits): one entry = {boundary inside this bucket or 0, code below, code above}, and then (3) codes each
// element with one shared-memory read and one integer compare, with no division in the stream.
// Whenever that construction is not available (precision zero, non-finite or outside 2^-100..2^100, or a
// codebook so dense that two boundaries share a bucket) the kernel takes the generic path: IEEE divide
// per element, then a 7-step search of the 127 thresholds.  Both paths give identical codes.
#include <math.h>
#include "cn_internal.h"

#define CODEC_THREADS 1024
#define ABSMAX_THREADS 512
#define LUT_SHIFT 16
#define LUT_MAX 2816

// The small per-codebook tables travel as kernel parameters (constant bank): read from global memory they would be a
// cold DRAM miss on the critical path of every launch's table build.
struct CodecConst {
    uint32_t thr[128];   // 127 thresholds + pad
    uint32_t lc[128];    // level codes
};
struct DecodeConst {
    float tbl[128];      // codebook (126 used)
};

struct CodecTables {
    uint2 lut[LUT_MAX];     // {boundary bits (0 = none), code_below | code_above << 16}
    uint32_t X[128];        // per-launch boundaries in |x| space (bit patterns), [127] = pad
    uint32_t T[128];        // thresholds in |x/precision| space, [127] = pad
    uint32_t lc[128];       // level codes
    uint32_t xtop;          // boundary of the top level (code 127), tested on its own: it lies too close to its neighbour for the table
    int base;
    int nb;
    int bad;
};

// number of entries of a sorted 127-array (+ one pad that is never <=) that are <= key
__device__ __forceinline__ int count_le(const uint32_t *s, uint32_t key)
{
    int lo = 0;
#pragma unroll
    for (int step = 64; step > 0; step >>= 1)
        if (s[lo + step - 1] <= key) lo += step;
    return lo;
}

__device__ __forceinline__ uint32_t generic_code(float x, float p, const CodecTables &t)
{
    float a = __fdiv_rn(x, p);
    if (a != a) return 1u;   // every comparison of the reference's search fails for NaN: it ends on index 1, sign clear
    bool neg = a < 0.0f;
    uint32_t ab = __float_as_uint(a) & 0x7fffffffu;
    uint32_t c = t.lc[count_le(t.T, ab)];
    return (neg && c != 254u) ? (c | 0x80u) : c;
}

__device__ __forceinline__ uint32_t fast_code(uint32_t xb, uint32_t pb, const CodecTables &t, int base, int nbm1, uint32_t xtop)
{
    uint32_t ab = xb & 0x7fffffffu;
    int key = (int)(ab >> LUT_SHIFT) - base;
    key = max(key, 0);
    key = min(key, nbm1);
    uint2 e = t.lut[key];
    uint32_t c = (ab >= e.x) ? (e.y >> 16) : e.y;
    if (ab >= xtop) c = 127u;
    c |= ((xb ^ pb) >> 24) & 0x80u;     // sign of x/precision; code 254 already has bit 7 set
    if (ab > 0x7f800000u) c = 1u;       // NaN input
    return c;                           // only the low byte is meaningful
}

__device__ __forceinline__ uint32_t pack4(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3)
{
    return __byte_perm(__byte_perm(c0, c1, 0x0040), __byte_perm(c2, c3, 0x0040), 0x5410);
}

// Four codes of the fast path for one 16-byte group.  The sign bits are taken from the top bytes of the four inputs in
// one go; a NaN anywhere in the group (rare) sends the group through the per-element form.
__device__ __forceinline__ uint32_t fast_code4(const float4 q, uint32_t pb, uint32_t psign4, const CodecTables &t, int base, int nbm1, uint32_t xtop)
{
    const uint32_t x0 = __float_as_uint(q.x), x1 = __float_as_uint(q.y), x2 = __float_as_uint(q.z), x3 = __float_as_uint(q.w);
    const uint32_t a0 = x0 & 0x7fffffffu, a1 = x1 & 0x7fffffffu, a2 = x2 & 0x7fffffffu, a3 = x3 & 0x7fffffffu;
    if (max(max(a0, a1), max(a2, a3)) > 0x7f800000u)
        return pack4(fast_code(x0, pb, t, base, nbm1, xtop), fast_code(x1, pb, t, base, nbm1, xtop),
                     fast_code(x2, pb, t, base, nbm1, xtop), fast_code(x3, pb, t, base, nbm1, xtop));
    uint32_t c[4];
    const uint32_t a[4] = {a0, a1, a2, a3};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int key = (int)(a[i] >> LUT_SHIFT) - base;
        key = min(max(key, 0), nbm1);
        const uint2 e = t.lut[key];
        c[i] = (a[i] >= e.x) ? (e.y >> 16) : e.y;
        if (a[i] >= xtop) c[i] = 127u;
    }
    // top bytes of x0..x3 -> one word; flip by the sign of precision; keep bit 7 of each byte
    const uint32_t tops = __byte_perm(__byte_perm(x0, x1, 0x0073), __byte_perm(x2, x3, 0x0073), 0x5410);
    return pack4(c[0], c[1], c[2], c[3]) | ((tops ^ psign4) & 0x80808080u);
}

template <bool PRECISION_ON_DEVICE>
__global__ void __launch_bounds__(CODEC_THREADS, 1)
cn_compress_kernel(const float *__restrict__ A, float precision_arg, const float *__restrict__ d_precision,
                   int64_t n, uint8_t *__restrict__ out, const __grid_constant__ CodecConst cc, int vector_ok)
{
    __shared__ CodecTables t;
    const int tid = threadIdx.x;
    const float p = PRECISION_ON_DEVICE ? *d_precision : precision_arg;
    const uint32_t pb = __float_as_uint(p);
    const uint32_t psign4 = (pb >> 31) * 0x80808080u;
    const float ap = fabsf(p);
    // 2^-100 <= |p| <= 2^100 keeps every boundary T*|p| a normal number; NaN fails both tests
    const bool p_ok = (ap >= 7.8886090522101181e-31f) && (ap <= 1.2676506002282294e30f);

    const int64_t nvec = vector_ok ? (n >> 2) : 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t step = 4 * stride;
    int64_t v = (int64_t)blockIdx.x * blockDim.x + tid;
    const float4 *A4 = reinterpret_cast<const float4 *>(A);
    uint32_t *out4 = reinterpret_cast<uint32_t *>(out);

    // the first group of loads is issued before the table build so that its latency overlaps it
    float4 cur[4];
    const bool have_group = v + 3 * stride < nvec;
    if (have_group) {
#pragma unroll
        for (int u = 0; u < 4; ++u) cur[u] = __ldcs(A4 + v + u * stride);
    }

    if (tid < 128) {
        t.T[tid] = cc.thr[tid];
        t.lc[tid] = cc.lc[tid];
        uint32_t xb = 0xffffffffu;
        bool good = true;
        if (tid < CN_NUM_THR && p_ok) {
            const float T = __uint_as_float(cc.thr[tid]);
            xb = __float_as_uint(__fmul_rn(T, ap));
            // smallest |x| with fl(|x|/|p|) >= T.  The product is within a few ulps of it: walk down while the lower
            // neighbour still reaches T, and up only if nothing was found below (then xb itself may fall short).
            int down = 0;
            for (; down < 6; ++down) {
                if (xb > 0u && __fdiv_rn(__uint_as_float(xb - 1u), ap) >= T) --xb; else break;
            }
            good = down < 6;
            if (down == 0) {
                int up = 0;
                for (; up < 6; ++up) {
                    if (__fdiv_rn(__uint_as_float(xb), ap) < T) ++xb; else break;
                }
                good = up < 6;
            }
        }
        t.X[tid] = good ? xb : 0xfffffffeu;   // 0xfffffffe marks a boundary that could not be pinned
    }
    __syncthreads();
    if (tid < 32) {
        bool bad = !p_ok;
        for (int k = 0; k < 4; ++k) {
            const int idx = tid + 32 * k;
            if (idx < CN_NUM_THR && t.X[idx] == 0xfffffffeu) bad = true;
        }
        bad = __any_sync(0xffffffffu, bad);
        if (tid == 0) {
            t.xtop = t.X[CN_NUM_THR - 1];
            t.X[CN_NUM_THR - 1] = 0xffffffffu;   // the table below covers boundaries 0..125 only
            const int base = (int)(t.X[0] >> LUT_SHIFT);
            const int nb = (int)(t.X[CN_NUM_THR - 2] >> LUT_SHIFT) - base + 1;
            t.base = base;
            t.nb = nb;
            t.bad = (bad || nb > LUT_MAX || nb < 1) ? 1 : 0;
        }
    }
    __syncthreads();
    if (!t.bad) {
        const int base = t.base, nb = t.nb;
        for (int b = tid; b < nb; b += CODEC_THREADS) {
            // boundaries that lie in lower buckets: compare on the bucket index
            const uint32_t kbv = (uint32_t)(b + base);
            int lo = 0;
#pragma unroll
            for (int step2 = 64; step2 > 0; step2 >>= 1)
                if ((t.X[lo + step2 - 1] >> LUT_SHIFT) < kbv) lo += step2;
            uint2 e;
            if (lo < CN_NUM_THR - 1 && (t.X[lo] >> LUT_SHIFT) == kbv) {
                e.x = t.X[lo];
                e.y = t.lc[lo] | (t.lc[lo + 1] << 16);
                if (lo + 1 < CN_NUM_THR - 1 && (t.X[lo + 1] >> LUT_SHIFT) == kbv) atomicOr(&t.bad, 1);  // two boundaries in one bucket
            } else {
                e.x = 0u;
                e.y = t.lc[lo] | (t.lc[lo] << 16);
            }
            t.lut[b] = e;
        }
    }
    __syncthreads();
    const bool fast = t.bad == 0;
    const int base = t.base, nbm1 = t.nb - 1;
    const uint32_t xtop = t.xtop;

#define CN_CODE4(q)                                                                                             \
    (fast ? fast_code4((q), pb, psign4, t, base, nbm1, xtop)                                                    \
          : pack4(generic_code((q).x, p, t), generic_code((q).y, p, t), generic_code((q).z, p, t), generic_code((q).w, p, t)))

    // whole groups of four 16-byte loads per thread; the next group is in flight while the current one is coded
    if (have_group) {
        while (true) {
            const int64_t vn = v + step;
            const bool more = vn + 3 * stride < nvec;
            float4 nxt[4];
            if (more) {
#pragma unroll
                for (int u = 0; u < 4; ++u) nxt[u] = __ldcs(A4 + vn + u * stride);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) __stcs(out4 + v + u * stride, CN_CODE4(cur[u]));
            v = vn;
            if (!more) break;
#pragma unroll
            for (int u = 0; u < 4; ++u) cur[u] = nxt[u];
        }
    }
    if (v < nvec) {   // last, partial group: all its loads are issued before any is used
        float4 q[3];
        bool has[3];
#pragma unroll
        for (int u = 0; u < 3; ++u) {
            has[u] = v + u * stride < nvec;
            if (has[u]) q[u] = __ldcs(A4 + v + u * stride);
        }
#pragma unroll
        for (int u = 0; u < 3; ++u)
            if (has[u]) __stcs(out4 + v + u * stride, CN_CODE4(q[u]));
    }
#undef CN_CODE4
    // elements not covered by whole 16-byte groups (all of them when the buffers are not aligned)
    for (int64_t i = (nvec << 2) + (int64_t)blockIdx.x * blockDim.x + tid; i < n; i += stride) {
        float x = A[i];
        uint32_t c = fast ? fast_code(__float_as_uint(x), pb, t, base, nbm1, xtop) : generic_code(x, p, t);
        out[i] = (uint8_t)c;
    }
}

// kDecompression_8bit (source/clusterKernels.cu:1135-1160): 256-entry table built in the reference's
// statement order, then out[i] = table[code].
template <bool PRECISION_ON_DEVICE>
__global__ void __launch_bounds__(CODEC_THREADS, 1)
cn_decompress_kernel(const uint8_t *__restrict__ codes, float precision_arg, const float *__restrict__ d_precision,
                     int64_t n, float *__restrict__ out, const __grid_constant__ DecodeConst dc, int vector_ok)
{
    __shared__ float lut[256];
    const int tid = threadIdx.x;
    const float p = PRECISION_ON_DEVICE ? *d_precision : precision_arg;
    if (tid < 256) {
        float v = 0.0f;
        const int i = tid & 127;
        if (i < CN_CODEBOOK_N) {
            v = __fmul_rn(dc.tbl[i], p);
            if (tid >= 128) v = -v;
        } else {
            v = (tid == 255) ? -p : p;   // 126, 127, 254 -> +precision; 255 -> -precision
        }
        lut[tid] = v;
    }
    __syncthreads();
    const int64_t nvec = vector_ok ? (n >> 2) : 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t v = (int64_t)blockIdx.x * blockDim.x + tid;
    const uint32_t *in4 = reinterpret_cast<const uint32_t *>(codes);
    float4 *out4 = reinterpret_cast<float4 *>(out);
#define CN_DEC4(w) make_float4(lut[(w) & 0xffu], lut[((w) >> 8) & 0xffu], lut[((w) >> 16) & 0xffu], lut[(w) >> 24])
    if (v + 3 * stride < nvec) {
        const int64_t step = 4 * stride;
        uint32_t cur[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) cur[u] = __ldcs(in4 + v + u * stride);
        while (true) {
            const int64_t vn = v + step;
            const bool more = vn + 3 * stride < nvec;
            uint32_t nxt[4];
            if (more) {
#pragma unroll
                for (int u = 0; u < 4; ++u) nxt[u] = __ldcs(in4 + vn + u * stride);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) __stcs(out4 + v + u * stride, CN_DEC4(cur[u]));
            v = vn;
            if (!more) break;
#pragma unroll
            for (int u = 0; u < 4; ++u) cur[u] = nxt[u];
        }
    }
    if (v < nvec) {   // last, partial group: all its loads are issued before any is used
        uint32_t q[3];
        bool has[3];
#pragma unroll
        for (int u = 0; u < 3; ++u) {
            has[u] = v + u * stride < nvec;
            if (has[u]) q[u] = __ldcs(in4 + v + u * stride);
        }
#pragma unroll
        for (int u = 0; u < 3; ++u)
            if (has[u]) __stcs(out4 + v + u * stride, CN_DEC4(q[u]));
    }
#undef CN_DEC4
    for (int64_t i = (nvec << 2) + (int64_t)blockIdx.x * blockDim.x + tid; i < n; i += stride) out[i] = lut[codes[i]];
}

// absmax (ABS) or plain max: one pass; every CTA leaves its partial maximum in the scratch array, the CTA that draws
// the last ticket folds the partials, writes the result and resets the ticket for the next launch.
template <bool ABS>
__device__ __forceinline__ float absmax_term(float x) { return ABS ? fabsf(x) : x; }

template <bool ABS>
__global__ void __launch_bounds__(ABSMAX_THREADS)
cn_absmax_kernel(const float *__restrict__ A, int64_t n, float *__restrict__ out, float *__restrict__ partials,
                 unsigned int *__restrict__ ticket, int vector_ok)
{
    __shared__ float warp_max[ABSMAX_THREADS / 32];
    __shared__ bool is_last;
    const int tid = threadIdx.x;
    float m = -1.0f;   // the reference seeds thrust::reduce with -1.0f (source/basicOps.cu:1079)
    const int64_t nvec = vector_ok ? (n >> 2) : 0;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const float4 *A4 = reinterpret_cast<const float4 *>(A);
    int64_t v = (int64_t)blockIdx.x * blockDim.x + tid;
    for (; v + 3 * stride < nvec; v += 4 * stride) {
        float4 q0 = __ldcs(A4 + v), q1 = __ldcs(A4 + v + stride), q2 = __ldcs(A4 + v + 2 * stride), q3 = __ldcs(A4 + v + 3 * stride);
        m = fmaxf(m, fmaxf(fmaxf(absmax_term<ABS>(q0.x), absmax_term<ABS>(q0.y)), fmaxf(absmax_term<ABS>(q0.z), absmax_term<ABS>(q0.w))));
        m = fmaxf(m, fmaxf(fmaxf(absmax_term<ABS>(q1.x), absmax_term<ABS>(q1.y)), fmaxf(absmax_term<ABS>(q1.z), absmax_term<ABS>(q1.w))));
        m = fmaxf(m, fmaxf(fmaxf(absmax_term<ABS>(q2.x), absmax_term<ABS>(q2.y)), fmaxf(absmax_term<ABS>(q2.z), absmax_term<ABS>(q2.w))));
        m = fmaxf(m, fmaxf(fmaxf(absmax_term<ABS>(q3.x), absmax_term<ABS>(q3.y)), fmaxf(absmax_term<ABS>(q3.z), absmax_term<ABS>(q3.w))));
    }
    if (v < nvec) {   // last, partial group: all its loads are issued before any is used
        float4 q[3];
#pragma unroll
        for (int u = 0; u < 3; ++u) q[u] = (v + u * stride < nvec) ? __ldcs(A4 + v + u * stride) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 3; ++u)
            if (v + u * stride < nvec) m = fmaxf(m, fmaxf(fmaxf(absmax_term<ABS>(q[u].x), absmax_term<ABS>(q[u].y)), fmaxf(absmax_term<ABS>(q[u].z), absmax_term<ABS>(q[u].w))));
    }
    for (int64_t i = (nvec << 2) + (int64_t)blockIdx.x * blockDim.x + tid; i < n; i += stride) m = fmaxf(m, absmax_term<ABS>(A[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31) == 0) warp_max[tid >> 5] = m;
    __syncthreads();
    if (tid < 32) {
        m = tid < ABSMAX_THREADS / 32 ? warp_max[tid] : -1.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (tid == 0) {
            partials[blockIdx.x] = m;
            __threadfence();
            unsigned int prev = atomicAdd(ticket, 1u);
            is_last = (prev == gridDim.x - 1);
        }
    }
    __syncthreads();
    if (is_last) {
        __threadfence();
        float r = -1.0f;
        for (int i = tid; i < (int)gridDim.x; i += ABSMAX_THREADS) r = fmaxf(r, __ldcg(partials + i));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
        __syncthreads();
        if ((tid & 31) == 0) warp_max[tid >> 5] = r;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < ABSMAX_THREADS / 32; ++w) r = fmaxf(r, warp_max[w]);
            *out = r;
            *ticket = 0u;
        }
    }
}

static int codec_grid(const cn_context *ctx, int64_t n, int threads, int per_thread, int ctas_per_sm)
{
    int64_t need = (n + (int64_t)threads * per_thread - 1) / ((int64_t)threads * per_thread);
    int64_t cap = (int64_t)ctx->sm_count * ctas_per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

static int compress_impl(cn_context *ctx, const float *d_A, float precision, const float *d_precision, int64_t n,
                         uint8_t *d_codes, void *stream)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_compress_8bit: null context");
    CN_REQUIRE(n >= 0, CN_ERR_ARG, "cn_compress_8bit: negative size");
    if (n == 0) return CN_OK;
    CN_REQUIRE(d_A && d_codes, CN_ERR_ARG, "cn_compress_8bit: null buffer");
    int vector_ok = ((uintptr_t)d_A % 16 == 0) && ((uintptr_t)d_codes % 4 == 0);
    int grid = codec_grid(ctx, n, CODEC_THREADS, 4, 1);
    CodecConst cc;
    for (int i = 0; i < 128; ++i) { cc.thr[i] = ctx->h_thr[i]; cc.lc[i] = ctx->h_level_codes[i]; }
    if (d_precision)
        cn_compress_kernel<true><<<grid, CODEC_THREADS, 0, cn_stream(stream)>>>(d_A, 0.f, d_precision, n, d_codes, cc, vector_ok);
    else
        cn_compress_kernel<false><<<grid, CODEC_THREADS, 0, cn_stream(stream)>>>(d_A, precision, nullptr, n, d_codes, cc, vector_ok);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

extern "C" int cn_compress_8bit(cn_context *ctx, const float *d_A, float precision, int64_t n, uint8_t *d_codes, void *stream)
{
    return compress_impl(ctx, d_A, precision, nullptr, n, d_codes, stream);
}

extern "C" int cn_compress_8bit_dp(cn_context *ctx, const float *d_A, const float *d_precision, int64_t n, uint8_t *d_codes, void *stream)
{
    CN_REQUIRE(d_precision, CN_ERR_ARG, "cn_compress_8bit_dp: null precision pointer");
    return compress_impl(ctx, d_A, 0.f, d_precision, n, d_codes, stream);
}

static int decompress_impl(cn_context *ctx, const uint8_t *d_codes, float precision, const float *d_precision, int64_t n,
                           float *d_out, void *stream)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_decompress_8bit: null context");
    CN_REQUIRE(n >= 0, CN_ERR_ARG, "cn_decompress_8bit: negative size");
    if (n == 0) return CN_OK;
    CN_REQUIRE(d_out && d_codes, CN_ERR_ARG, "cn_decompress_8bit: null buffer");
    int vector_ok = ((uintptr_t)d_out % 16 == 0) && ((uintptr_t)d_codes % 4 == 0);
    int grid = codec_grid(ctx, n, CODEC_THREADS, 4, 1);   // 1024 threads x 64 registers fill an SM: one resident CTA
    DecodeConst dc;
    for (int i = 0; i < 128; ++i) dc.tbl[i] = ctx->h_tbl[i];
    if (d_precision)
        cn_decompress_kernel<true><<<grid, CODEC_THREADS, 0, cn_stream(stream)>>>(d_codes, 0.f, d_precision, n, d_out, dc, vector_ok);
    else
        cn_decompress_kernel<false><<<grid, CODEC_THREADS, 0, cn_stream(stream)>>>(d_codes, precision, nullptr, n, d_out, dc, vector_ok);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

extern "C" int cn_decompress_8bit(cn_context *ctx, const uint8_t *d_codes, float precision, int64_t n, float *d_out, void *stream)
{
    return decompress_impl(ctx, d_codes, precision, nullptr, n, d_out, stream);
}

extern "C" int cn_decompress_8bit_dp(cn_context *ctx, const uint8_t *d_codes, const float *d_precision, int64_t n, float *d_out, void *stream)
{
    CN_REQUIRE(d_precision, CN_ERR_ARG, "cn_decompress_8bit_dp: null precision pointer");
    return decompress_impl(ctx, d_codes, 0.f, d_precision, n, d_out, stream);
}

extern "C" int cn_absmax_f32(cn_context *ctx, const float *d_A, int64_t n, float *d_out, void *stream)
{
    CN_REQUIRE(ctx && d_out, CN_ERR_ARG, "cn_absmax_f32: null argument");
    CN_REQUIRE(n >= 0 && (n == 0 || d_A), CN_ERR_ARG, "cn_absmax_f32: bad input");
    int vector_ok = ((uintptr_t)d_A % 16 == 0);
    // measured: two CTAs per SM keep the last-ticket tail short on tensors of tens of MiB (64 MiB: 16.4 us vs 18.6 us with
    // four), eight per SM stream best on large ones (1 GiB: 6737 GB/s vs 6332)
    int grid = codec_grid(ctx, n, ABSMAX_THREADS, 16, n < (1LL << 27) ? 2 : 8);
    if (grid > CN_MAX_PARTIALS) grid = CN_MAX_PARTIALS;
    cn_absmax_kernel<true><<<grid, ABSMAX_THREADS, 0, cn_stream(stream)>>>(d_A, n, d_out, ctx->d_partials, ctx->d_ticket, vector_ok);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

// max() of the reference (source/basicOps.cu:1076-1081): thrust::reduce seeded with -1.0f, so the result is never below -1
extern "C" int cn_max_f32(cn_context *ctx, const float *d_A, int64_t n, float *d_out, void *stream)
{
    CN_REQUIRE(ctx && d_out, CN_ERR_ARG, "cn_max_f32: null argument");
    CN_REQUIRE(n >= 0 && (n == 0 || d_A), CN_ERR_ARG, "cn_max_f32: bad input");
    int vector_ok = ((uintptr_t)d_A % 16 == 0);
    int grid = codec_grid(ctx, n, ABSMAX_THREADS, 16, n < (1LL << 27) ? 2 : 8);
    if (grid > CN_MAX_PARTIALS) grid = CN_MAX_PARTIALS;
    cn_absmax_kernel<false><<<grid, ABSMAX_THREADS, 0, cn_stream(stream)>>>(d_A, n, d_out, ctx->d_partials, ctx->d_ticket, vector_ok);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

// ------------------------------------------------------------------------------------------------
// cn_absmax_f32_noalloc: absmax for callers that must not allocate.
//
// Some hosts cannot call cudaMalloc on the path where they need the scale of a tensor: real-time or plugin
// callbacks that are forbidden to take the allocator's lock (cudaMalloc may block and synchronise the device),
// processes that handed their whole device memory to another allocator at start-up, and recovery paths that run
// when device memory is already exhausted.
// cn_absmax_f32 needs a cn_context, whose creation allocates the scratch for the per-CTA partial maxima.  This entry
// point takes no context: the same kernel runs with its scratch in the fixed array below, which is part of the
// library image (every GPU that loads the library holds these 4352 bytes until the process exits).
//
// Consequences of the shared, fixed scratch:
//   * at most CN_ABSMAX_NOALLOC_MAX_CTAS partial maxima, and inputs of at most CN_ABSMAX_NOALLOC_MAX_N elements;
//     larger inputs are refused with CN_ERR_ARG;
//   * every call on a device uses the same array, so two calls that overlap on the GPU (different streams, or
//     different host threads) race; serialise them on one stream;
//   * the ticket word must be zero when a launch starts.  The array is zero when the module is loaded and the
//     kernel puts the ticket back to zero before it ends, so no clearing launch is needed between calls.
//
// In host code `g_absmax_noalloc_scratch` is only a handle of the device symbol, not an address the GPU can use:
// the set-up below asks the runtime for the device address with cudaGetSymbolAddress, once per device, with that
// device current, and the kernel receives that pointer.  The set-up happens inside the first call on a device;
// make that first call before starting any stream capture.
// ------------------------------------------------------------------------------------------------
#define CN_ABSMAX_NOALLOC_MAX_CTAS 1024
#define CN_ABSMAX_NOALLOC_MAX_N (1LL << 32)
#define CN_ABSMAX_NOALLOC_MAX_DEVICES 64

// [0, 1024): partial maxima (float bits); [1024]: ticket; rest: padding to a 256-byte multiple
static __device__ __align__(256) unsigned int g_absmax_noalloc_scratch[CN_ABSMAX_NOALLOC_MAX_CTAS + 64];

struct NoallocDevice {
    unsigned int *scratch = nullptr;   // device address of the array on this device
    int sm_count = 0;
};
static NoallocDevice g_noalloc_dev[CN_ABSMAX_NOALLOC_MAX_DEVICES];

extern "C" int cn_absmax_f32_noalloc(const float *d_A, int64_t n, float *d_out, void *stream)
{
    CN_REQUIRE(d_out, CN_ERR_ARG, "cn_absmax_f32_noalloc: null output pointer");
    CN_REQUIRE(n >= 0 && (n == 0 || d_A), CN_ERR_ARG, "cn_absmax_f32_noalloc: bad input");
    CN_REQUIRE(n <= CN_ABSMAX_NOALLOC_MAX_N, CN_ERR_ARG,
               "cn_absmax_f32_noalloc: %lld elements exceed the limit of %lld of the fixed scratch variant; use cn_absmax_f32",
               (long long)n, (long long)CN_ABSMAX_NOALLOC_MAX_N);
    int dev = -1;
    CN_CUDA(cudaGetDevice(&dev));
    CN_REQUIRE(dev >= 0 && dev < CN_ABSMAX_NOALLOC_MAX_DEVICES, CN_ERR_UNSUPPORTED, "cn_absmax_f32_noalloc: device index %d", dev);
    NoallocDevice &nd = g_noalloc_dev[dev];
    if (!nd.scratch) {
        // once per device, with that device current: device address of the symbol, and the SM count for the grid
        void *p = nullptr;
        CN_CUDA(cudaGetSymbolAddress(&p, g_absmax_noalloc_scratch));
        int sms = 0;
        CN_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        nd.sm_count = sms;
        nd.scratch = static_cast<unsigned int *>(p);
    }
    int64_t need = (n + (int64_t)ABSMAX_THREADS * 16 - 1) / ((int64_t)ABSMAX_THREADS * 16);
    int64_t cap = (int64_t)nd.sm_count * 4;
    if (cap > CN_ABSMAX_NOALLOC_MAX_CTAS) cap = CN_ABSMAX_NOALLOC_MAX_CTAS;
    if (need < 1) need = 1;
    const int grid = (int)(need < cap ? need : cap);
    const int vector_ok = ((uintptr_t)d_A % 16 == 0);
    cn_absmax_kernel<true><<<grid, ABSMAX_THREADS, 0, cn_stream(stream)>>>(d_A, n, d_out, reinterpret_cast<float *>(nd.scratch),
                                                                     nd.scratch + CN_ABSMAX_NOALLOC_MAX_CTAS, vector_ok);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}
