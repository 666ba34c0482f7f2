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
//
// Streaming.  For 16-byte aligned buffers the compressor (cn_compress_ring_kernel) stages its input through a
// shared-memory ring filled by bulk asynchronous copies (cp.async.bulk global -> shared, completion on mbarriers):
// one elected thread keeps six 32 KB tiles per SM in flight from the first microsecond, independently of what the
// 1024 coding threads are doing, so the depth of the prefetch does not cost registers and the table build overlaps the
// first loads.  The coding threads read the staged tile with conflict-free 16-byte shared loads.
//
// Launch overlap.  All codec kernels are launched with programmatic stream serialisation: each kernel lets its
// successor start as soon as it is resident (griddepcontrol.launch_dependents), does everything that needs no global
// memory (barrier set-up, and the table build when the scale came from the host) and only then waits for the
// predecessor to finish (griddepcontrol.wait) - before its first access to global memory.  In a series of codec
// calls the launch latency, the CTA start-up and the table build of call i+1 then overlap the tail of call i.
#include <math.h>
#include <string.h>
#include "cn_internal.h"

#define CODEC_THREADS 1024
#define ABSMAX_THREADS 512
#define LUT_SHIFT 16
#define LUT_MAX 2816

// Programmatic dependent launch: "my successor in the stream may start" / "my predecessor has finished and its writes are
// visible".  Without the launch attribute both are no-ops.
__device__ __forceinline__ void cdc_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void cdc_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

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
    cdc_pdl_launch_dependents();
    cdc_pdl_wait();
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


// ---------------------------------------------------------------------------------------------- ring compressor
#define RING_THREADS 512                    // two CTAs per SM
#define RING_TILE 8192                      // elements per tile: 32 KB of input, four 16-byte groups per thread
#define RING_STAGES 3                       // per CTA: 6 tiles = 192 KB in flight per SM
#define RING_GROUPS_PER_THREAD (RING_TILE / 4 / RING_THREADS)
#define CN_FUSED_ABSMAX_MAX_N (4LL << 20)   // above this size cn_absmax_compress_8bit issues two launches
#define RING_WAIT_LIMIT (4000000000LL)      // clock cycles (~2 s)

__device__ __forceinline__ uint32_t cdc_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cdc_mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void cdc_mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cdc_mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t cdc_mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done;
}
// Bounded wait: false when the limit ran out (the caller stops streaming and reports through *status).
__device__ __forceinline__ bool cdc_mbar_wait(uint32_t bar, uint32_t parity, unsigned int *status)
{
    if (cdc_mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (cdc_mbar_try(bar, parity)) return true;
        if ((it & 255u) == 0u && clock64() - t0 > RING_WAIT_LIMIT) {
            if (status) atomicMax(status, 12u);
            return false;
        }
    }
}
__device__ __forceinline__ void cdc_bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// Per-launch tables of the ring compressor.  The magnitudes are looked up in a shifted and clamped domain,
//     c = clamp(|x| bits + delta - lo, 0, hi - lo),
// with delta (< 65536) chosen so that the boundary of the top level (code 127) falls exactly on the start of a bucket
// (the top level then owns whole buckets and never shares one with its close neighbour), lo = start of a bucket that
// lies entirely below the first boundary and hi = start of the top level's bucket.  The clamp is one instruction
// (min.relu.s32).  One 4-byte entry per bucket of 65536 consecutive c: bits 31..16 = low 16 bits of the boundary inside
// the bucket (0 = none: every c of the bucket counts as "at or above"), bits 15..8 = code at and above the boundary,
// bits 7..0 = code below it; c is compared as (c << 16 | 0xffff) >= entry.
// Two resources bound the stream next to HBM: the integer pipe (64 lanes per SM and clock against 128 for fp32) and the
// shared-memory pipe (the table reads of a warp hit random banks: ~4 wavefronts per read).  Hence 4-byte entries, and
// a per-element sequence of: and, add, min.relu, shift, address, shared load, multiply-add (the compare key, on the
// fp32/imad pipe), compare, predicated shift.
struct RingTables {
    uint32_t lut[LUT_MAX];
    uint32_t X[128];        // boundaries in |x| space (bit patterns); [126] = top level, [127] = pad
    uint32_t T[128];        // thresholds in |x/precision| space (generic path)
    uint32_t lc[128];       // level codes
    uint32_t kadd;          // delta - lo (mod 2^32)
    int32_t span;           // hi - lo
    int nb, bad;
};

// Boundaries found on the host for a host-side scale (same IEEE arithmetic), or left to the kernel (device scale).
struct RingConst {
    uint32_t thr[128];
    uint32_t lc[128];
    uint32_t X[128];
    int x_valid;            // X holds the boundaries for this launch's precision
};

__device__ __forceinline__ uint32_t ring_generic(float x, float p, const RingTables &t)
{
    float a = __fdiv_rn(x, p);
    if (a != a) return 1u;
    const bool neg = a < 0.0f;
    const uint32_t ab = __float_as_uint(a) & 0x7fffffffu;
    const uint32_t c = t.lc[count_le(t.T, ab)];
    return (neg && c != 254u) ? (c | 0x80u) : c;
}

// code of one magnitude (low byte of the result; the bytes above are not meaningful): finite or infinite input
__device__ __forceinline__ uint32_t ring_lookup(uint32_t xbits, uint32_t kadd, int32_t span, uint32_t lut_addr)
{
    const int32_t w = (int32_t)((xbits & 0x7fffffffu) + kadd);
    int32_t c;
    asm("min.relu.s32 %0, %1, %2;" : "=r"(c) : "r"(w), "r"(span));
    uint32_t bucket, e, key;
    asm("shr.u32 %0, %1, 16;" : "=r"(bucket) : "r"(c));             // kept apart from the scaling below: index * 4 + base is an addressing mode
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(e) : "r"(bucket * 4u + lut_addr));
    asm("mad.lo.u32 %0, %1, 65536, 65535;" : "=r"(key) : "r"(c));   // (c << 16) | 0xffff
    asm("{\n\t.reg .pred p;\n\tsetp.ge.u32 p, %1, %0;\n\t@p shr.u32 %0, %0, 8;\n\t}" : "+r"(e) : "r"(key));
    return e;
}

__device__ __forceinline__ uint32_t ring_code(uint32_t xb, uint32_t pb, uint32_t kadd, int32_t span, uint32_t lut_addr)
{
    if ((xb & 0x7fffffffu) > 0x7f800000u) return 1u;      // NaN: the reference's search ends on index 1, sign clear
    return (ring_lookup(xb, kadd, span, lut_addr) & 0xffu) | (((xb ^ pb) >> 24) & 0x80u);
}

// four codes for one 16-byte group.  A NaN anywhere in the group (rare) sends it through the per-element form; the test
// is a floating-point sum (x != x for the sum: NaN inputs, and +inf with -inf, which the per-element form codes
// correctly as well), which keeps it off the integer pipe.
template <bool NEGP>
__device__ __forceinline__ uint32_t ring_code4(const float4 q, uint32_t pb, uint32_t kadd, int32_t span, uint32_t lut_addr)
{
    const uint32_t x0 = __float_as_uint(q.x), x1 = __float_as_uint(q.y), x2 = __float_as_uint(q.z), x3 = __float_as_uint(q.w);
    const float sum = (q.x + q.y) + (q.z + q.w);
    if (sum != sum)
        return pack4(ring_code(x0, pb, kadd, span, lut_addr), ring_code(x1, pb, kadd, span, lut_addr),
                     ring_code(x2, pb, kadd, span, lut_addr), ring_code(x3, pb, kadd, span, lut_addr));
    const uint32_t c0 = ring_lookup(x0, kadd, span, lut_addr), c1 = ring_lookup(x1, kadd, span, lut_addr);
    const uint32_t c2 = ring_lookup(x2, kadd, span, lut_addr), c3 = ring_lookup(x3, kadd, span, lut_addr);
    // top bytes of x0..x3 -> one word; keep bit 7 of each byte, flipped when precision is negative (code 254 has the bit set
    // already); one three-input logic operation either way
    const uint32_t tops = __byte_perm(__byte_perm(x0, x1, 0x0073), __byte_perm(x2, x3, 0x0073), 0x5410);
    const uint32_t codes = pack4(c0, c1, c2, c3);
    return NEGP ? (codes | (~tops & 0x80808080u)) : (codes | (tops & 0x80808080u));
}

// Shift, clamp range and bucket table from the 127 boundaries in t.X (all threads of the CTA; ends with a barrier).
__device__ __forceinline__ void ring_build_tables(RingTables &t, int tid, bool usable)
{
    __shared__ uint32_t s_delta;
    __shared__ int s_base;
    if (tid < 32) {
        bool bad = !usable;
        for (int k = 0; k < 4; ++k) {
            const int idx = tid + 32 * k;
            if (idx < CN_NUM_THR && t.X[idx] >= 0x7f800000u) bad = true;   // unpinned (0xfffffffe) or not finite
        }
        bad = __any_sync(0xffffffffu, bad);
        if (tid == 0) {
            const uint32_t xtop = t.X[CN_NUM_THR - 1];
            const uint32_t delta = ((xtop + 0xffffu) & 0xffff0000u) - xtop;
            const uint32_t hi = xtop + delta;
            const int base = (int)((t.X[0] + delta) >> 16) - 1;       // bucket 0 lies entirely below the first boundary
            const int nb = (int)(hi >> 16) - base + 1;
            const uint32_t lo = (uint32_t)base << 16;
            s_delta = delta;
            s_base = base;
            t.kadd = delta - lo;
            t.span = (int32_t)(hi - lo);
            t.nb = nb;
            t.bad = (bad || base < 1 || nb > LUT_MAX || nb < 3) ? 1 : 0;
        }
    }
    __syncthreads();
    if (!t.bad) {
        const int base = s_base, nb = t.nb;
        const uint32_t delta = s_delta;
        for (int b = tid; b < nb; b += RING_THREADS) {
            const uint32_t kbv = (uint32_t)(b + base);
            // first boundary (of 0..126) whose shifted bucket is >= this one
            int first = 0;
#pragma unroll
            for (int step2 = 64; step2 > 0; step2 >>= 1)
                if (first + step2 - 1 < CN_NUM_THR && ((t.X[first + step2 - 1] + delta) >> 16) < kbv) first += step2;
            uint32_t e;
            if (first < CN_NUM_THR && ((t.X[first] + delta) >> 16) == kbv) {
                e = ((t.X[first] + delta) << 16) | (t.lc[first + 1] << 8) | t.lc[first];
                if (first + 1 < CN_NUM_THR && ((t.X[first + 1] + delta) >> 16) == kbv) atomicOr(&t.bad, 1);   // two boundaries in one bucket
            } else {
                e = (t.lc[first] << 8) | t.lc[first];
            }
            t.lut[b] = e;
        }
    }
    __syncthreads();
}

// Grid-wide barrier of a cooperative launch (all CTAs resident).  Two words in device memory, nothing on the host, so a
// launch that was recorded in a CUDA graph can be replayed: every CTA reads the generation, adds one to the arrival
// count, and the CTA that arrives last clears the count and advances the generation, which releases the others.  The wait
// has a clock limit; a wait that runs out records status 13 and lets the CTA go on, so the kernel always ends (its
// output is then undefined).  One kernel at a time may use a pair of words (launches of one context are stream-ordered).
__device__ __forceinline__ void cdc_grid_barrier(unsigned int *arrive, unsigned int *generation, unsigned int *status)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int gen, seen;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(gen) : "l"(generation) : "memory");
        __threadfence();
        if (atomicAdd(arrive, 1u) == gridDim.x - 1) {
            *reinterpret_cast<volatile unsigned int *>(arrive) = 0u;
            __threadfence();
            atomicAdd(generation, 1u);
        } else {
            const long long t0 = clock64();
            for (;;) {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(generation) : "memory");
                if (seen != gen) break;
                if (clock64() - t0 > RING_WAIT_LIMIT) { if (status) atomicMax(status, 13u); break; }
                __nanosleep(40);
            }
        }
        __threadfence();
    }
    __syncthreads();
}

enum { RING_SCALE_HOST = 0, RING_SCALE_DEVICE = 1, RING_SCALE_ABSMAX = 2 };

// Work split: every CTA codes the same number of tiles (tiles_per_cta) of the same size (tile_groups 16-byte groups,
// at most RING_TILE / 4), chosen on the host so that grid * tiles_per_cta tiles cover the tensor with less than one
// group of slack per tile; tile j goes to CTA j % grid.  The last tiles may be short or missing.
//
// SCALE = RING_SCALE_ABSMAX is the fused form of "scale = absmax(A); codes = compress(A, scale)" (cooperative launch):
// pass 1 reduces |A| over the CTA's own tiles with plain loads that leave the lines in L2, a grid barrier publishes the
// per-CTA maxima, every CTA folds them, and pass 2 codes the CTA's tiles in reverse order - most recently read first -
// so that a tensor that fits the L2 is read from HBM once.  d_precision then receives the scale.
template <int SCALE>
__global__ void __launch_bounds__(RING_THREADS, 2)
cn_compress_ring_kernel(const float *__restrict__ A, float precision_arg, float *__restrict__ d_precision,
                        int64_t n, uint8_t *__restrict__ out, const __grid_constant__ RingConst rc, unsigned int *status,
                        int tile_groups, int tiles_per_cta, float *__restrict__ partials, unsigned int *barrier_words,
                        int input_ready_before_predecessor)
{
    extern __shared__ __align__(128) uint8_t ring_smem[];
    __shared__ RingTables t;
    __shared__ __align__(8) uint64_t bars[2 * RING_STAGES];
    __shared__ float s_red[RING_THREADS / 32];
    const int tid = threadIdx.x;
    const uint32_t ring_base = (cdc_smem_u32(ring_smem) + 127u) & ~127u;
    const uint8_t *ring_gen = ring_smem + (ring_base - cdc_smem_u32(ring_smem));
    auto full_bar = [&](int s) { return cdc_smem_u32(&bars[s]); };
    auto empty_bar = [&](int s) { return cdc_smem_u32(&bars[RING_STAGES + s]); };

    if (tid == 0) {
        for (int s = 0; s < RING_STAGES; ++s) { cdc_mbar_init(full_bar(s), 1); cdc_mbar_init(empty_bar(s), RING_THREADS / 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    cdc_pdl_launch_dependents();
    if (tid < 128) {
        t.T[tid] = rc.thr[tid];
        t.lc[tid] = rc.lc[tid];
        if (SCALE == RING_SCALE_HOST) t.X[tid] = rc.X[tid];
    }
    const int64_t groups_total = n >> 2;                    // 16-byte groups of the tensor
    // tiles of this CTA that hold data: tile (blockIdx.x + k * gridDim.x), k = 0 .. my_tiles - 1
    int my_tiles = 0;
    {
        const int64_t tiles_total = (groups_total + tile_groups - 1) / tile_groups;
        if ((int64_t)blockIdx.x < tiles_total) {
            const int64_t mine = (tiles_total - blockIdx.x + gridDim.x - 1) / gridDim.x;
            my_tiles = (int)(mine < tiles_per_cta ? mine : tiles_per_cta);
        }
    }
    // the i-th tile this CTA codes (pass 2 of the fused form walks its tiles backwards) and its size in 16-byte groups
    auto tile_of = [&](int i) { return (int64_t)blockIdx.x + (int64_t)(SCALE == RING_SCALE_ABSMAX ? my_tiles - 1 - i : i) * gridDim.x; };
    auto tile_count = [&](int64_t j) {
        const int64_t left = groups_total - j * tile_groups;
        return (int)(left < tile_groups ? left : tile_groups);
    };
    __syncthreads();   // barriers initialised, constant tables in shared memory

    // input_ready_before_predecessor: the launch directly before this one in the stream is this library's absmax of the
    // same tensor (cn_absmax_compress_8bit): it does not write A, and it released this kernel only after everything
    // before it had finished, so A may be loaded already - the ring fills while absmax drains.  Only the scale needs the wait.
    auto fill_ring = [&]() {
        for (int i = 0; i < RING_STAGES && i < my_tiles; ++i) {
            const int64_t j = tile_of(i);
            const uint32_t bytes = (uint32_t)tile_count(j) * 16u;
            cdc_mbar_expect_tx(full_bar(i), bytes);
            cdc_bulk_load(ring_base + (uint32_t)i * (RING_TILE * 4), A + j * tile_groups * 4, bytes, full_bar(i));
        }
    };
    if (SCALE == RING_SCALE_DEVICE && input_ready_before_predecessor && tid == 0) fill_ring();
    // ---- everything below may touch global memory: the predecessor in the stream must have finished
    cdc_pdl_wait();
    float p = precision_arg;
    if (SCALE == RING_SCALE_ABSMAX) {
        // pass 1: maximum of |A| over this CTA's tiles (and, in CTA 0, the last n % 4 elements)
        float m = -1.0f;   // seed of the reference's reduction (source/basicOps.cu:1079)
        const float4 *A4 = reinterpret_cast<const float4 *>(A);
        for (int k = 0; k < my_tiles; ++k) {
            const int64_t j = (int64_t)blockIdx.x + (int64_t)k * gridDim.x;
            const int groups = tile_count(j);
            const float4 *src = A4 + j * tile_groups;
            float4 q[RING_GROUPS_PER_THREAD];
#pragma unroll
            for (int u = 0; u < RING_GROUPS_PER_THREAD; ++u)
                q[u] = (tid + u * RING_THREADS < groups) ? src[tid + u * RING_THREADS] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < RING_GROUPS_PER_THREAD; ++u)
                if (tid + u * RING_THREADS < groups)
                    m = fmaxf(m, fmaxf(fmaxf(fabsf(q[u].x), fabsf(q[u].y)), fmaxf(fabsf(q[u].z), fabsf(q[u].w))));
        }
        if (blockIdx.x == 0 && tid < (int)(n - (groups_total << 2))) m = fmaxf(m, fabsf(A[(groups_total << 2) + tid]));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if ((tid & 31) == 0) s_red[tid >> 5] = m;
        __syncthreads();
        if (tid < 32) {
            m = tid < RING_THREADS / 32 ? s_red[tid] : -1.0f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
            if (tid == 0) partials[blockIdx.x] = m;
        }
        cdc_grid_barrier(barrier_words, barrier_words + 1, status);
    }
    // fill the ring before anything else: the first loads are in flight while the tables are built
    if (tid == 0 && !(SCALE == RING_SCALE_DEVICE && input_ready_before_predecessor)) fill_ring();
    if (SCALE == RING_SCALE_DEVICE) p = *d_precision;
    if (SCALE == RING_SCALE_ABSMAX) {
        // every CTA folds the per-CTA maxima (the same values in the same order everywhere)
        float m = -1.0f;
        for (int i = tid; i < (int)gridDim.x; i += RING_THREADS) m = fmaxf(m, __ldcg(partials + i));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        __syncthreads();   // s_red was read above
        if ((tid & 31) == 0) s_red[tid >> 5] = m;
        __syncthreads();
        m = s_red[0];
#pragma unroll
        for (int w = 1; w < RING_THREADS / 32; ++w) m = fmaxf(m, s_red[w]);
        p = m;
        if (blockIdx.x == 0 && tid == 0) *d_precision = p;
    }
    const uint32_t pb = __float_as_uint(p);
    const float ap = fabsf(p);
    // 2^-100 <= |p| <= 2^100 keeps every boundary T*|p| a normal number; NaN fails both tests
    const bool p_ok = (ap >= 7.8886090522101181e-31f) && (ap <= 1.2676506002282294e30f);
    if (SCALE == RING_SCALE_HOST) {
        ring_build_tables(t, tid, rc.x_valid && p_ok);   // boundaries came with the launch (found on the host)
    } else {
        if (tid < 128) {
            // smallest |x| with fl(|x|/|p|) >= T for each of the 127 thresholds (see cn_compress_kernel)
            uint32_t xb = 0xffffffffu;
            bool good = true;
            if (tid < CN_NUM_THR && p_ok) {
                const float T = __uint_as_float(rc.thr[tid]);
                xb = __float_as_uint(__fmul_rn(T, ap));
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
            t.X[tid] = good ? xb : 0xfffffffeu;
        }
        __syncthreads();
        ring_build_tables(t, tid, p_ok);
    }
    const bool fast = t.bad == 0;
    const uint32_t kadd = t.kadd;
    const int32_t span = t.span;
    const uint32_t lut_addr = cdc_smem_u32(t.lut);

    uint32_t *out4 = reinterpret_cast<uint32_t *>(out);
    bool ok = true;
    for (int i = 0; i < my_tiles && ok; ++i) {
        const int s = i % RING_STAGES;
        const uint32_t ph = (uint32_t)(i / RING_STAGES) & 1u;
        if (tid == 0 && i >= 1 && i - 1 + RING_STAGES < my_tiles) {
            // refill the stage that every warp finished in the previous iteration
            const int ps = (i - 1) % RING_STAGES;
            const uint32_t pph = (uint32_t)((i - 1) / RING_STAGES) & 1u;
            const int64_t j = tile_of(i - 1 + RING_STAGES);
            const uint32_t bytes = (uint32_t)tile_count(j) * 16u;
            if (cdc_mbar_wait(empty_bar(ps), pph, status)) {
                cdc_mbar_expect_tx(full_bar(ps), bytes);
                cdc_bulk_load(ring_base + (uint32_t)ps * (RING_TILE * 4), A + j * tile_groups * 4, bytes, full_bar(ps));
            }
        }
        const int64_t j = tile_of(i);
        const int groups = tile_count(j);
        ok = cdc_mbar_wait(full_bar(s), ph, status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const float4 *src = reinterpret_cast<const float4 *>(ring_gen + (size_t)s * (RING_TILE * 4));
        uint32_t *dst = out4 + j * tile_groups;
        if (fast) {
            // table path: all loads of the thread first, then the lookups of its (up to) four groups interleave.  Whole
            // tiles (the common case: the host prefers them) need no per-thread bounds
            float4 q[RING_GROUPS_PER_THREAD];
            if (groups == RING_TILE / 4) {
#pragma unroll
                for (int u = 0; u < RING_GROUPS_PER_THREAD; ++u) q[u] = src[tid + u * RING_THREADS];
                if (pb >> 31) {
#pragma unroll
                    for (int u = 0; u < RING_GROUPS_PER_THREAD; ++u) __stcs(dst + tid + u * RING_THREADS, ring_code4<true>(q[u], pb, kadd, span, lut_addr));
                } else {
#pragma unroll
                    for (int u = 0; u < RING_GROUPS_PER_THREAD; ++u) __stcs(dst + tid + u * RING_THREADS, ring_code4<false>(q[u], pb, kadd, span, lut_addr));
                }
            } else {
#pragma unroll
                for (int u = 0; u < RING_GROUPS_PER_THREAD; ++u)
                    if (tid + u * RING_THREADS < groups) q[u] = src[tid + u * RING_THREADS];
#pragma unroll
                for (int u = 0; u < RING_GROUPS_PER_THREAD; ++u)
                    if (tid + u * RING_THREADS < groups)
                        __stcs(dst + tid + u * RING_THREADS, (pb >> 31) ? ring_code4<true>(q[u], pb, kadd, span, lut_addr)
                                                                        : ring_code4<false>(q[u], pb, kadd, span, lut_addr));
            }
        } else {
#pragma unroll 1
            for (int g = tid; g < groups; g += RING_THREADS) {
                const float4 q = src[g];
                __stcs(dst + g, pack4(ring_generic(q.x, p, t), ring_generic(q.y, p, t), ring_generic(q.z, p, t), ring_generic(q.w, p, t)));
            }
        }
        __syncwarp();
        if ((tid & 31) == 0) cdc_mbar_arrive(empty_bar(s));
    }
    if (!ok && tid == 0) {
        // a wait ran out: give the copies that are still in flight a bounded chance to land before the CTA exits
        for (int s = 0; s < RING_STAGES; ++s) {
            const long long t0 = clock64();
            while (!cdc_mbar_try(full_bar(s), 0u) && !cdc_mbar_try(full_bar(s), 1u) && clock64() - t0 < 20000000LL) {}
        }
    }
    // the last n % 4 elements
    const int64_t n4 = groups_total << 2;
    if (blockIdx.x == 0 && tid < (int)(n - n4)) {
        const float x = A[n4 + tid];
        out[n4 + tid] = (uint8_t)(fast ? ring_code(__float_as_uint(x), pb, kadd, span, lut_addr) : ring_generic(x, p, t));
    }
}

// ---- code and push in one launch (the gradient exchange of small tensors)
//
// scale = absmax(A); codes = compress(A, scale) as in the fused form above, but the codes (and the scale) go to this
// rank's block AND to the same place in every peer's area, framed by the two flag exchanges of the pushed block exchange:
// CTA 0 tells the peers "my area may be written" when the kernel starts (everything queued before it has finished), every
// CTA waits (bounded) for the peers' flags after the grid barrier - the first pass hides the round trip - and the CTA that
// finishes last tells the peers "my block has arrived" and waits for theirs.  Tensors of this size (at most 4 Mi
// elements) stay in L2 between the passes, so the second pass reads with plain loads.  Stores to the peers are 4-byte
// words that a warp lays down 128 contiguous bytes at a time; no multicast.
__device__ __forceinline__ bool push_wait_flags(const unsigned int *local_flags, int slot, int nranks, int my_rank, unsigned int epoch,
                                                unsigned int *status)
{
    bool ok = true;
    const int r = threadIdx.x;
    if (r < nranks && r != my_rank) {
        const volatile unsigned int *f = local_flags + slot * nranks + r;
        const long long t0 = clock64();
        while ((int)(*f - epoch) < 0) {
            if (clock64() - t0 > RING_WAIT_LIMIT) { atomicMax(status, 10u); ok = false; break; }
            __nanosleep(100);
        }
        __threadfence_system();
    }
    return __syncthreads_and(ok);
}

__global__ void __launch_bounds__(RING_THREADS, 2)
cn_absmax_compress_push_kernel(const float *__restrict__ A, int64_t n, float *__restrict__ scale_out, uint8_t *__restrict__ out,
                               const __grid_constant__ RingConst rc, unsigned int *status, float *__restrict__ partials,
                               unsigned int *barrier_words, const __grid_constant__ cn_codec_push cp)
{
    __shared__ RingTables t;
    __shared__ float s_red[RING_THREADS / 32];
    __shared__ int s_last;
    const int tid = threadIdx.x;
    if (tid < 128) {
        t.T[tid] = rc.thr[tid];
        t.lc[tid] = rc.lc[tid];
    }
    const unsigned int epoch = *reinterpret_cast<volatile unsigned int *>(cp.state) + 1u;   // advanced by the last CTA, at the very end
    if (blockIdx.x == 0 && tid < cp.nranks && tid != cp.my_rank) {
        __threadfence_system();
        *reinterpret_cast<volatile unsigned int *>(cp.peer_flags[tid] + cp.slot * cp.nranks + cp.my_rank) = epoch;
    }
    const int64_t groups_total = n >> 2, n4 = groups_total << 2;
    const int64_t stride = (int64_t)gridDim.x * RING_THREADS, g0 = (int64_t)blockIdx.x * RING_THREADS + tid;
    const float4 *A4 = reinterpret_cast<const float4 *>(A);
    // pass 1: maximum of |A|
    float m = -1.0f;   // seed of the reference's reduction (source/basicOps.cu:1079)
#pragma unroll 4
    for (int64_t g = g0; g < groups_total; g += stride) {
        const float4 q = A4[g];
        m = fmaxf(m, fmaxf(fmaxf(fabsf(q.x), fabsf(q.y)), fmaxf(fabsf(q.z), fabsf(q.w))));
    }
    if (blockIdx.x == 0 && tid < (int)(n - n4)) m = fmaxf(m, fabsf(A[n4 + tid]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31) == 0) s_red[tid >> 5] = m;
    __syncthreads();
    if (tid < 32) {
        m = tid < RING_THREADS / 32 ? s_red[tid] : -1.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (tid == 0) partials[blockIdx.x] = m;
    }
    cdc_grid_barrier(barrier_words, barrier_words + 1, status);
    // every CTA folds the per-CTA maxima (the same values in the same order everywhere)
    m = -1.0f;
    for (int i = tid; i < (int)gridDim.x; i += RING_THREADS) m = fmaxf(m, __ldcg(partials + i));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    __syncthreads();   // s_red was read above
    if ((tid & 31) == 0) s_red[tid >> 5] = m;
    __syncthreads();
    m = s_red[0];
#pragma unroll
    for (int w = 1; w < RING_THREADS / 32; ++w) m = fmaxf(m, s_red[w]);
    const float p = m;
    const uint32_t pb = __float_as_uint(p);
    const float ap = fabsf(p);
    const bool p_ok = (ap >= 7.8886090522101181e-31f) && (ap <= 1.2676506002282294e30f);
    if (tid < 128) {
        // smallest |x| with fl(|x|/|p|) >= T for each of the 127 thresholds (see cn_compress_kernel)
        uint32_t xb = 0xffffffffu;
        bool good = true;
        if (tid < CN_NUM_THR && p_ok) {
            const float T = __uint_as_float(rc.thr[tid]);
            xb = __float_as_uint(__fmul_rn(T, ap));
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
        t.X[tid] = good ? xb : 0xfffffffeu;
    }
    __syncthreads();
    ring_build_tables(t, tid, p_ok);
    const bool fast = t.bad == 0;
    const uint32_t kadd = t.kadd;
    const int32_t span = t.span;
    const uint32_t lut_addr = cdc_smem_u32(t.lut);
    // the peers' areas may be written once every peer has said so
    const bool may_write = push_wait_flags(cp.local_flags, cp.slot, cp.nranks, cp.my_rank, epoch, status);
    if (blockIdx.x == 0 && tid == 0) {
        *scale_out = p;
        if (may_write)
            for (int d = 0; d < cp.ndst; ++d) *cp.scale_dst[d] = p;
    }
    // pass 2: code; this CTA's groups in reverse order (most recently read first)
    uint32_t *out4 = reinterpret_cast<uint32_t *>(out);
    const int ndst = may_write ? cp.ndst : 0;
    if (g0 < groups_total) {
        const int64_t last = g0 + (groups_total - 1 - g0) / stride * stride;
        for (int64_t g = last; g >= g0; g -= stride) {
            const float4 q = A4[g];
            uint32_t w;
            if (fast) w = (pb >> 31) ? ring_code4<true>(q, pb, kadd, span, lut_addr) : ring_code4<false>(q, pb, kadd, span, lut_addr);
            else w = pack4(ring_generic(q.x, p, t), ring_generic(q.y, p, t), ring_generic(q.z, p, t), ring_generic(q.w, p, t));
            out4[g] = w;
#pragma unroll 1
            for (int d = 0; d < ndst; ++d) reinterpret_cast<uint32_t *>(cp.codes_dst[d])[g] = w;
        }
    }
    if (blockIdx.x == 0 && tid < (int)(n - n4)) {
        const float x = A[n4 + tid];
        const uint8_t c = (uint8_t)(fast ? ring_code(__float_as_uint(x), pb, kadd, span, lut_addr) : ring_generic(x, p, t));
        out[n4 + tid] = c;
        for (int d = 0; d < ndst; ++d) cp.codes_dst[d][n4 + tid] = c;
    }
    // the CTA that finishes last closes the exchange
    __threadfence_system();
    __syncthreads();
    if (tid == 0) s_last = (atomicAdd(barrier_words, 1u) == gridDim.x - 1) ? 1 : 0;   // the arrival count is zero again after the barrier
    __syncthreads();
    if (!s_last) return;
    if (tid == 0) *reinterpret_cast<volatile unsigned int *>(barrier_words) = 0u;
    __threadfence_system();
    if (may_write && tid < cp.nranks && tid != cp.my_rank)
        *reinterpret_cast<volatile unsigned int *>(cp.peer_flags[tid] + (cp.slot + 1) * cp.nranks + cp.my_rank) = epoch;
    if (may_write) push_wait_flags(cp.local_flags, cp.slot + 1, cp.nranks, cp.my_rank, epoch, status);
    __syncthreads();
    if (tid == 0) {
        *cp.state = epoch;
        __threadfence();
    }
}

// kDecompression_8bit (source/clusterKernels.cu:1135-1160): 256-entry table built in the reference's
// statement order, then out[i] = table[code].
// vector_ok: 0 = byte by byte; 1 = four codes per load (codes 4-byte, output 16-byte aligned).  When the codes are 16-byte
// aligned too, cn_decompress16_kernel takes over: a warp reads 512 consecutive codes with one 16-byte load per lane and writes the 2048
// bytes they decode to with four store instructions of 512 consecutive bytes each - word j of lane l holds float4
// number 4l + j of the warp's 128, store k of lane l writes number 32k + l, fetched from lane 8k + l/4 by shuffles.
// Used for large tensors (see decompress_impl).
template <bool PRECISION_ON_DEVICE>
__global__ void __launch_bounds__(CODEC_THREADS, 1)
cn_decompress_kernel(const uint8_t *__restrict__ codes, float precision_arg, const float *__restrict__ d_precision,
                     int64_t n, float *__restrict__ out, const __grid_constant__ DecodeConst dc, int vector_ok)
{
    __shared__ float lut[256];
    const int tid = threadIdx.x;
    cdc_pdl_launch_dependents();
    if (PRECISION_ON_DEVICE) cdc_pdl_wait();   // the scale is in global memory; a host scale lets the table precede the wait
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
    if (!PRECISION_ON_DEVICE) cdc_pdl_wait();
    __syncthreads();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    float4 *out4 = reinterpret_cast<float4 *>(out);
#define CN_DEC4(w) make_float4(lut[(w) & 0xffu], lut[((w) >> 8) & 0xffu], lut[((w) >> 16) & 0xffu], lut[(w) >> 24])
    const int64_t nvec = vector_ok ? (n >> 2) : 0;
    int64_t v = (int64_t)blockIdx.x * blockDim.x + tid;
    const uint32_t *in4 = reinterpret_cast<const uint32_t *>(codes);
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

template <bool PRECISION_ON_DEVICE>
__global__ void __launch_bounds__(CODEC_THREADS, 2)
cn_decompress16_kernel(const uint8_t *__restrict__ codes, float precision_arg, const float *__restrict__ d_precision,
                       int64_t n, float *__restrict__ out, const __grid_constant__ DecodeConst dc)
{
    __shared__ float lut[256];
    const int tid = threadIdx.x;
    cdc_pdl_launch_dependents();
    if (PRECISION_ON_DEVICE) cdc_pdl_wait();   // the scale is in global memory; a host scale lets the table precede the wait
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
    if (!PRECISION_ON_DEVICE) cdc_pdl_wait();
    __syncthreads();
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    float4 *out4 = reinterpret_cast<float4 *>(out);
#define CN_DEC4(w) make_float4(lut[(w) & 0xffu], lut[((w) >> 8) & 0xffu], lut[((w) >> 16) & 0xffu], lut[(w) >> 24])
    const int64_t n16 = (n >> 4) & ~(int64_t)31;   // whole warps only: the shuffles need all 32 lanes
    const uint4 *in16 = reinterpret_cast<const uint4 *>(codes);
    const int lane = tid & 31, j = lane & 3;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + tid; v < n16; v += stride) {
        const uint4 w = __ldcs(in16 + v);
        const int64_t base = (v - lane) << 2;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int src = 8 * k + (lane >> 2);
            const uint32_t a = __shfl_sync(0xffffffffu, w.x, src), b = __shfl_sync(0xffffffffu, w.y, src),
                           c = __shfl_sync(0xffffffffu, w.z, src), d = __shfl_sync(0xffffffffu, w.w, src);
            const uint32_t x = j == 0 ? a : j == 1 ? b : j == 2 ? c : d;
            __stcs(out4 + base + 32 * k + lane, CN_DEC4(x));
        }
    }
#undef CN_DEC4
    for (int64_t i = (n16 << 4) + (int64_t)blockIdx.x * blockDim.x + tid; i < n; i += stride) out[i] = lut[codes[i]];
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
    // wait first, then release the successor: a kernel that follows absmax in the stream may then rely on everything
    // before absmax having finished (cn_absmax_compress_8bit's compressor starts loading A before its own wait)
    cdc_pdl_wait();
    cdc_pdl_launch_dependents();
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

// absmax through the same bulk-copy ring as the compressor (16-byte aligned input): the elected thread keeps three 32 KB
// tiles per CTA (two CTAs per SM) in flight, so the bytes in flight do not depend on how many loads each thread can
// hold in registers - at a few tens of MiB, where every microsecond of ramp shows, this is what keeps HBM busy.
// Same partial-maximum + last-ticket fold as cn_absmax_kernel; work split as in cn_compress_ring_kernel.
__global__ void __launch_bounds__(RING_THREADS, 2)
cn_absmax_ring_kernel(const float *__restrict__ A, int64_t n, float *__restrict__ out, float *__restrict__ partials,
                      unsigned int *__restrict__ ticket, unsigned int *status, int tile_groups, int tiles_per_cta)
{
    extern __shared__ __align__(128) uint8_t ring_smem[];
    __shared__ __align__(8) uint64_t bars[2 * RING_STAGES];
    __shared__ float warp_max[RING_THREADS / 32];
    __shared__ bool is_last;
    const int tid = threadIdx.x;
    const uint32_t ring_base = (cdc_smem_u32(ring_smem) + 127u) & ~127u;
    const uint8_t *ring_gen = ring_smem + (ring_base - cdc_smem_u32(ring_smem));
    auto full_bar = [&](int s) { return cdc_smem_u32(&bars[s]); };
    auto empty_bar = [&](int s) { return cdc_smem_u32(&bars[RING_STAGES + s]); };
    if (tid == 0) {
        for (int s = 0; s < RING_STAGES; ++s) { cdc_mbar_init(full_bar(s), 1); cdc_mbar_init(empty_bar(s), RING_THREADS / 32); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int64_t groups_total = n >> 2;
    int my_tiles = 0;
    {
        const int64_t tiles_total = (groups_total + tile_groups - 1) / tile_groups;
        if ((int64_t)blockIdx.x < tiles_total) {
            const int64_t mine = (tiles_total - blockIdx.x + gridDim.x - 1) / gridDim.x;
            my_tiles = (int)(mine < tiles_per_cta ? mine : tiles_per_cta);
        }
    }
    auto tile_count = [&](int64_t j) {
        const int64_t left = groups_total - j * tile_groups;
        return (int)(left < tile_groups ? left : tile_groups);
    };
    __syncthreads();
    cdc_pdl_wait();
    cdc_pdl_launch_dependents();   // after the wait: see cn_absmax_kernel
    if (tid == 0) {
        for (int i = 0; i < RING_STAGES && i < my_tiles; ++i) {
            const int64_t j = blockIdx.x + (int64_t)i * gridDim.x;
            const uint32_t bytes = (uint32_t)tile_count(j) * 16u;
            cdc_mbar_expect_tx(full_bar(i), bytes);
            cdc_bulk_load(ring_base + (uint32_t)i * (RING_TILE * 4), A + j * tile_groups * 4, bytes, full_bar(i));
        }
    }
    float m = -1.0f;   // the reference seeds thrust::reduce with -1.0f (source/basicOps.cu:1079)
    bool ok = true;
    for (int i = 0; i < my_tiles && ok; ++i) {
        const int s = i % RING_STAGES;
        const uint32_t ph = (uint32_t)(i / RING_STAGES) & 1u;
        if (tid == 0 && i >= 1 && i - 1 + RING_STAGES < my_tiles) {
            const int ps = (i - 1) % RING_STAGES;
            const uint32_t pph = (uint32_t)((i - 1) / RING_STAGES) & 1u;
            const int64_t j = blockIdx.x + (int64_t)(i - 1 + RING_STAGES) * gridDim.x;
            const uint32_t bytes = (uint32_t)tile_count(j) * 16u;
            if (cdc_mbar_wait(empty_bar(ps), pph, status)) {
                cdc_mbar_expect_tx(full_bar(ps), bytes);
                cdc_bulk_load(ring_base + (uint32_t)ps * (RING_TILE * 4), A + j * tile_groups * 4, bytes, full_bar(ps));
            }
        }
        const int64_t j = blockIdx.x + (int64_t)i * gridDim.x;
        const int groups = tile_count(j);
        ok = cdc_mbar_wait(full_bar(s), ph, status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const float4 *src = reinterpret_cast<const float4 *>(ring_gen + (size_t)s * (RING_TILE * 4));
#pragma unroll
        for (int u = 0; u < RING_GROUPS_PER_THREAD; ++u) {
            if (tid + u * RING_THREADS < groups) {
                const float4 q = src[tid + u * RING_THREADS];
                m = fmaxf(m, fmaxf(fmaxf(fabsf(q.x), fabsf(q.y)), fmaxf(fabsf(q.z), fabsf(q.w))));
            }
        }
        __syncwarp();
        if ((tid & 31) == 0) cdc_mbar_arrive(empty_bar(s));
    }
    if (!ok && tid == 0) {
        for (int s = 0; s < RING_STAGES; ++s) {
            const long long t0 = clock64();
            while (!cdc_mbar_try(full_bar(s), 0u) && !cdc_mbar_try(full_bar(s), 1u) && clock64() - t0 < 20000000LL) {}
        }
    }
    if (blockIdx.x == 0 && tid < (int)(n - (groups_total << 2))) m = fmaxf(m, fabsf(A[(groups_total << 2) + tid]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & 31) == 0) warp_max[tid >> 5] = m;
    __syncthreads();
    if (tid < 32) {
        m = tid < RING_THREADS / 32 ? warp_max[tid] : -1.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (tid == 0) {
            partials[blockIdx.x] = m;
            __threadfence();
            const unsigned int prev = atomicAdd(ticket, 1u);
            is_last = (prev == gridDim.x - 1);
        }
    }
    __syncthreads();
    if (is_last) {
        __threadfence();
        float r = -1.0f;
        for (int i = tid; i < (int)gridDim.x; i += RING_THREADS) r = fmaxf(r, __ldcg(partials + i));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) r = fmaxf(r, __shfl_xor_sync(0xffffffffu, r, o));
        __syncthreads();
        if ((tid & 31) == 0) warp_max[tid >> 5] = r;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < RING_THREADS / 32; ++w) r = fmaxf(r, warp_max[w]);
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

// Launch with programmatic stream serialisation: the kernel may become resident while its predecessor in the stream is
// still running; it synchronises with it through griddepcontrol.wait.
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t s, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3((unsigned)block);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// The 127 boundaries in |x| space for a host-side scale: the smallest fp32 |x| with fl(|x| / |p|) >= T_j, found with the
// same IEEE single-precision products and quotients the kernel uses for a device-side scale (this file is compiled
// without fast-math or contraction).  Kept per context for the last scale seen.
static bool host_boundaries(cn_context *ctx, float precision, uint32_t X[128])
{
    uint32_t pbits;
    memcpy(&pbits, &precision, 4);
    if (ctx->codec_cache_valid && ctx->codec_cache_pbits == pbits) {
        memcpy(X, ctx->codec_cache_X, sizeof(ctx->codec_cache_X));
        return ctx->codec_cache_ok;
    }
    const float ap = fabsf(precision);
    bool ok = (ap >= 7.8886090522101181e-31f) && (ap <= 1.2676506002282294e30f);
    for (int j = 0; j < 128; ++j) X[j] = 0xffffffffu;
    for (int j = 0; j < CN_NUM_THR && ok; ++j) {
        float T;
        memcpy(&T, &ctx->h_thr[j], 4);
        volatile float prod = T * ap;
        float pf = prod;
        uint32_t xb;
        memcpy(&xb, &pf, 4);
        auto quot = [&](uint32_t bits) { float v; memcpy(&v, &bits, 4); volatile float q = v / ap; return (float)q; };
        int down = 0;
        for (; down < 6; ++down) {
            if (xb > 0u && quot(xb - 1u) >= T) --xb; else break;
        }
        bool good = down < 6;
        if (down == 0) {
            int up = 0;
            for (; up < 6; ++up) {
                if (quot(xb) < T) ++xb; else break;
            }
            good = up < 6;
        }
        if (!good) ok = false;
        X[j] = xb;
    }
    ctx->codec_cache_valid = true;
    ctx->codec_cache_pbits = pbits;
    ctx->codec_cache_ok = ok;
    memcpy(ctx->codec_cache_X, X, sizeof(ctx->codec_cache_X));
    return ok;
}

// scale_mode: RING_SCALE_HOST (precision), RING_SCALE_DEVICE (d_precision read) or RING_SCALE_ABSMAX (d_precision written)
static int compress_impl(cn_context *ctx, const float *d_A, float precision, float *d_precision, int scale_mode, int64_t n,
                         uint8_t *d_codes, void *stream, int after_own_absmax = 0)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_compress_8bit: null context");
    CN_REQUIRE(n >= 0, CN_ERR_ARG, "cn_compress_8bit: negative size");
    cudaStream_t s = cn_stream(stream);
    const bool ring_ok = ((uintptr_t)d_A % 16 == 0) && ((uintptr_t)d_codes % 4 == 0) && n >= 4;
    // The single cooperative launch pays off while the pair of launches is bound by launch latency; from a few million
    // elements on, two pipelined launches are faster (measured on a B200: 13.7 vs 21.6 us at 2.4 M elements, 39.2 vs 33.6 us at
    // 16.8 M: the second pass is bound by the integer pipe, not by HBM, so reading it from L2 gains nothing).
    if (scale_mode == RING_SCALE_ABSMAX && (!ring_ok || n > CN_FUSED_ABSMAX_MAX_N)) {
        // also for buffers the ring kernel does not take (unaligned, tiny, empty): the two-call form
        int st = cn_absmax_f32(ctx, d_A, n, d_precision, stream);
        if (st != CN_OK || n == 0) return st;
        return compress_impl(ctx, d_A, 0.f, d_precision, RING_SCALE_DEVICE, n, d_codes, stream, 1);
    }
    if (n == 0) return CN_OK;
    CN_REQUIRE(d_A && d_codes, CN_ERR_ARG, "cn_compress_8bit: null buffer");
    if (ring_ok) {
        static bool attr_set[64] = {};   // per device: the attribute belongs to the device's copy of the function
        static int occupancy[64] = {};
        const size_t smem = (size_t)RING_STAGES * RING_TILE * 4 + 128;
        const int dev = ctx->device;
        if (dev < 0 || dev >= 64 || !attr_set[dev]) {
            CN_CUDA(cudaFuncSetAttribute(cn_compress_ring_kernel<RING_SCALE_HOST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            CN_CUDA(cudaFuncSetAttribute(cn_compress_ring_kernel<RING_SCALE_DEVICE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            CN_CUDA(cudaFuncSetAttribute(cn_compress_ring_kernel<RING_SCALE_ABSMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            int occ = 0;
            CN_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, cn_compress_ring_kernel<RING_SCALE_ABSMAX>, RING_THREADS, smem));
            if (dev >= 0 && dev < 64) { attr_set[dev] = true; occupancy[dev] = occ; }
        }
        unsigned int *d_status = nullptr;
        int st = cn_status_block(ctx, &d_status);
        if (st != CN_OK) return st;
        RingConst rc;
        for (int i = 0; i < 128; ++i) { rc.thr[i] = ctx->h_thr[i]; rc.lc[i] = ctx->h_level_codes[i]; rc.X[i] = 0xffffffffu; }
        rc.x_valid = 0;
        if (scale_mode == RING_SCALE_HOST) rc.x_valid = host_boundaries(ctx, precision, rc.X) ? 1 : 0;
        // every CTA gets the same number of equally sized tiles (at most RING_TILE elements each)
        const int64_t groups = n >> 2, max_groups = RING_TILE / 4;
        const int64_t min_tiles = (groups + max_groups - 1) / max_groups;
        int ctas_per_sm = 2;
        if (scale_mode == RING_SCALE_ABSMAX) {   // cooperative launch: all CTAs must be resident at once
            const int occ = (dev >= 0 && dev < 64) ? occupancy[dev] : 1;
            CN_REQUIRE(occ >= 1, CN_ERR_UNSUPPORTED, "cn_absmax_compress_8bit: the kernel does not fit this device");
            if (occ < ctas_per_sm) ctas_per_sm = occ;
        }
        const int64_t max_grid = (int64_t)ctas_per_sm * ctx->sm_count;
        int grid = (int)(min_tiles < max_grid ? min_tiles : max_grid);
        if (grid > CN_MAX_PARTIALS) grid = CN_MAX_PARTIALS;
        const int64_t tpc64 = (min_tiles + grid - 1) / grid;
        CN_REQUIRE(tpc64 < (1LL << 30), CN_ERR_UNSUPPORTED, "cn_compress_8bit: tensor too large");
        const int tiles_per_cta = (int)tpc64;
        int tile_groups = (int)((groups + (int64_t)grid * tiles_per_cta - 1) / ((int64_t)grid * tiles_per_cta));
        // whole tiles save the per-thread bounds tests: take them when the busiest CTA gets at most 2 % more work than with
        // the exactly balanced size
        if ((int64_t)tiles_per_cta * max_groups * 100 <= (int64_t)tiles_per_cta * tile_groups * 102) tile_groups = (int)max_groups;
        unsigned int *barrier_words = ctx->d_ticket + 4;   // words 4, 5 of the ticket block: arrival count, generation
        if (scale_mode == RING_SCALE_ABSMAX) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)grid);
            cfg.blockDim = dim3(RING_THREADS);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = s;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeCooperative;
            attr[0].val.cooperative = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            CN_CUDA(cudaLaunchKernelEx(&cfg, cn_compress_ring_kernel<RING_SCALE_ABSMAX>, d_A, 0.f, d_precision, n, d_codes, rc, d_status, tile_groups,
                                       tiles_per_cta, ctx->d_partials, barrier_words, 0));
        } else if (scale_mode == RING_SCALE_DEVICE) {
            CN_CUDA(launch_pdl(cn_compress_ring_kernel<RING_SCALE_DEVICE>, grid, RING_THREADS, smem, s, d_A, 0.f, d_precision, n, d_codes, rc, d_status,
                               tile_groups, tiles_per_cta, (float *)nullptr, (unsigned int *)nullptr, after_own_absmax));
        } else {
            CN_CUDA(launch_pdl(cn_compress_ring_kernel<RING_SCALE_HOST>, grid, RING_THREADS, smem, s, d_A, precision, (float *)nullptr, n, d_codes, rc,
                               d_status, tile_groups, tiles_per_cta, (float *)nullptr, (unsigned int *)nullptr, 0));
        }
        cn_count_launch();
        return CN_OK;
    }
    int grid = codec_grid(ctx, n, CODEC_THREADS, 4, 1);
    CodecConst cc;
    for (int i = 0; i < 128; ++i) { cc.thr[i] = ctx->h_thr[i]; cc.lc[i] = ctx->h_level_codes[i]; }
    if (scale_mode == RING_SCALE_DEVICE)
        CN_CUDA(launch_pdl(cn_compress_kernel<true>, grid, CODEC_THREADS, 0, s, d_A, 0.f, (const float *)d_precision, n, d_codes, cc, 0));
    else
        CN_CUDA(launch_pdl(cn_compress_kernel<false>, grid, CODEC_THREADS, 0, s, d_A, precision, (const float *)nullptr, n, d_codes, cc, 0));
    cn_count_launch();
    return CN_OK;
}

int cn_absmax_compress_push(cn_context *ctx, const float *d_A, int64_t n, float *d_scale_out, uint8_t *d_codes, const cn_codec_push *push,
                            void *stream, int *done)
{
    *done = 0;
    CN_REQUIRE(ctx && d_scale_out && push, CN_ERR_ARG, "cn_absmax_compress_push: null argument");
    if (n < 4 || n > CN_FUSED_ABSMAX_MAX_N || (uintptr_t)d_A % 16 != 0 || (uintptr_t)d_codes % 4 != 0) return CN_OK;
    for (int d = 0; d < push->ndst; ++d)
        if ((uintptr_t)push->codes_dst[d] % 4 != 0) return CN_OK;
    static bool have_occ[64] = {};
    static int occupancy[64] = {};
    const int dev = ctx->device;
    int occ = (dev >= 0 && dev < 64 && have_occ[dev]) ? occupancy[dev] : 0;
    if (occ == 0) {
        CN_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, cn_absmax_compress_push_kernel, RING_THREADS, 0));
        if (dev >= 0 && dev < 64) { have_occ[dev] = true; occupancy[dev] = occ; }
    }
    if (occ < 1) return CN_OK;
    unsigned int *d_status = nullptr;
    int st = cn_status_block(ctx, &d_status);
    if (st != CN_OK) return st;
    RingConst rc;
    for (int i = 0; i < 128; ++i) { rc.thr[i] = ctx->h_thr[i]; rc.lc[i] = ctx->h_level_codes[i]; rc.X[i] = 0xffffffffu; }
    rc.x_valid = 0;
    // cooperative launch: all CTAs resident; four 16-byte groups per thread and pass at least
    const int64_t groups = n >> 2;
    int64_t grid = (groups + (int64_t)RING_THREADS * 4 - 1) / ((int64_t)RING_THREADS * 4);
    const int64_t max_grid = (int64_t)(occ < 2 ? occ : 2) * ctx->sm_count;
    if (grid > max_grid) grid = max_grid;
    if (grid > CN_MAX_PARTIALS) grid = CN_MAX_PARTIALS;
    if (grid < 1) grid = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(RING_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = cn_stream(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    CN_CUDA(cudaLaunchKernelEx(&cfg, cn_absmax_compress_push_kernel, d_A, n, d_scale_out, d_codes, rc, d_status, ctx->d_partials,
                               ctx->d_ticket + 4, *push));
    cn_count_launch();
    *done = 1;
    return CN_OK;
}

extern "C" int cn_compress_8bit(cn_context *ctx, const float *d_A, float precision, int64_t n, uint8_t *d_codes, void *stream)
{
    return compress_impl(ctx, d_A, precision, nullptr, RING_SCALE_HOST, n, d_codes, stream);
}

extern "C" int cn_compress_8bit_dp(cn_context *ctx, const float *d_A, const float *d_precision, int64_t n, uint8_t *d_codes, void *stream)
{
    CN_REQUIRE(d_precision, CN_ERR_ARG, "cn_compress_8bit_dp: null precision pointer");
    return compress_impl(ctx, d_A, 0.f, const_cast<float *>(d_precision), RING_SCALE_DEVICE, n, d_codes, stream);
}

extern "C" int cn_absmax_compress_8bit(cn_context *ctx, const float *d_A, int64_t n, float *d_scale_out, uint8_t *d_codes, void *stream)
{
    CN_REQUIRE(ctx && d_scale_out, CN_ERR_ARG, "cn_absmax_compress_8bit: null argument");
    CN_REQUIRE(n >= 0 && (n == 0 || (d_A && d_codes)), CN_ERR_ARG, "cn_absmax_compress_8bit: bad input");
    return compress_impl(ctx, d_A, 0.f, d_scale_out, RING_SCALE_ABSMAX, n, d_codes, stream);
}

static int decompress_impl(cn_context *ctx, const uint8_t *d_codes, float precision, const float *d_precision, int64_t n,
                           float *d_out, void *stream)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_decompress_8bit: null context");
    CN_REQUIRE(n >= 0, CN_ERR_ARG, "cn_decompress_8bit: negative size");
    if (n == 0) return CN_OK;
    CN_REQUIRE(d_out && d_codes, CN_ERR_ARG, "cn_decompress_8bit: null buffer");
    int vector_ok = ((uintptr_t)d_out % 16 == 0) && ((uintptr_t)d_codes % 4 == 0);
    // Sixteen codes per load for large tensors (2^28 codes: 218 vs 236 us).  Up to tens of MiB the four-codes kernel stays:
    // in a series of calls its one 1024-thread CTA per SM leaves room for the next launch to become resident early
    // (programmatic dependent launch), which is worth more there (4096 x 4096: 15.8 vs 16.9 us).
    if (vector_ok && (uintptr_t)d_codes % 16 == 0 && n >= (1LL << 26)) vector_ok = 2;
    int grid = codec_grid(ctx, n, CODEC_THREADS, vector_ok == 2 ? 16 : 4, 1);   // one resident CTA per SM
    DecodeConst dc;
    for (int i = 0; i < 128; ++i) dc.tbl[i] = ctx->h_tbl[i];
    if (vector_ok == 2) {
        if (d_precision)
            CN_CUDA(launch_pdl(cn_decompress16_kernel<true>, grid, CODEC_THREADS, 0, cn_stream(stream), d_codes, 0.f, d_precision, n, d_out, dc));
        else
            CN_CUDA(launch_pdl(cn_decompress16_kernel<false>, grid, CODEC_THREADS, 0, cn_stream(stream), d_codes, precision, (const float *)nullptr, n, d_out, dc));
        cn_count_launch();
        return CN_OK;
    }
    if (d_precision)
        CN_CUDA(launch_pdl(cn_decompress_kernel<true>, grid, CODEC_THREADS, 0, cn_stream(stream), d_codes, 0.f, d_precision, n, d_out, dc, vector_ok));
    else
        CN_CUDA(launch_pdl(cn_decompress_kernel<false>, grid, CODEC_THREADS, 0, cn_stream(stream), d_codes, precision, (const float *)nullptr, n, d_out, dc, vector_ok));
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
    if (vector_ok && n >= (1LL << 16) && n < (1LL << 27)) {
        // mid-sized tensors: the ring kernel (see there); small ones are launch-bound, large ones stream best below
        static bool attr_set[64] = {};
        const size_t smem = (size_t)RING_STAGES * RING_TILE * 4 + 128;
        if (ctx->device < 0 || ctx->device >= 64 || !attr_set[ctx->device]) {
            CN_CUDA(cudaFuncSetAttribute(cn_absmax_ring_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            if (ctx->device >= 0 && ctx->device < 64) attr_set[ctx->device] = true;
        }
        unsigned int *d_status = nullptr;
        int st = cn_status_block(ctx, &d_status);
        if (st != CN_OK) return st;
        const int64_t groups = n >> 2, max_groups = RING_TILE / 4;
        const int64_t min_tiles = (groups + max_groups - 1) / max_groups, max_grid = 2 * (int64_t)ctx->sm_count;
        const int grid = (int)(min_tiles < max_grid ? min_tiles : max_grid);
        const int tiles_per_cta = (int)((min_tiles + grid - 1) / grid);
        int tile_groups = (int)((groups + (int64_t)grid * tiles_per_cta - 1) / ((int64_t)grid * tiles_per_cta));
        if (max_groups * 100 <= (int64_t)tile_groups * 102) tile_groups = (int)max_groups;   // whole tiles when nearly balanced anyway
        CN_CUDA(launch_pdl(cn_absmax_ring_kernel, grid, RING_THREADS, smem, cn_stream(stream), d_A, n, d_out, ctx->d_partials, ctx->d_ticket,
                           d_status, tile_groups, tiles_per_cta));
        cn_count_launch();
        return CN_OK;
    }
    // measured: two CTAs per SM keep the last-ticket tail short on tensors of tens of MiB (64 MiB: 16.4 us vs 18.6 us with
    // four), eight per SM stream best on large ones (1 GiB: 6737 GB/s vs 6332)
    int grid = codec_grid(ctx, n, ABSMAX_THREADS, 16, n < (1LL << 27) ? 2 : 8);
    if (grid > CN_MAX_PARTIALS) grid = CN_MAX_PARTIALS;
    CN_CUDA(launch_pdl(cn_absmax_kernel<true>, grid, ABSMAX_THREADS, 0, cn_stream(stream), d_A, n, d_out, ctx->d_partials, ctx->d_ticket, vector_ok));
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
