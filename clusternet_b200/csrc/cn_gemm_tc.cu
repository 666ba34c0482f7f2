// Tensor-core GEMM for sm_100a: TMA -> shared memory -> (converter warps) -> TMEM -> tcgen05.mma -> TMEM
// accumulators -> tcgen05.ld -> fused bias / activation / maxout -> global stores.
//
// Problem: C (M x N) = A (M x K) . W (K x N), everything fp32 column-major (the reference's device layout),
// which is the product ClusterNet::dot hands to cublasSgemm (source/clusterNet.cpp:459-461).
//
// Mapping.  A column-major W has its K index contiguous for a fixed column n, i.e. it is a K-major operand with
// N "rows".  The kernel therefore computes the transposed tile D[n, m] = sum_k W[k, n] * A[m, k]:
//   * the tcgen05 "A" operand (128 rows = 128 columns n of W) is read from TENSOR MEMORY.  W is streamed from
//     HBM exactly once as raw fp32 by TMA; four converter warps read each 128 x 32 tile from shared memory,
//     split every value into TF32 hi = rna(x) and lo = rna(x - hi) in registers and write both planes to TMEM
//     with tcgen05.st.  No shared-memory traffic is spent on the split and the raw weights never need a
//     second copy in HBM;
//   * the tcgen05 "B" operand (UMMA N = 128 rows m of the activations) is read from shared memory.  The
//     activations are small next to W (M = 128 in the reference's layers), so a pre-pass re-lays them K-major
//     and pre-split into hi / lo planes once per call; every CTA then pulls 128 x 32 tiles of both planes by TMA;
//   * three products per k-step give fp32-level accuracy: D += Whi.Ahi + Wlo.Ahi + Whi.Alo ("3xTF32").
//     CN_GEMM_TF32 issues only the first.
//   * the accumulator tile lives in TMEM with lane = n and column = m, so in the epilogue one thread owns one
//     output column n and 32 consecutive rows m: the bias is a per-thread scalar, the stores are contiguous
//     128-byte runs of the column-major C, and maxout over L consecutive columns is a shuffle across L lanes.
//
// Work decomposition.  One CTA per (m tile of 128, group of NT n tiles of 128, K split).  Skinny products have
// few tiles, so K is split across CTAs; each split leaves its partial tile in scratch and a second, grid-wide
// kernel adds the partials in split order (a fixed order, so results are reproducible) and runs the epilogue.  Launch order is split-major, which makes the CTAs resident at one time walk the same K
// range of the activations and share it through L2.
//
// Every wait on an mbarrier is bounded by a clock limit; a wait that runs out sets a status word that the host
// reads back as CN_ERR_TIMEOUT, lets the other roles drain, frees the tensor memory and returns.
#include <cuda.h>
#include <stdlib.h>
#include "cn_epilogue.cuh"
#include "cn_gemm.h"

#define TC_BM 128          // activation rows per CTA = UMMA N
#define TC_BN 128          // W columns per tile       = UMMA M
#define TC_BK 32           // fp32 per 128-byte swizzle row
#define TC_TILE_BYTES (128 * 128)
#define TC_CHAIN_DEFAULT 16   // K blocks (of 32) accumulated in TMEM before the sum is drained to registers
#define TC_DRAIN_SLEEP_NS 200   // poll interval of the drain warps while a chain accumulates
#define TC_WAIT_LIMIT (6000000000LL)   // clock cycles (~3 s)

template <int NT>
struct TcCfg {
    static constexpr int THREADS = 256 + 128 * NT;    // WG0 (producers, MMA), WG1 (converters), NT drain warpgroups
    // Two shared-memory rings with their own depth: raw W tiles (released by the converters as soon as they have
    // been read) and activation hi / lo tiles (released when the MMAs that read them retire).
    static constexpr int W_STAGES = NT == 1 ? 4 : 3;
    static constexpr int A_STAGES = NT == 1 ? 4 : 3;
    static constexpr int W_STAGE_BYTES = NT * TC_TILE_BYTES;
    static constexpr int A_STAGE_BYTES = 2 * TC_TILE_BYTES;
    static constexpr int W_RING = 0;
    static constexpr int A_RING = W_STAGES * W_STAGE_BYTES;
    static constexpr int RING_BYTES = A_RING + A_STAGES * A_STAGE_BYTES;
    static constexpr int TMEM_STAGES = NT == 1 ? 4 : 2;
    static constexpr int ACC_BUFS = NT == 1 ? 2 : 1;  // accumulators per W tile
    static constexpr int ACC_COL = 0;                 // NT * ACC_BUFS accumulators of 128 columns
    static constexpr int A_COL = NT * ACC_BUFS * TC_BM;   // then TMEM_STAGES x NT x (32 hi + 32 lo) columns
    static constexpr int A_STAGE_COLS = NT * 64;
    static constexpr int SMEM_BYTES = RING_BYTES + 1024 /*align*/ + 512 /*barriers*/;
    // register budgets after the warpgroups re-balance (multiples of 8); launch value is 65536 / THREADS
    static constexpr int REGS_WG0 = 88;
    static constexpr int REGS_CONV = 72;
    static constexpr int REGS_DRAIN = NT == 1 ? 232 : 176;
};

struct TcParams {
    int64_t M, N, K;
    float *C;
    int64_t ldc;
    const float *bias;
    int act;
    int maxout_level;
    float *argmax;
    int64_t tiles_n;        // groups of NT*128 columns
    int64_t tiles_m;
    int splits;
    int kb_per_split;       // K blocks (of 32) per split
    int kb_total;
    int chain_kb;           // K blocks accumulated in TMEM before the sum is drained to registers
    float *partials;        // [tile * NT + w][split][128 n][128 m]: every partial tile laid out like C
    unsigned int *status;
    // fused all-gather: peer copies of the C window (same leading dimension), flags the peers raise when ready
    int npeers;
    float *peerC[CN_MAX_PEERS];
    const unsigned int *ready;
    unsigned int *const *peer_flags;
    int nranks;
    int my_rank;
    unsigned int epoch;
};

// ---------------------------------------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done;
}
// Bounded wait.  Returns false when the limit ran out or another role already gave up.
// SLEEP_NS > 0 parks the warp between polls: used by roles that wait for a long time (the drain warps sit out a
// whole accumulation chain) so that their polling does not take issue slots from the converter and MMA warps.
template <int SLEEP_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, unsigned int *status, unsigned int code)
{
    if (mbar_try(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; ++it) {
        if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
        if (mbar_try(bar, parity)) return true;
        if ((it & 63u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > TC_WAIT_LIMIT) {
                *abort_flag = 1;
                atomicMax(status, code);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t x, int32_t y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[tmem] * B[smem desc]; A: 128 lanes x 8 columns of TF32, B: 128 x 8 K-major TF32 tile.
// The descriptor travels as two 32-bit halves so that stepping along K is a 32-bit add on the low half.
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_desc_lo, uint32_t b_desc_hi, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 bd;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 bd, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], bd, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_desc_lo), "r"(b_desc_hi), "r"(idesc), "r"(accumulate) : "memory");
}

#define TC_R32(a) \
    a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], a[8], a[9], a[10], a[11], a[12], a[13], a[14], a[15], a[16], a[17], \
    a[18], a[19], a[20], a[21], a[22], a[23], a[24], a[25], a[26], a[27], a[28], a[29], a[30], a[31]

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, "
        "%24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, "
        "%25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// fp32 -> TF32 (10 mantissa bits kept, low 13 bits zero), round to nearest with ties away from zero: add half a
// TF32 ulp to the magnitude bits and truncate.  Same result as cvt.rna.tf32.f32 for finite inputs, but two full-rate
// integer operations; the cvt form issues at a fraction of that rate and made the converter warps the bottleneck.
__device__ __forceinline__ uint32_t to_tf32(float x)
{
    return (__float_as_uint(x) + 0x1000u) & 0xffffe000u;
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (32 fp32) with the 128-byte
// swizzle TMA applies: 8-row groups are 1024 bytes apart (stride byte offset), the leading byte offset is
// unused for swizzled K-major layouts, version field 1 (sm_100), layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// kind::tf32 instruction descriptor: D fp32 (bits 4-5 = 1), A and B TF32 (format 2 at bits 7-9 and 10-12),
// both operands K-major (bits 15, 16 = 0), N >> 3 at bits 17-22, M >> 4 at bits 24-28.
__host__ __device__ constexpr uint32_t make_idesc_tf32(int m, int n)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ------------------------------------------------------------------------------------------ activation pre-pass
// A (M x K, column-major, lda) -> planes hi, lo : [M][Kpad] with k contiguous; k in [K, Kpad) is zero.
__global__ void __launch_bounds__(256)
cn_act_split_kernel(const float *__restrict__ A, int64_t lda, int64_t M, int64_t K, int64_t Kpad,
                    float *__restrict__ hi, float *__restrict__ lo, int64_t tiles_k)
{
    __shared__ float tile[32][33];
    const int64_t tm = blockIdx.x / tiles_k, tk = blockIdx.x % tiles_k;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t m_in = tm * 32 + tx;
#pragma unroll
    for (int j = ty; j < 32; j += 8) {
        const int64_t k = tk * 32 + j;
        tile[j][tx] = (m_in < M && k < K) ? A[m_in + k * lda] : 0.0f;
    }
    __syncthreads();
    const int64_t k_out = tk * 32 + tx;
#pragma unroll
    for (int j = ty; j < 32; j += 8) {
        const int64_t m = tm * 32 + j;
        if (m < M && k_out < Kpad) {
            const float x = tile[tx][j];
            const uint32_t h = to_tf32(x);
            hi[m * Kpad + k_out] = __uint_as_float(h);
            if (lo) lo[m * Kpad + k_out] = __uint_as_float(to_tf32(x - __uint_as_float(h)));
        }
    }
}

// The consumer-side half of the 8-bit exchange: the activations arrive as gathered codes (column-major like the fp32
// matrix; column block r was coded by rank r with scale scales[r]) and are decoded here, inside the pre-pass of the GEMM
// that consumes them, instead of being written out as fp32 first.  This rank's own block is taken from its exact fp32
// values.  Decode table as kDecompression_8bit builds it (source/clusterKernels.cu:1141-1152).
__global__ void __launch_bounds__(256)
cn_act_split_coded_kernel(const uint8_t *__restrict__ codes, const float *__restrict__ scales, const float *__restrict__ g_tbl,
                          const float *__restrict__ own_fp32, int own_rank, int nranks, int64_t M, int64_t K, int64_t Kpad,
                          float *__restrict__ hi, float *__restrict__ lo, int64_t tiles_k)
{
    __shared__ float tile[32][33];
    extern __shared__ float lut[];   // nranks x 256
    for (int e = threadIdx.x; e < nranks * 256; e += blockDim.x) {
        const int r = e >> 8, c = e & 255, i = c & 127;
        const float p = scales[r];
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
    const int64_t split = K / nranks;
    const int64_t tm = blockIdx.x / tiles_k, tk = blockIdx.x % tiles_k;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t m_in = tm * 32 + tx;
#pragma unroll
    for (int j = ty; j < 32; j += 8) {
        const int64_t k = tk * 32 + j;
        float x = 0.0f;
        if (m_in < M && k < K) {
            int r = split > 0 ? (int)(k / split) : nranks - 1;
            if (r > nranks - 1) r = nranks - 1;
            if (r == own_rank && own_fp32) x = own_fp32[m_in + (k - split * own_rank) * M];
            else x = lut[(r << 8) + codes[m_in + k * M]];
        }
        tile[j][tx] = x;
    }
    __syncthreads();
    const int64_t k_out = tk * 32 + tx;
#pragma unroll
    for (int j = ty; j < 32; j += 8) {
        const int64_t m = tm * 32 + j;
        if (m < M && k_out < Kpad) {
            const float x = tile[tx][j];
            const uint32_t h = to_tf32(x);
            hi[m * Kpad + k_out] = __uint_as_float(h);
            if (lo) lo[m * Kpad + k_out] = __uint_as_float(to_tf32(x - __uint_as_float(h)));
        }
    }
}

// Same planes for a transposed activation operand: op(A)(m, k) = A[k + m * lda] is already K-major (this is also what
// a row-major M x K batch looks like), so this is a copy-and-split: four consecutive k per thread, 16-byte loads and
// stores when the row pitch and the base allow, one block row per m.
__global__ void __launch_bounds__(256)
cn_act_split_t_kernel(const float *__restrict__ A, int64_t lda, int64_t M, int64_t K, int64_t Kpad,
                      float *__restrict__ hi, float *__restrict__ lo, int vec_ok)
{
    const int64_t k4 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (k4 >= Kpad) return;
    for (int64_t m = blockIdx.y; m < M; m += gridDim.y) {
        const float *src = A + m * lda + k4;
        float x[4];
        if (vec_ok && k4 + 3 < K) {
            const float4 v = __ldg(reinterpret_cast<const float4 *>(src));
            x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) x[e] = (k4 + e < K) ? src[e] : 0.0f;
        }
        uint32_t h[4], l[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            h[e] = to_tf32(x[e]);
            l[e] = to_tf32(x[e] - __uint_as_float(h[e]));
        }
        const int64_t o = m * Kpad + k4;   // Kpad is a multiple of 32 and the planes are 256-byte aligned
        *reinterpret_cast<uint4 *>(hi + o) = make_uint4(h[0], h[1], h[2], h[3]);
        if (lo) *reinterpret_cast<uint4 *>(lo + o) = make_uint4(l[0], l[1], l[2], l[3]);
    }
}

// -------------------------------------------------------------------------------------------------- main kernel
// Warp roles (warpgroups of 4 warps so that register budgets can be moved between them):
//   WG0  warp 0: TMA producer for W, warp 1: MMA issuer of W tile 0 + TMEM owner, warp 2: TMA producer for the
//        activations, warp 3: MMA issuer of W tile 1 (NT == 2)
//   WG1  warps 4-7:  converters (raw W tile in shared memory -> TF32 hi / lo planes in TMEM)
//   WG2  warps 8-11: accumulator drain + epilogue of W tile 0
//   WG3  warps 12-15 (NT == 2 only): the same for W tile 1
//
// Accumulation chains.  The tensor core adds into its fp32 accumulator with truncation, so a long chain of
// accumulating MMAs drifts (about 6e-8 of the running sum per step, all in one direction).  The K loop is therefore
// cut into chains of a few hundred k (TC_CHAIN_DEFAULT K blocks): each chain starts a fresh TMEM accumulator, and when it ends the drain warps
// read it with tcgen05.ld and add it, in round-to-nearest fp32, to running sums that they keep in registers
// (one thread = one output column n, 128 sums = 128 rows m).  With two W tiles per CTA the drain of one tile runs
// while the MMAs of the other tile execute; with one tile the accumulator is double-buffered in TMEM instead.
// TRANSB: the weight operand is stored transposed (N x K column-major, n contiguous).  Its tiles then arrive in shared
// memory as [32 k][128 n] without swizzle and the converters read them column-wise (conflict-free: consecutive lanes
// read consecutive n); everything downstream of TMEM is unchanged.
template <int NT, bool MODE3X, bool TRANSB>
__global__ void __launch_bounds__(TcCfg<NT>::THREADS, 1)
cn_gemm_tc_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_ahi,
                  const __grid_constant__ CUtensorMap tm_alo, const TcParams p)
{
    using Cfg = TcCfg<NT>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    // barriers and small words sit after the rings
    const uint32_t bar_base = smem_base + Cfg::RING_BYTES;
    uint8_t *bar_gen = smem_gen + Cfg::RING_BYTES;
    constexpr int B_WFULL = 0, B_WEMPTY = B_WFULL + Cfg::W_STAGES, B_AFULL = B_WEMPTY + Cfg::W_STAGES,
                  B_AEMPTY = B_AFULL + Cfg::A_STAGES, B_TFULL = B_AEMPTY + Cfg::A_STAGES, B_TEMPTY = B_TFULL + Cfg::TMEM_STAGES,
                  B_ACCFULL = B_TEMPTY + Cfg::TMEM_STAGES, B_ACCEMPTY = B_ACCFULL + NT * Cfg::ACC_BUFS,
                  B_COUNT = B_ACCEMPTY + NT * Cfg::ACC_BUFS;
    static_assert(B_COUNT * 8 <= 448, "barrier area");
    auto bar = [&](int idx) { return bar_base + 8u * idx; };
    auto wfull_bar = [&](int s) { return bar(B_WFULL + s); };
    auto wempty_bar = [&](int s) { return bar(B_WEMPTY + s); };
    auto afull_bar = [&](int s) { return bar(B_AFULL + s); };
    auto aempty_bar = [&](int s) { return bar(B_AEMPTY + s); };
    auto tfull_bar = [&](int t) { return bar(B_TFULL + t); };
    auto tempty_bar = [&](int t) { return bar(B_TEMPTY + t); };
    auto accfull_bar = [&](int w, int b) { return bar(B_ACCFULL + w * Cfg::ACC_BUFS + b); };
    auto accempty_bar = [&](int w, int b) { return bar(B_ACCEMPTY + w * Cfg::ACC_BUFS + b); };
    volatile uint32_t *tmem_holder = reinterpret_cast<volatile uint32_t *>(bar_gen + 448);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(bar_gen + 452);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Fused all-gather: the start of this kernel means everything queued earlier on this GPU's stream has finished, so
    // this rank's copy of C may now be overwritten by its peers: tell them (slot 0 of their flag block).
    if (p.npeers > 0 && blockIdx.x == 0 && threadIdx.x < p.nranks && (int)threadIdx.x != p.my_rank) {
        __threadfence_system();
        volatile unsigned int *f = p.peer_flags[threadIdx.x] + p.my_rank;
        *f = p.epoch;
    }

    // unit decode: split-major launch order
    const int64_t tiles = p.tiles_n * p.tiles_m;
    const int split = (int)(blockIdx.x / tiles);
    const int64_t tile_id = blockIdx.x % tiles;
    const int64_t tile_n = tile_id % p.tiles_n, tile_m = tile_id / p.tiles_n;
    const int64_t n0 = tile_n * (NT * TC_BN), m0 = tile_m * TC_BM;
    const int kb_begin = split * p.kb_per_split;
    int kb_end = kb_begin + p.kb_per_split;
    if (kb_end > p.kb_total) kb_end = p.kb_total;
    const int num_kb = kb_end - kb_begin;   // >= 1 by construction on the host
    const int chain_kb = p.chain_kb;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::W_STAGES; ++s) { mbar_init(wfull_bar(s), 1); mbar_init(wempty_bar(s), 128); }
        for (int s = 0; s < Cfg::A_STAGES; ++s) { mbar_init(afull_bar(s), 1); mbar_init(aempty_bar(s), NT); }
        for (int t = 0; t < Cfg::TMEM_STAGES; ++t) { mbar_init(tfull_bar(t), 128); mbar_init(tempty_bar(t), NT); }
        for (int w = 0; w < NT; ++w)
            for (int b = 0; b < Cfg::ACC_BUFS; ++b) { mbar_init(accfull_bar(w, b), 1); mbar_init(accempty_bar(w, b), 128); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // this warp owns the tensor-memory allocation
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_holder)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp < 4) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_WG0));
        if (warp == 0 || warp == 2) {
            // ------------------------------------------------------------ TMA producers: warp 0 streams W, warp 2 the activations
            if (lane == 0) {
                const bool is_w = warp == 0;
                const int depth = is_w ? Cfg::W_STAGES : Cfg::A_STAGES;
                int issued = 0;
                for (int i = 0; i < num_kb; ++i) {
                    const int s = i % depth;
                    const uint32_t ph = (uint32_t)(i / depth) & 1u;
                    const int32_t kx = (kb_begin + i) * TC_BK;
                    if (is_w) {
                        if (!mbar_wait(wempty_bar(s), ph ^ 1u, abort_flag, p.status, 1u)) break;
                        const uint32_t stage = smem_base + Cfg::W_RING + s * Cfg::W_STAGE_BYTES;
                        mbar_expect_tx(wfull_bar(s), (uint32_t)Cfg::W_STAGE_BYTES);
#pragma unroll
                        for (int t = 0; t < NT; ++t) {
                            if (TRANSB) tma_load_2d(stage + t * TC_TILE_BYTES, &tm_w, wfull_bar(s), (int32_t)(n0 + t * TC_BN), kx);
                            else        tma_load_2d(stage + t * TC_TILE_BYTES, &tm_w, wfull_bar(s), kx, (int32_t)(n0 + t * TC_BN));
                        }
                    } else {
                        if (!mbar_wait(aempty_bar(s), ph ^ 1u, abort_flag, p.status, 8u)) break;
                        const uint32_t stage = smem_base + Cfg::A_RING + s * Cfg::A_STAGE_BYTES;
                        mbar_expect_tx(afull_bar(s), (uint32_t)((MODE3X ? 2 : 1) * TC_TILE_BYTES));
                        tma_load_2d(stage, &tm_ahi, afull_bar(s), kx, (int32_t)m0);
                        if (MODE3X) tma_load_2d(stage + TC_TILE_BYTES, &tm_alo, afull_bar(s), kx, (int32_t)m0);
                    }
                    issued = i + 1;
                }
                if (*abort_flag) {
                    // give copies that are still in flight a bounded chance to land before the CTA exits
                    for (int i = issued > depth ? issued - depth : 0; i < issued; ++i) {
                        const int s = i % depth;
                        const uint32_t ph = (uint32_t)(i / depth) & 1u;
                        const long long t0 = clock64();
                        while (!mbar_try(is_w ? wfull_bar(s) : afull_bar(s), ph) && clock64() - t0 < 20000000LL) {}
                    }
                }
            }
            __syncwarp();
        } else if (warp == 1 || (NT == 2 && warp == 3)) {
            // ------------------------------------------------------------ MMA issuers: one thread per W tile (a single thread
            // cannot issue the 64-cycle TF32 MMAs of two tiles fast enough to keep the tensor pipe busy)
            if (lane == 0) {
                const int w = warp == 1 ? 0 : 1;
                constexpr uint32_t idesc = make_idesc_tf32(TC_BN, TC_BM);
                bool ok = true;
                // chain bookkeeping without divisions: position inside the chain, accumulator buffer and its phase
                // W tile 1 starts half a chain into its schedule, so that the two tiles never reach a chain end (and the
                // wait for their drain warps) on the same K block: while one tile's accumulator is read out, the MMAs of
                // the other keep the tensor pipe busy
                int chain_pos = (NT == 2 && w == 1) ? chain_kb / 2 : 0, ab = 0;
                bool chain_first = true;   // the next K block opens a chain: it overwrites the accumulator
                uint32_t aph = 0;
                // operands of the first K block
                ok = mbar_wait(afull_bar(0), 0u, abort_flag, p.status, 2u) && mbar_wait(tfull_bar(0), 0u, abort_flag, p.status, 3u);
                for (int i = 0; i < num_kb && ok; ++i) {
                    const int s = i % Cfg::A_STAGES, t = i % Cfg::TMEM_STAGES;
                    const bool chain_last = chain_pos == chain_kb - 1 || i == num_kb - 1;
                    tc_fence_after();
                    const uint32_t stage = smem_base + Cfg::A_RING + s * Cfg::A_STAGE_BYTES;
                    const uint64_t bhi = make_kmajor_sw128_desc(stage);
                    const uint64_t blo = make_kmajor_sw128_desc(stage + TC_TILE_BYTES);
                    const uint32_t bhi_lo = (uint32_t)bhi, bhi_hi = (uint32_t)(bhi >> 32), blo_lo = (uint32_t)blo, blo_hi = (uint32_t)(blo >> 32);
                    if (chain_first) {   // the drain warps must have emptied this accumulator
                        ok = mbar_wait(accempty_bar(w, ab), aph ^ 1u, abort_flag, p.status, 7u);
                        if (!ok) break;
                        tc_fence_after();
                    }
                    const uint32_t acc = tmem_base + Cfg::ACC_COL + (w * Cfg::ACC_BUFS + ab) * TC_BM;
                    const uint32_t a_hi = tmem_base + Cfg::A_COL + t * Cfg::A_STAGE_COLS + w * 64;
                    const uint32_t a_lo = a_hi + 32;
#pragma unroll
                    for (int j = 0; j < TC_BK / 8; ++j) {
                        if (j == TC_BK / 8 - 1 && i + 1 < num_kb) {
                            // Look ahead: make sure the operands of the next K block are there BEFORE the last MMAs of
                            // this one are issued.  Issue is back-pressured by the tensor pipe, so once those are in,
                            // only the commits stand between them and the next block's first MMA.
                            const int s1 = (i + 1) % Cfg::A_STAGES, t1 = (i + 1) % Cfg::TMEM_STAGES;
                            const uint32_t ph1 = (uint32_t)((i + 1) / Cfg::A_STAGES) & 1u, tph1 = (uint32_t)((i + 1) / Cfg::TMEM_STAGES) & 1u;
                            ok = mbar_wait(afull_bar(s1), ph1, abort_flag, p.status, 2u) && mbar_wait(tfull_bar(t1), tph1, abort_flag, p.status, 3u);
                        }
                        // 8 TF32 per k-step: 8 TMEM columns of A, 32 bytes (descriptor units of 16 B) of B
                        tc_mma_ts(acc, a_hi + j * 8, bhi_lo + j * 2, bhi_hi, idesc, (!chain_first || j > 0) ? 1u : 0u);
                        if (MODE3X) {
                            tc_mma_ts(acc, a_lo + j * 8, bhi_lo + j * 2, bhi_hi, idesc, 1u);
                            tc_mma_ts(acc, a_hi + j * 8, blo_lo + j * 2, blo_hi, idesc, 1u);
                        }
                    }
                    if (chain_last) {
                        tc_commit(accfull_bar(w, ab));
                        chain_pos = 0;
                        chain_first = true;
                        if (++ab == Cfg::ACC_BUFS) { ab = 0; aph ^= 1u; }
                    } else {
                        ++chain_pos;
                        chain_first = false;
                    }
                    tc_commit(aempty_bar(s));   // activation stage may be refilled once these MMAs retire
                    tc_commit(tempty_bar(t));   // and the TMEM operand stage rewritten
                }
            }
            __syncwarp();
        }
    } else if (warp < 8) {
        // ---------------------------------------------------------------- converter warps
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_CONV));
        const int q = warp & 3;                       // TMEM lane quarter this warp may touch
        const int row = q * 32 + lane;                // row of the W tile = TMEM lane
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        bool ok = true;
        for (int i = 0; i < num_kb && ok; ++i) {
            const int s = i % Cfg::W_STAGES, t = i % Cfg::TMEM_STAGES;
            const uint32_t ph = (uint32_t)(i / Cfg::W_STAGES) & 1u, tph = (uint32_t)(i / Cfg::TMEM_STAGES) & 1u;
            ok = mbar_wait(wfull_bar(s), ph, abort_flag, p.status, 4u) && mbar_wait(tempty_bar(t), tph ^ 1u, abort_flag, p.status, 5u);
            ok = __all_sync(0xffffffffu, ok);   // the tcgen05 stores below need the whole warp
            if (!ok) break;
            tc_fence_after();
            const uint8_t *stage = smem_gen + Cfg::W_RING + s * Cfg::W_STAGE_BYTES;
#pragma unroll 1
            for (int w = 0; w < NT; ++w) {
                const uint8_t *tilep = stage + w * TC_TILE_BYTES;
                const uint32_t a_hi = tmem_base + lane_addr + Cfg::A_COL + t * Cfg::A_STAGE_COLS + w * 64;
                uint32_t hi[32], lo[32];
                if (TRANSB) {
#pragma unroll
                    for (int k = 0; k < 32; ++k) {
                        const float x = *reinterpret_cast<const float *>(tilep + k * (TC_BN * 4) + row * 4);
                        const uint32_t h = to_tf32(x);
                        hi[k] = h;
                        if (MODE3X) lo[k] = to_tf32(x - __uint_as_float(h));
                    }
                } else {
                    const uint8_t *rowp = tilep + row * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        // 16-byte chunk c of row r sits at chunk position c ^ (r & 7) under the 128-byte swizzle
                        const float4 v = *reinterpret_cast<const float4 *>(rowp + ((c ^ (row & 7)) << 4));
                        const float x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t h = to_tf32(x[e]);
                            hi[c * 4 + e] = h;
                            if (MODE3X) lo[c * 4 + e] = to_tf32(x[e] - __uint_as_float(h));
                        }
                    }
                }
                tc_st32(a_hi, hi);
                if (MODE3X) tc_st32(a_hi + 32, lo);
            }
            mbar_arrive(wempty_bar(s));   // the raw tile now lives in registers / TMEM: its ring slot may be refilled
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(tfull_bar(t));
        }
    } else {
        // ---------------------------------------------------------------- drain + epilogue warps, one warpgroup per W tile
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Cfg::REGS_DRAIN));
        const int w = (warp - 8) >> 2;                // W tile of this warpgroup
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const int et = threadIdx.x & 127;
        float acc[TC_BM];
#pragma unroll
        for (int i = 0; i < TC_BM; ++i) acc[i] = 0.0f;
        bool ok = true;
        // chains of this W tile: tile 1's first chain is the short one (see the MMA issuer)
        const int my_chains = (num_kb + ((NT == 2 && w == 1) ? chain_kb / 2 : 0) + chain_kb - 1) / chain_kb;
        for (int c = 0; c < my_chains && ok; ++c) {
            const int ab = c % Cfg::ACC_BUFS;
            const uint32_t aph = (uint32_t)(c / Cfg::ACC_BUFS) & 1u;
            ok = mbar_wait<TC_DRAIN_SLEEP_NS>(accfull_bar(w, ab), aph, abort_flag, p.status, 6u);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t src = tmem_base + lane_addr + Cfg::ACC_COL + (w * Cfg::ACC_BUFS + ab) * TC_BM;
#pragma unroll
            for (int cc = 0; cc < TC_BM / 32; ++cc) {
                uint32_t r[32];
                tc_ld32(src + cc * 32, r);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[cc * 32 + i] += __uint_as_float(r[i]);
            }
            tc_fence_before();
            mbar_arrive(accempty_bar(w, ab));
        }
        {   // all 128 threads of the warpgroup go on together or not at all
            uint32_t all_ok;
            asm volatile(
                "{\n\t.reg .pred pi, po;\n\t"
                "setp.ne.u32 pi, %1, 0;\n\t"
                "bar.red.and.pred po, %2, 128, pi;\n\t"
                "selp.u32 %0, 1, 0, po;\n\t}"
                : "=r"(all_ok) : "r"((uint32_t)ok), "r"(1 + w) : "memory");
            ok = all_ok != 0;
        }
        if (ok && NT == 2 && w == 1) {
            // This warpgroup stages its output tile in the activation ring.  Its own accumulator being complete says
            // nothing about the other tile's MMAs, which read the same ring stages: wait until the last K block's stage
            // has been released by both issuers (their commits arrive in issue order, so every earlier stage is free too).
            const int last = num_kb - 1;
            ok = mbar_wait(aempty_bar(last % Cfg::A_STAGES), (uint32_t)(last / Cfg::A_STAGES) & 1u, abort_flag, p.status, 11u);
            uint32_t all_ok;
            asm volatile(
                "{\n\t.reg .pred pi, po;\n\t"
                "setp.ne.u32 pi, %1, 0;\n\t"
                "bar.red.and.pred po, %2, 128, pi;\n\t"
                "selp.u32 %0, 1, 0, po;\n\t}"
                : "=r"(all_ok) : "r"((uint32_t)ok), "r"(1 + w) : "memory");
            ok = all_ok != 0;
            tc_fence_after();
        }
        if (ok) {
            const int64_t ticket_id = tile_id * NT + w;
            const size_t tile_elems = (size_t)TC_BM * TC_BN;
            bool do_final = true;
            if (p.splits > 1) {
                // Split-K: this CTA's partial tile goes to scratch as one contiguous 64 KB block laid out like C (column n =
                // 512 bytes), staged through the idle rings and written with a single bulk copy; cn_splitk_reduce_kernel adds
                // the partials of all splits in split order and applies the epilogue, spread over the whole GPU.
                float *stg = reinterpret_cast<float *>(smem_gen + (w == 0 ? Cfg::W_RING : Cfg::A_RING));
#pragma unroll
                for (int i = 0; i < TC_BM; i += 4)
                    *reinterpret_cast<float4 *>(stg + row * TC_BM + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("bar.sync %0, 128;" ::"r"(1 + w) : "memory");
                if (et == 0) {
                    float *P = p.partials + ((size_t)ticket_id * p.splits + split) * tile_elems;
                    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                                 ::"l"(P), "r"(smem_u32(stg)), "r"((uint32_t)(tile_elems * sizeof(float))) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                }
                do_final = false;
            }
            if (do_final) {
                const int L = p.maxout_level;
                const int64_t n = n0 + w * TC_BN + row;
                const float bias = (p.bias && n < p.N) ? p.bias[n] : 0.0f;
#pragma unroll
                for (int i = 0; i < TC_BM; ++i) acc[i] = cn_apply_activation(p.bias ? acc[i] + bias : acc[i], p.act);
                if (L <= 1) {
                    if (p.npeers > 0) {
                        // the peers must have announced that their copy of C may be overwritten (bounded wait)
                        if (et == 0) {
                            const long long t0 = clock64();
                            for (int r = 0; r < p.nranks; ++r) {
                                if (r == p.my_rank) continue;
                                const volatile unsigned int *f = p.ready + r;
                                while ((int)(*f - p.epoch) < 0) {
                                    if (clock64() - t0 > TC_WAIT_LIMIT) { atomicMax(p.status, 9u); break; }
                                    __nanosleep(100);
                                }
                            }
                        }
                        asm volatile("bar.sync %0, 128;" ::"r"(1 + w) : "memory");
                    }
                    const int64_t rows_valid = (p.M - m0) < TC_BM ? (p.M - m0) : TC_BM;
                    if (p.npeers > 0 && (rows_valid & 3) == 0 && (p.ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(p.C) & 15u) == 0) {
                        // Fused all-gather.  Scattered 16-byte stores from registers are a poor fit for NVLink, so the tile is
                        // first laid out in shared memory exactly as it lies in C (column n = 512 contiguous bytes; the rings
                        // are idle by now: tile 0 borrows the W ring, tile 1 the activation ring) and then written to the
                        // local C and to every peer's C with bulk asynchronous copies.
                        float *stg = reinterpret_cast<float *>(smem_gen + (w == 0 ? Cfg::W_RING : Cfg::A_RING));
#pragma unroll
                        for (int i = 0; i < TC_BM; i += 4)
                            *reinterpret_cast<float4 *>(stg + row * TC_BM + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        asm volatile("bar.sync %0, 128;" ::"r"(1 + w) : "memory");
                        const int64_t col0 = n0 + w * TC_BN;
                        const int64_t cols_valid = (p.N - col0) < TC_BN ? (p.N - col0) : TC_BN;
                        if (rows_valid == TC_BM && p.ldc == TC_BM) {
                            // the tile is one contiguous block of C: one copy per destination
                            if (et == 0 && cols_valid > 0) {
                                const uint32_t bytes = (uint32_t)(cols_valid * TC_BM * sizeof(float));
                                const int64_t off = col0 * p.ldc + m0;
                                for (int d = 0; d <= p.npeers; ++d) {
                                    float *dst = (d == 0 ? p.C : p.peerC[d - 1]) + off;
                                    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                                                 ::"l"(dst), "r"(smem_u32(stg)), "r"(bytes) : "memory");
                                }
                                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                                asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                            }
                        } else if (n < p.N) {
                            // one copy per column and destination
                            const uint32_t bytes = (uint32_t)(rows_valid * sizeof(float));
                            const int64_t off = n * p.ldc + m0;
                            for (int d = 0; d <= p.npeers; ++d) {
                                float *dst = (d == 0 ? p.C : p.peerC[d - 1]) + off;
                                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                                             ::"l"(dst), "r"(smem_u32(stg + row * TC_BM)), "r"(bytes) : "memory");
                            }
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
                        }
                    } else if (n < p.N) {
                        const int64_t off = n * p.ldc + m0;
                        float *dst = p.C + off;
                        if (m0 + TC_BM <= p.M && ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0)) {
#pragma unroll
                            for (int i = 0; i < TC_BM; i += 4)
                                *reinterpret_cast<float4 *>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
                        } else {
#pragma unroll
                            for (int i = 0; i < TC_BM; ++i)
                                if (m0 + i < p.M) dst[i] = acc[i];
                        }
                        for (int pr = 0; pr < p.npeers; ++pr) {   // rare shapes only: rows not a multiple of four
                            float *pd = p.peerC[pr] + off;
#pragma unroll
                            for (int i = 0; i < TC_BM; ++i)
                                if (m0 + i < p.M) pd[i] = acc[i];
                        }
                    }
                } else {
                    // maxout over L consecutive columns = L adjacent lanes (L is a power of two <= 32).
                    // Same comparison tree as the reference's 32-slot reduction: at offsets L/2 .. 1 slot t
                    // takes slot t+offset when strictly smaller; larger offsets only meet -FLT_MAX padding.
                    const int tl = lane & (L - 1);
#pragma unroll
                    for (int i = 0; i < TC_BM; ++i) {
                        float val = acc[i], idx = (float)n;
                        for (int off = L >> 1; off > 0; off >>= 1) {
                            const float ov = __shfl_down_sync(0xffffffffu, val, off, L);
                            const float oi = __shfl_down_sync(0xffffffffu, idx, off, L);
                            if (tl < off && val < ov) { val = ov; idx = oi; }
                        }
                        if (tl == 0 && n < p.N && m0 + i < p.M) {
                            const int64_t g = n / L;
                            p.C[g * p.ldc + m0 + i] = val;
                            if (p.argmax) p.argmax[g * p.ldc + m0 + i] = idx;
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------------------------------- split-K reduction
// One thread = four consecutive rows m of one output column n: adds the partial tiles of all splits in split order (a
// fixed order, so the result does not depend on scheduling), applies bias and activation, stores to C and, for the
// fused all-gather, to every peer's C (a warp writes 512 contiguous bytes of a column: full NVLink packets).
struct ReduceParams {
    const float *partials;
    int splits, nt;
    int64_t tiles_n, tiles_m, M, N;
    float *C;
    int64_t ldc;
    const float *bias;
    int act;
    int npeers;
    float *peerC[CN_MAX_PEERS];
    const unsigned int *ready;
    int nranks, my_rank;
    unsigned int epoch;
    unsigned int *status;
};

__global__ void __launch_bounds__(256)
cn_splitk_reduce_kernel(const ReduceParams p)
{
    if (p.npeers > 0) {   // peers must have announced that their copy of C may be overwritten (bounded wait)
        if (threadIdx.x == 0) {
            const long long t0 = clock64();
            for (int r = 0; r < p.nranks; ++r) {
                if (r == p.my_rank) continue;
                const volatile unsigned int *f = p.ready + r;
                while ((int)(*f - p.epoch) < 0) {
                    if (clock64() - t0 > TC_WAIT_LIMIT) { atomicMax(p.status, 9u); break; }
                    __nanosleep(100);
                }
            }
        }
        __syncthreads();
    }
    const size_t tile_elems = (size_t)TC_BM * TC_BN;
    const int64_t quads_per_tile = tile_elems / 4;
    const int64_t total = p.tiles_n * p.tiles_m * p.nt * quads_per_tile;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; q < total; q += stride) {
        const int64_t ticket = q / quads_per_tile;          // (tile_id * nt + w)
        const int64_t inner = q - ticket * quads_per_tile;  // n_local * 32 + m4
        const int n_local = (int)(inner >> 5), m_local = (int)(inner & 31) * 4;
        const int64_t tile_id = ticket / p.nt;
        const int w = (int)(ticket - tile_id * p.nt);
        const int64_t tile_n = tile_id % p.tiles_n, tile_m = tile_id / p.tiles_n;
        const int64_t n = tile_n * (p.nt * TC_BN) + w * TC_BN + n_local, m = tile_m * TC_BM + m_local;
        if (n >= p.N || m >= p.M) continue;
        const float *src = p.partials + (size_t)ticket * p.splits * tile_elems + (size_t)n_local * TC_BM + m_local;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        int sp = 0;
        // four loads in flight at a time; the additions stay in split order, so the sum does not depend on the grouping
        for (; sp + 4 <= p.splits; sp += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)(sp + u) * tile_elems));
#pragma unroll
            for (int u = 0; u < 4; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
        }
        for (; sp < p.splits; ++sp) {
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(src + (size_t)sp * tile_elems));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        const float b = p.bias ? p.bias[n] : 0.0f;
        float r[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) r[i] = cn_apply_activation(p.bias ? r[i] + b : r[i], p.act);
        const int64_t off = n * p.ldc + m;
        const bool vec = (m + 4 <= p.M) && ((p.ldc & 3) == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0);
        for (int d = 0; d <= p.npeers; ++d) {
            float *dst = (d == 0 ? p.C : p.peerC[d - 1]) + off;
            if (vec) {
                *reinterpret_cast<float4 *>(dst) = make_float4(r[0], r[1], r[2], r[3]);
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    if (m + i < p.M) dst[i] = r[i];
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int get_encode_fn(cn_context *ctx, EncodeTiledFn *out)
{
    if (!ctx->gemm) ctx->gemm = cn_gemm_workspace_new();
    if (!ctx->gemm->encode_fn) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        CN_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        CN_REQUIRE(fn && qres == cudaDriverEntryPointSuccess, CN_ERR_CUDA, "cuTensorMapEncodeTiled is not available in this driver");
        ctx->gemm->encode_fn = fn;
    }
    *out = (EncodeTiledFn)ctx->gemm->encode_fn;
    return CN_OK;
}

// 2-D fp32 map over a K-major array: inner extent `inner` (k), outer extent `outer` (rows), row pitch in elements.
// transposed = false: box 32 (k, inner) x 128 rows with the 128-byte swizzle; transposed = true (weight stored with n
// contiguous): box 128 (n, inner) x 32 k-rows, no swizzle.
static int make_map(EncodeTiledFn enc, CUtensorMap *map, const float *base, int64_t inner, int64_t outer, int64_t pitch, bool transposed = false)
{
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)pitch * sizeof(float)};
    cuuint32_t box[2] = {transposed ? 128u : (cuuint32_t)TC_BK, transposed ? (cuuint32_t)TC_BK : 128u};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, transposed ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    CN_REQUIRE(r == CUDA_SUCCESS, CN_ERR_CUDA, "cuTensorMapEncodeTiled failed with %d (inner %lld outer %lld pitch %lld)", (int)r,
               (long long)inner, (long long)outer, (long long)pitch);
    return CN_OK;
}

bool cn_gemm_tc_can_fuse_maxout(int L) { return L == 2 || L == 4 || L == 8 || L == 16 || L == 32; }

bool cn_gemm_tc_supported(cn_context *, int transA, int transB, int64_t M, int64_t N, int64_t K, const float *,
                          int64_t, const float *B, int64_t ldb, const float *, int64_t)
{
    (void)transA;   // a transposed activation operand only changes the pre-pass
    (void)transB;   // a transposed weight only changes the TMA box and the converter's read pattern
    if (M < 1 || N < 1 || K < 1) return false;   // short dimensions are zero-filled by TMA up to the tile
    if ((ldb & 3) != 0 || (reinterpret_cast<uintptr_t>(B) & 15u) != 0) return false;   // TMA: 16-byte pitch and base
    if (K >= (1LL << 31) - 64 || N >= (1LL << 31) - 256 || M >= (1LL << 31) - 256) return false;   // TMA coordinates are 32-bit
    return true;
}

static int pick_splits(int64_t tiles, int kb_total, int sm_count)
{
    if (tiles >= 2 * (int64_t)sm_count) return 1;
    int best = 1;
    double best_score = -1.0;
    for (int s = 1; s <= 32; ++s) {
        if (kb_total / s < 8) break;   // keep at least 8 K blocks (256 k) per split
        const int64_t units = tiles * s;
        const int64_t waves = (units + sm_count - 1) / sm_count;
        const double eff = (double)units / (double)(waves * sm_count);
        const double score = eff - 0.004 * s;   // prefer fewer splits when the fill is about equal
        if (score > best_score) { best_score = score; best = s; }
    }
    return best;
}

template <int NT, bool MODE3X, bool TRANSB>
static int launch_cfg(const CUtensorMap &mw, const CUtensorMap &mhi, const CUtensorMap &mlo, const TcParams &prm, int64_t grid, cudaStream_t s)
{
    static bool attr_set[64] = {};   // per device: the attribute belongs to the device's copy of the function
    int dev = 0;
    CN_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
        CN_CUDA(cudaFuncSetAttribute(cn_gemm_tc_kernel<NT, MODE3X, TRANSB>, cudaFuncAttributeMaxDynamicSharedMemorySize, TcCfg<NT>::SMEM_BYTES));
        if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
    cn_gemm_tc_kernel<NT, MODE3X, TRANSB><<<(unsigned)grid, TcCfg<NT>::THREADS, TcCfg<NT>::SMEM_BYTES, s>>>(mw, mhi, mlo, prm);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

int cn_gemm_tc_split_activations(cn_context *ctx, int transA, int64_t M, int64_t K, const float *A, int64_t lda, float *hi, float *lo,
                                 cudaStream_t s)
{
    (void)ctx;
    const int64_t Kpad = (K + TC_BK - 1) / TC_BK * TC_BK;
    const int64_t tiles_k = Kpad / 32, tiles_mm = (M + 31) / 32;
    CN_REQUIRE(tiles_k * tiles_mm < (1LL << 31), CN_ERR_UNSUPPORTED, "cn_gemm_f32: activation matrix too large for the split pre-pass");
    if (transA) {
        const int vec_ok = ((lda & 3) == 0) && ((reinterpret_cast<uintptr_t>(A) & 15u) == 0);
        dim3 grid((unsigned)((Kpad / 4 + 255) / 256), (unsigned)(M < 65535 ? M : 65535));
        cn_act_split_t_kernel<<<grid, 256, 0, s>>>(A, lda, M, K, Kpad, hi, lo, vec_ok);
    } else {
        cn_act_split_kernel<<<(unsigned)(tiles_k * tiles_mm), 256, 0, s>>>(A, lda, M, K, Kpad, hi, lo, tiles_k);
    }
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

int cn_gemm_tc_launch(cn_context *ctx, int64_t M, int64_t N, int64_t K, const float *A, int64_t lda, const float *B,
                      int64_t ldb, float *C, int64_t ldc, const cn_epilogue *epi, int mode, cudaStream_t s, const cn_peer_out *peers,
                      int transA, int transB)
{
    EncodeTiledFn enc = nullptr;
    int st = get_encode_fn(ctx, &enc);
    if (st != CN_OK) return st;
    cn_gemm_workspace *ws = ctx->gemm;
    {
        unsigned int *d_status = nullptr;
        if ((st = cn_status_block(ctx, &d_status)) != CN_OK) return st;
    }
    const bool mode3x = mode == CN_GEMM_3XTF32;
    const int64_t Kpad = (K + TC_BK - 1) / TC_BK * TC_BK;

    // 1. activations -> K-major hi / lo planes (made here, or ahead of the call by cn_gemm_prepare)
    const size_t plane_elems = (size_t)M * Kpad;
    float *hi = nullptr, *lo = nullptr;
    if (ws->prepared) {
        const cn_prepared *pr = ws->prepared;
        ws->prepared = nullptr;
        CN_REQUIRE(pr->filled && pr->M == M && pr->K == K && pr->Kpad == Kpad && pr->mode == mode, CN_ERR_SHAPE,
                   "prepared activations are %lld x %lld for mode %d, the product wants %lld x %lld for mode %d", (long long)pr->M,
                   (long long)pr->K, pr->mode, (long long)M, (long long)K, mode);
        hi = pr->hi;
        lo = mode3x ? pr->lo : nullptr;
    } else {
        void *planes = nullptr;
        st = cn_gemm_scratch(ctx, CN_GEMM_SLOT_ASPLIT, plane_elems * sizeof(float) * (mode3x ? 2 : 1), &planes);
        if (st != CN_OK) return st;
        hi = (float *)planes;
        lo = mode3x ? hi + plane_elems : nullptr;
        if (ws->coded_src) {
            const int64_t tiles_k = Kpad / 32, tiles_mm = (M + 31) / 32;
            CN_REQUIRE(tiles_k * tiles_mm < (1LL << 31), CN_ERR_UNSUPPORTED, "cn_gemm_f32: activation matrix too large for the split pre-pass");
            const cn_coded_src *cs = ws->coded_src;
            ws->coded_src = nullptr;
            CN_REQUIRE(!transA && lda == M, CN_ERR_UNSUPPORTED, "coded activations must be untransposed with ld = rows");
            cn_act_split_coded_kernel<<<(unsigned)(tiles_k * tiles_mm), 256, (size_t)cs->nranks * 256 * sizeof(float), s>>>(
                cs->codes, cs->scales, ctx->d_tbl, cs->own_fp32, cs->own_rank, cs->nranks, M, K, Kpad, hi, lo, tiles_k);
            CN_CUDA(cudaGetLastError());
            cn_count_launch();
        } else if ((st = cn_gemm_tc_split_activations(ctx, transA, M, K, A, lda, hi, lo, s)) != CN_OK) {
            return st;
        }
    }

    // 2. tiling
    const int prm_maxout = epi ? epi->maxout_level : 1;
    int nt = (N >= 2048) ? 2 : 1;
    if (ws->force_nt == 1 || ws->force_nt == 2) nt = ws->force_nt;
    const int64_t tiles_n = (N + nt * TC_BN - 1) / (nt * TC_BN), tiles_m = (M + TC_BM - 1) / TC_BM;
    const int64_t tiles = tiles_n * tiles_m;
    const int kb_total = (int)(Kpad / TC_BK);
    int splits = pick_splits(tiles, kb_total, ctx->sm_count);
    if (ws->force_splits >= 1 && ws->force_splits <= kb_total) splits = ws->force_splits;
    if (prm_maxout > 1) splits = 1;   // the split-K reduction kernel has no maxout; such layers are small
    int kb_per_split = (kb_total + splits - 1) / splits;
    splits = (kb_total + kb_per_split - 1) / kb_per_split;   // no empty split
    CN_REQUIRE(tiles * splits < (1LL << 31), CN_ERR_UNSUPPORTED, "cn_gemm_f32: too many work units");

    TcParams prm;
    prm.M = M; prm.N = N; prm.K = K;
    prm.C = C; prm.ldc = ldc;
    prm.bias = epi ? epi->bias : nullptr;
    prm.act = epi ? epi->activation : CN_ACT_LINEAR;
    prm.maxout_level = epi ? epi->maxout_level : 1;
    prm.argmax = epi ? epi->argmax_out : nullptr;
    prm.tiles_n = tiles_n; prm.tiles_m = tiles_m;
    prm.splits = splits; prm.kb_per_split = kb_per_split; prm.kb_total = kb_total;
    prm.chain_kb = TC_CHAIN_DEFAULT;
    if (ws->force_chain >= 1) prm.chain_kb = ws->force_chain;
    prm.partials = nullptr;
    prm.status = ws->d_status;
    prm.npeers = 0;
    prm.ready = nullptr;
    prm.peer_flags = nullptr;
    prm.nranks = 0; prm.my_rank = 0; prm.epoch = 0;
    for (int i = 0; i < CN_MAX_PEERS; ++i) prm.peerC[i] = nullptr;
    if (peers && peers->npeers > 0) {
        prm.npeers = peers->npeers;
        for (int i = 0; i < peers->npeers; ++i) prm.peerC[i] = peers->C[i];
        prm.ready = peers->ready;
        prm.peer_flags = peers->peer_flags;
        prm.nranks = peers->nranks; prm.my_rank = peers->my_rank; prm.epoch = peers->epoch;
    }
    if (splits > 1) {
        const size_t part_bytes = (size_t)tiles * splits * nt * TC_BM * TC_BN * sizeof(float);
        void *buf = nullptr;
        st = cn_gemm_scratch(ctx, CN_GEMM_SLOT_SPLITK, part_bytes, &buf);
        if (st != CN_OK) return st;
        prm.partials = (float *)buf;
    }

    // 3. tensor maps
    CUtensorMap mw, mhi, mlo;
    if (transB) st = make_map(enc, &mw, B, N, K, ldb, true);   // stored N x K, n contiguous
    else        st = make_map(enc, &mw, B, K, N, ldb);
    if (st != CN_OK) return st;
    if ((st = make_map(enc, &mhi, hi, Kpad, M, Kpad)) != CN_OK) return st;
    if ((st = make_map(enc, &mlo, mode3x ? lo : hi, Kpad, M, Kpad)) != CN_OK) return st;

    const int64_t grid = tiles * splits;
    cudaEvent_t ev_stop = nullptr;
    if (ws->profile) {
        while (ws->prof_events.size() < ws->prof_used + 2) {
            cudaEvent_t e;
            CN_CUDA(cudaEventCreate(&e));
            ws->prof_events.push_back(e);
        }
        CN_CUDA(cudaEventRecord(ws->prof_events[ws->prof_used], s));
        ev_stop = ws->prof_events[ws->prof_used + 1];
        ws->prof_used += 2;
    }
#define CN_LAUNCH(NTV, M3, TB) launch_cfg<NTV, M3, TB>(mw, mhi, mlo, prm, grid, s)
    if (nt == 1) {
        if (transB) st = mode3x ? CN_LAUNCH(1, true, true) : CN_LAUNCH(1, false, true);
        else        st = mode3x ? CN_LAUNCH(1, true, false) : CN_LAUNCH(1, false, false);
    } else {
        if (transB) st = mode3x ? CN_LAUNCH(2, true, true) : CN_LAUNCH(2, false, true);
        else        st = mode3x ? CN_LAUNCH(2, true, false) : CN_LAUNCH(2, false, false);
    }
#undef CN_LAUNCH
    if (st != CN_OK) return st;
    if (splits > 1) {
        ReduceParams rp;
        rp.partials = prm.partials; rp.splits = splits; rp.nt = nt;
        rp.tiles_n = tiles_n; rp.tiles_m = tiles_m; rp.M = M; rp.N = N;
        rp.C = C; rp.ldc = ldc; rp.bias = prm.bias; rp.act = prm.act;
        rp.npeers = prm.npeers;
        for (int i = 0; i < CN_MAX_PEERS; ++i) rp.peerC[i] = prm.peerC[i];
        rp.ready = prm.ready; rp.nranks = prm.nranks; rp.my_rank = prm.my_rank; rp.epoch = prm.epoch; rp.status = prm.status;
        const int64_t quads = tiles * nt * (TC_BM * TC_BN / 4);
        int64_t blocks = (quads + 255) / 256, cap = (int64_t)ctx->sm_count * 8;
        cn_splitk_reduce_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, s>>>(rp);
        CN_CUDA(cudaGetLastError());
        cn_count_launch();
    }
    if (ev_stop) CN_CUDA(cudaEventRecord(ev_stop, s));
    ctx->gemm_last_path = mode3x ? "tcgen05_3xtf32" : "tcgen05_tf32";
    return CN_OK;
}

// Reads the status word that a kernel sets when one of its bounded waits ran out (0 = clean).
extern "C" int cn_gemm_check_status(cn_context *ctx, void *stream)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_gemm_check_status: null context");
    cudaStream_t s = cn_stream(stream);
    if (!ctx->gemm || !ctx->gemm->d_status) return CN_OK;
    unsigned int h = 0;
    CN_CUDA(cudaMemcpyAsync(&h, ctx->gemm->d_status, sizeof(h), cudaMemcpyDeviceToHost, s));
    CN_CUDA(cudaStreamSynchronize(s));
    if (h != 0) {
        cudaMemsetAsync(ctx->gemm->d_status, 0, sizeof(h), s);
        cn_set_error("cn_gemm_f32: a pipeline wait ran out in the tensor-core kernel (role code %u)", h);
        return CN_ERR_TIMEOUT;
    }
    return CN_OK;
}

extern "C" int cn_gemm_profile_enable(cn_context *ctx, int enable)
{
    CN_REQUIRE(ctx, CN_ERR_ARG, "cn_gemm_profile_enable: null context");
    if (!ctx->gemm) ctx->gemm = cn_gemm_workspace_new();
    ctx->gemm->profile = enable != 0;
    return CN_OK;
}

extern "C" int cn_gemm_profile_read(cn_context *ctx, float *ms_out, int max, int *count)
{
    CN_REQUIRE(ctx && count, CN_ERR_ARG, "cn_gemm_profile_read: null argument");
    *count = 0;
    if (!ctx->gemm) return CN_OK;
    cn_gemm_workspace *ws = ctx->gemm;
    const size_t pairs = ws->prof_used / 2;
    for (size_t i = 0; i < pairs; ++i) {
        CN_CUDA(cudaEventSynchronize(ws->prof_events[2 * i + 1]));
        float ms = 0.f;
        CN_CUDA(cudaEventElapsedTime(&ms, ws->prof_events[2 * i], ws->prof_events[2 * i + 1]));
        if ((int)i < max && ms_out) ms_out[i] = ms;
    }
    *count = (int)pairs;
    ws->prof_used = 0;
    return CN_OK;
}
