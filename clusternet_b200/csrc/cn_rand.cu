// Counter-based random numbers (Philox-4x32-10, written from the published algorithm) for rand, randn,
// dropout and weight creation.  Replaces the cuRAND XORWOW host generator of ClusterNet::rand /
// randn / dropout / uniformSqrtWeight (source/clusterNet.cpp:746-796,842-894) and
// kCreateRdmSqrtWeight_Logistic (source/clusterKernels.cu:126-138).  Element i of a stream is a pure
// function of (seed, offset + i / 4, i % 4), so results do not depend on the launch geometry and a
// column shard can be generated on its own rank without generating the columns before it.
#include "cn_internal.h"

#define PHILOX_M0 0xD2511F53u
#define PHILOX_M1 0xCD9E8D57u
#define PHILOX_W0 0x9E3779B9u
#define PHILOX_W1 0xBB67AE85u

__device__ __forceinline__ uint4 philox4x32_10(uint64_t counter, uint64_t seed)
{
    uint32_t c0 = (uint32_t)counter, c1 = (uint32_t)(counter >> 32), c2 = 0u, c3 = 0u;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(PHILOX_M0, c0), lo0 = PHILOX_M0 * c0;
        const uint32_t hi1 = __umulhi(PHILOX_M1, c2), lo1 = PHILOX_M1 * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0; c1 = lo1; c2 = n2; c3 = lo0;
        k0 += PHILOX_W0; k1 += PHILOX_W1;
    }
    return make_uint4(c0, c1, c2, c3);
}

// uniform in (0, 1], the range of curandGenerateUniform that the reference's kernels assume
__device__ __forceinline__ float u01(uint32_t x) { return fmaf((float)x, 2.3283064365386963e-10f, 2.3283064365386963e-10f * 0.5f); }

enum { RAND_UNIFORM = 0, RAND_NORMAL = 1, RAND_SQRT_WEIGHT = 2, RAND_DROPOUT = 3, RAND_INT = 4 };

template <int KIND>
__global__ void cn_rand_kernel(const float *__restrict__ A, float *__restrict__ out, int64_t n, uint64_t seed_arg, uint64_t offset,
                               float p0, float p1, const uint64_t *__restrict__ d_seed)
{
    const uint64_t seed = d_seed ? *d_seed : seed_arg;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t ngroups = (n + 3) >> 2;
    for (int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; g < ngroups; g += stride) {
        const uint4 r = philox4x32_10(offset + (uint64_t)g, seed);
        float v[4] = {u01(r.x), u01(r.y), u01(r.z), u01(r.w)};
        if (KIND == RAND_NORMAL) {
            // Box-Muller on the two pairs
            const float r0 = sqrtf(-2.0f * logf(v[0])), r1 = sqrtf(-2.0f * logf(v[2]));
            float s0, c0, s1, c1;
            sincospif(2.0f * v[1], &s0, &c0);
            sincospif(2.0f * v[3], &s1, &c1);
            v[0] = fmaf(r0 * c0, p1, p0); v[1] = fmaf(r0 * s0, p1, p0);
            v[2] = fmaf(r1 * c1, p1, p0); v[3] = fmaf(r1 * s1, p1, p0);
        }
        const int64_t i0 = g << 2;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int64_t i = i0 + k;
            if (i >= n) break;
            if (KIND == RAND_SQRT_WEIGHT) out[i] = p0 + v[k] * p1;            // lower + u * range, as the reference kernel
            else if (KIND == RAND_DROPOUT) out[i] = v[k] > p0 ? A[i] : 0.0f;  // kDropout: keep where u > rate, no rescale
            else if (KIND == RAND_INT) out[i] = fminf((float)((int)(v[k] * p1)) + p0, p0 + p1 - 1.0f);   // kRandInt; u == 1 stays in range
            else out[i] = v[k];
        }
    }
}

template <int KIND>
static int rand_launch(cn_context *ctx, const float *A, float *out, int64_t n, uint64_t seed, uint64_t offset, float p0, float p1, void *stream,
                       const uint64_t *d_seed = nullptr)
{
    CN_REQUIRE(ctx && n >= 0 && (n == 0 || out), CN_ERR_ARG, "rand: bad argument");
    if (n == 0) return CN_OK;
    int64_t blocks = ((n + 3) / 4 + 255) / 256;
    int64_t cap = (int64_t)ctx->sm_count * 8;
    cn_rand_kernel<KIND><<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, cn_stream(stream)>>>(A, out, n, seed, offset, p0, p1, d_seed);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}

extern "C" int cn_rand_uniform(cn_context *ctx, float *d_A, int64_t n, uint64_t seed, uint64_t offset, void *stream)
{
    return rand_launch<RAND_UNIFORM>(ctx, nullptr, d_A, n, seed, offset, 0.f, 0.f, stream);
}

extern "C" int cn_rand_normal(cn_context *ctx, float *d_A, int64_t n, float mean, float std, uint64_t seed, uint64_t offset, void *stream)
{
    return rand_launch<RAND_NORMAL>(ctx, nullptr, d_A, n, seed, offset, mean, std, stream);
}

extern "C" int cn_uniform_sqrt_weight(cn_context *ctx, float *d_A, int64_t n, int64_t fan_in, int64_t fan_out_total,
                                      uint64_t seed, uint64_t offset, void *stream)
{
    CN_REQUIRE(fan_in + fan_out_total > 0, CN_ERR_ARG, "cn_uniform_sqrt_weight: fan_in + fan_out must be positive");
    // limits as in kCreateRdmSqrtWeight_Logistic: +-4*sqrtf(6/((float)in + out))
    const float lim = 4.0f * sqrtf(6.0f / ((float)fan_in + (float)fan_out_total));
    const float lower = -lim, range = lim - lower;
    return rand_launch<RAND_SQRT_WEIGHT>(ctx, nullptr, d_A, n, seed, offset, lower, range, stream);
}

extern "C" int cn_dropout(cn_context *ctx, const float *d_A, float *d_out, int64_t n, float rate, uint64_t seed, uint64_t offset, void *stream)
{
    CN_REQUIRE(n == 0 || d_A, CN_ERR_ARG, "cn_dropout: null input");
    return rand_launch<RAND_DROPOUT>(ctx, d_A, d_out, n, seed, offset, rate, 0.f, stream);
}

// rand_int (source/clusterNet.cpp:790-796, kRandInt source/clusterKernels.cu:159-170): integers low..high as floats,
// (int)(u * (high - low + 1)) + low.  The reference lets u == 1.0 produce high + 1; here that one value maps to high.
extern "C" int cn_rand_int(cn_context *ctx, float *d_A, int64_t n, int low, int high, uint64_t seed, uint64_t offset, void *stream)
{
    CN_REQUIRE(high >= low, CN_ERR_ARG, "cn_rand_int: high < low");
    return rand_launch<RAND_INT>(ctx, nullptr, d_A, n, seed, offset, (float)low, (float)(high - low + 1), stream);
}

// dropout whose seed lives in device memory, so that a step captured once (for instance in a CUDA graph) draws new
// masks every time it runs: cn_seed_advance bumps the seed on the stream.
extern "C" int cn_dropout_dp(cn_context *ctx, const float *d_A, float *d_out, int64_t n, float rate, const uint64_t *d_seed, uint64_t offset, void *stream)
{
    CN_REQUIRE(d_seed, CN_ERR_ARG, "cn_dropout_dp: null seed pointer");
    CN_REQUIRE(n == 0 || d_A, CN_ERR_ARG, "cn_dropout_dp: null input");
    return rand_launch<RAND_DROPOUT>(ctx, d_A, d_out, n, 0, offset, rate, 0.f, stream, d_seed);
}

__global__ void cn_seed_advance_kernel(uint64_t *seed) { *seed += 0x9E3779B97F4A7C15ull; }

extern "C" int cn_seed_advance(cn_context *ctx, uint64_t *d_seed, void *stream)
{
    CN_REQUIRE(ctx && d_seed, CN_ERR_ARG, "cn_seed_advance: null argument");
    cn_seed_advance_kernel<<<1, 1, 0, cn_stream(stream)>>>(d_seed);
    CN_CUDA(cudaGetLastError());
    cn_count_launch();
    return CN_OK;
}
