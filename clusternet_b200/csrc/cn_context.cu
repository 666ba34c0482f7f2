// Context, error reporting, codebook loading, compressor threshold derivation, timers.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>
#include "cn_internal.h"

#include <atomic>
static thread_local char g_err[512] = "";
static std::atomic<unsigned long long> g_launches{0};

void cn_count_launch(void) { g_launches.fetch_add(1, std::memory_order_relaxed); }
extern "C" uint64_t cn_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

void cn_set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int cn_cuda_fail(cudaError_t e, const char *what)
{
    cn_set_error("CUDA error %d (%s) in %s", (int)e, cudaGetErrorString(e), what);
    return CN_ERR_CUDA;
}

extern "C" const char *cn_last_error(void) { return g_err; }

extern "C" const char *cn_status_string(int s)
{
    switch (s) {
        case CN_OK: return "CN_OK";
        case CN_ERR_ARG: return "CN_ERR_ARG";
        case CN_ERR_SHAPE: return "CN_ERR_SHAPE";
        case CN_ERR_CUDA: return "CN_ERR_CUDA";
        case CN_ERR_NCCL: return "CN_ERR_NCCL";
        case CN_ERR_TIMEOUT: return "CN_ERR_TIMEOUT";
        case CN_ERR_UNSUPPORTED: return "CN_ERR_UNSUPPORTED";
        case CN_ERR_NOMEM: return "CN_ERR_NOMEM";
    }
    return "CN_ERR_?";
}

extern "C" int cn_version(void) { return 100; }
extern "C" int cn_compiled_arch(void) { return 100; }

// ------------------------------------------------------------------------------------------------
// Codebook file.  The reference loads dataset "/Default" of source/8bit_floats.hdf5 through libhdf5
// (source/clusterNet.cpp:73, source/util.cu:100-131).  That file is a version-0 HDF5 container whose
// only dataset (126 x 1 float32, little endian, contiguous layout) occupies the last 504 bytes, so
// the payload is read from the tail after checking the container signature.  A raw 504-byte dump of
// the table is accepted as well.
// ------------------------------------------------------------------------------------------------
extern "C" int cn_codebook_load(const char *path, float *tbl)
{
    CN_REQUIRE(path && tbl, CN_ERR_ARG, "cn_codebook_load: null argument");
    static const unsigned char sig[8] = {0x89, 'H', 'D', 'F', '\r', '\n', 0x1a, '\n'};
    FILE *f = fopen(path, "rb");
    CN_REQUIRE(f, CN_ERR_ARG, "cn_codebook_load: cannot open %s", path);
    fseek(f, 0, SEEK_END);
    long size = ftell(f);
    const long payload = CN_CODEBOOK_N * 4;
    if (size == payload) {
        fseek(f, 0, SEEK_SET);
    } else {
        unsigned char head[8];
        fseek(f, 0, SEEK_SET);
        if (size < 8 + payload || fread(head, 1, 8, f) != 8 || memcmp(head, sig, 8) != 0) {
            fclose(f);
            cn_set_error("cn_codebook_load: %s is neither an HDF5 container nor a 504-byte table", path);
            return CN_ERR_ARG;
        }
        fseek(f, size - payload, SEEK_SET);
    }
    size_t got = fread(tbl, 4, CN_CODEBOOK_N, f);
    fclose(f);
    CN_REQUIRE(got == CN_CODEBOOK_N, CN_ERR_ARG, "cn_codebook_load: short read from %s", path);
    for (int i = 0; i < CN_CODEBOOK_N; ++i) {
        bool ok = tbl[i] > 0.f && tbl[i] < 1.f && (i == 0 || tbl[i] > tbl[i - 1]);
        CN_REQUIRE(ok, CN_ERR_ARG, "cn_codebook_load: entry %d of %s is not an increasing value in (0,1)", i, path);
    }
    return CN_OK;
}

// ------------------------------------------------------------------------------------------------
// Compressor decision function on a magnitude a = |x / precision| that is not NaN.
// Follows kCompression_8bit (source/clusterKernels.cu:1189-1229): two range tests, a six-step search
// that visits odd table indices starting at 63, then a nearest-of-two pick between the final (even)
// pivot and its lower neighbour.  Index 126 is outside the 126-entry table; the reference reads an
// unwritten shared-memory word there, this code takes it as +infinity (=> index 125 is chosen).
// ------------------------------------------------------------------------------------------------
static inline float tbl_at(const float *tbl, int i) { return i < CN_CODEBOOK_N ? tbl[i] : INFINITY; }

static uint8_t code_of_magnitude(const float *tbl, float a)
{
    const float threshold_lower = 0.0000015;
    const float threshold_upper = 0.995703;
    if (a < threshold_lower) return 254;
    if (a > threshold_upper) return 127;
    int pivot = 63, upper = 125, lower = 0;
    for (int j = 32; j > 0; j >>= 1) {
        if (a > tbl_at(tbl, pivot)) { lower = pivot; pivot += j; }
        else                        { upper = pivot; pivot -= j; }
    }
    float tp = tbl_at(tbl, pivot);
    if (lower == pivot) return (uint8_t)(fabsf(tp - a) < (tbl[upper] - a) ? pivot : upper);
    return (uint8_t)((tp - a) < fabsf(tbl[lower] - a) ? pivot : lower);
}

static inline int level_of_code(uint8_t c) { return c == 254 ? 0 : (c == 127 ? 127 : (int)c + 1); }

extern "C" int cn_codec_build_thresholds(const float *tbl, uint32_t *thr, uint8_t *level_codes)
{
    CN_REQUIRE(tbl && thr && level_codes, CN_ERR_ARG, "cn_codec_build_thresholds: null argument");
    for (int i = 0; i < CN_CODEBOOK_N; ++i) {
        bool ok = tbl[i] > 0.f && tbl[i] < 1.f && (i == 0 || tbl[i] > tbl[i - 1]);
        CN_REQUIRE(ok, CN_ERR_ARG, "codebook entry %d is not an increasing value in (0,1)", i);
    }
    level_codes[0] = 254;
    for (int i = 0; i < CN_CODEBOOK_N; ++i) level_codes[i + 1] = (uint8_t)i;
    level_codes[127] = 127;
    // The code is a non-decreasing step function of the magnitude (both rounded differences in the
    // pick move monotonically with a), so each level boundary is found by bisection on the ordered
    // fp32 bit patterns 0 .. +inf.
    for (int j = 1; j <= CN_NUM_THR; ++j) {
        uint32_t lo = 0, hi = 0x7f800000u;
        while (lo < hi) {
            uint32_t mid = lo + ((hi - lo) >> 1);
            float a;
            memcpy(&a, &mid, 4);
            if (level_of_code(code_of_magnitude(tbl, a)) >= j) hi = mid; else lo = mid + 1;
        }
        thr[j - 1] = lo;
    }
    // Spot-check the bisection's premise on both sides of every boundary and on the table values.
    for (int j = 0; j < CN_NUM_THR; ++j) {
        for (int d = -2; d <= 2; ++d) {
            int64_t ub = (int64_t)thr[j] + d;
            if (ub < 0 || ub > 0x7f800000LL) continue;
            uint32_t u = (uint32_t)ub;
            float a;
            memcpy(&a, &u, 4);
            int cnt = 0;
            for (int k = 0; k < CN_NUM_THR; ++k) cnt += thr[k] <= u;
            CN_REQUIRE(level_codes[cnt] == code_of_magnitude(tbl, a), CN_ERR_UNSUPPORTED,
                       "codebook yields a non-monotone decision function near threshold %d", j);
        }
    }
    return CN_OK;
}

// ------------------------------------------------------------------------------------------------
extern "C" int cn_context_create(int device, const float *codebook, cn_context **out)
{
    CN_REQUIRE(out && codebook, CN_ERR_ARG, "cn_context_create: null argument");
    *out = nullptr;
    int ndev = 0;
    CN_CUDA(cudaGetDeviceCount(&ndev));
    CN_REQUIRE(device >= 0 && device < ndev, CN_ERR_ARG, "cn_context_create: device %d of %d", device, ndev);
    CN_CUDA(cudaSetDevice(device));
    cudaDeviceProp prop;
    CN_CUDA(cudaGetDeviceProperties(&prop, device));
    CN_REQUIRE(prop.major == 10, CN_ERR_UNSUPPORTED,
               "this library holds sm_100a code only; device %d is sm_%d%d", device, prop.major, prop.minor);
    cn_context *c = new cn_context();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    memcpy(c->h_tbl, codebook, CN_CODEBOOK_N * sizeof(float));
    c->h_tbl[126] = INFINITY;
    c->h_tbl[127] = INFINITY;
    int st = cn_codec_build_thresholds(codebook, c->h_thr, c->h_level_codes);
    if (st != CN_OK) { delete c; return st; }
    c->h_thr[127] = 0xffffffffu;
    cudaError_t e;
    if ((e = cudaMalloc(&c->d_tbl, 128 * sizeof(float))) != cudaSuccess ||
        (e = cudaMalloc(&c->d_thr, 128 * sizeof(uint32_t))) != cudaSuccess ||
        (e = cudaMalloc(&c->d_level_codes, 128)) != cudaSuccess ||
        (e = cudaMalloc(&c->d_partials, CN_MAX_PARTIALS * sizeof(float))) != cudaSuccess ||
        (e = cudaMalloc(&c->d_ticket, 64)) != cudaSuccess ||
        (e = cudaMemcpy(c->d_tbl, c->h_tbl, 128 * sizeof(float), cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemcpy(c->d_thr, c->h_thr, 128 * sizeof(uint32_t), cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemcpy(c->d_level_codes, c->h_level_codes, 128, cudaMemcpyHostToDevice)) != cudaSuccess ||
        (e = cudaMemset(c->d_ticket, 0, 64)) != cudaSuccess) {
        cn_context_destroy(c);
        return cn_cuda_fail(e, "cn_context_create");
    }
    *out = c;
    return CN_OK;
}

extern "C" int cn_context_destroy(cn_context *c)
{
    if (!c) return CN_OK;
    cudaSetDevice(c->device);
    cn_comm_state_free(c);
    cn_gemm_workspace_free(c);
    for (auto &kv : c->timers) {
        if (kv.second.start) cudaEventDestroy(kv.second.start);
        if (kv.second.stop) cudaEventDestroy(kv.second.stop);
    }
    cudaFree(c->d_tbl);
    cudaFree(c->d_thr);
    cudaFree(c->d_level_codes);
    cudaFree(c->d_partials);
    cudaFree(c->d_ticket);
    delete c;
    return CN_OK;
}

extern "C" int cn_context_device(const cn_context *c) { return c ? c->device : -1; }

// ------------------------------------------------------------------------------------------------
// Named cumulative timers (ClusterNet::tick / tock, source/clusterNet.cpp:798-840): tick records a
// start event on the stream; tock records the stop event, waits for it and adds the elapsed
// milliseconds to the named total, which it returns.
// ------------------------------------------------------------------------------------------------
extern "C" int cn_tick(cn_context *c, const char *name, void *stream)
{
    CN_REQUIRE(c && name, CN_ERR_ARG, "cn_tick: null argument");
    cn_timer_slot &t = c->timers[name];
    if (!t.start) {
        CN_CUDA(cudaEventCreate(&t.start));
        CN_CUDA(cudaEventCreate(&t.stop));
    }
    CN_CUDA(cudaEventRecord(t.start, cn_stream(stream)));
    return CN_OK;
}

extern "C" int cn_tock(cn_context *c, const char *name, void *stream, float *cumulative_ms)
{
    CN_REQUIRE(c && name, CN_ERR_ARG, "cn_tock: null argument");
    auto it = c->timers.find(name);
    CN_REQUIRE(it != c->timers.end() && it->second.start, CN_ERR_ARG, "cn_tock: no tick for '%s'", name);
    cn_timer_slot &t = it->second;
    CN_CUDA(cudaEventRecord(t.stop, cn_stream(stream)));
    CN_CUDA(cudaEventSynchronize(t.stop));
    float ms = 0.f;
    CN_CUDA(cudaEventElapsedTime(&ms, t.start, t.stop));
    t.cumulative_ms += ms;
    if (cumulative_ms) *cumulative_ms = t.cumulative_ms;
    return CN_OK;
}
