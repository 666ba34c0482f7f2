// Several GPUs driven from ONE process (cn_comm_init_all): the sharded product with one host thread per rank, and with
// a single thread that brackets the per-rank calls with cn_group_start / cn_group_end.  Checks: dotMPI == dot
// elementwise on the constant matrices of the reference's own test (tests/clusterNet_test.cu:257-276), a random product
// with uneven shards against an fp64 host product, the 8-bit exchange (own block exact), and an all-reduce.
// Usage: initall_test <codebook file>      (needs at least two GPUs; prints "SKIP" and exits 0 otherwise)
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "../include/clusternet_b200.h"

#define CHECK(cond)                                                                                   \
    do {                                                                                              \
        if (!(cond)) {                                                                                \
            printf("FAILED %s:%d: %s   [%s]\n", __FILE__, __LINE__, #cond, cn_last_error());          \
            exit(1);                                                                                  \
        }                                                                                             \
    } while (0)
#define OK(call) CHECK((call) == CN_OK)

static float *dev_copy(const std::vector<float> &h)
{
    float *d = nullptr;
    CHECK(cudaMalloc(&d, h.size() * sizeof(float)) == cudaSuccess);
    CHECK(cudaMemcpy(d, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess);
    return d;
}
static std::vector<float> host_copy(const float *d, size_t n)
{
    std::vector<float> h(n);
    CHECK(cudaMemcpy(h.data(), d, n * sizeof(float), cudaMemcpyDeviceToHost) == cudaSuccess);
    return h;
}

int main(int argc, char **argv)
{
    setvbuf(stdout, nullptr, _IONBF, 0);
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev < 2 || argc < 2) {
        printf("SKIP: needs two GPUs and a codebook path\n");
        return 0;
    }
    const int G = ndev < 4 ? ndev : 4;
    float tbl[126];
    OK(cn_codebook_load(argv[1], tbl));
    std::vector<cn_context *> ctx(G, nullptr);
    for (int r = 0; r < G; ++r) OK(cn_context_create(r, tbl, &ctx[r]));
    OK(cn_comm_init_all(ctx.data(), G));
    for (int r = 0; r < G; ++r) CHECK(cn_comm_rank(ctx[r]) == r && cn_comm_size(ctx[r]) == G);

    // ---- data: column-major A (M x K), full W (K x N) on the host, uneven shards
    const int64_t M = 128, K = 512, N = 1000 + G + 1;
    std::vector<float> hA(M * K), hW(K * N), hConstA(200 * 400, 0.3f), hConstB(400 * 800, 1.1748345f);
    uint32_t seed = 12345u;
    auto rnd = [&]() { seed = seed * 1664525u + 1013904223u; return (float)(seed >> 8) * (2.0f / 16777216.0f) - 1.0f; };
    for (auto &v : hA) v = rnd();
    for (auto &v : hW) v = rnd();
    std::vector<double> ref(M * N, 0.0);
    for (int64_t n = 0; n < N; ++n)
        for (int64_t k = 0; k < K; ++k) {
            const double w = hW[k + n * K];
            for (int64_t m = 0; m < M; ++m) ref[m + n * M] += (double)hA[m + k * M] * w;
        }
    double ref_max = 0.0;
    for (double v : ref) ref_max = fmax(ref_max, fabs(v));

    std::vector<float *> dA(G), dW(G), dC(G), dC8(G), dCA(G), dCB(G), dCC(G), dRed(G);
    std::vector<int64_t> start(G), cnt(G), cstart(G), ccnt(G);
    for (int r = 0; r < G; ++r) {
        OK(cn_context_make_current(ctx[r]));
        OK(cn_shard_cols(N, r, G, &start[r], &cnt[r]));
        OK(cn_shard_cols(800, r, G, &cstart[r], &ccnt[r]));
        dA[r] = dev_copy(hA);
        dW[r] = dev_copy(std::vector<float>(hW.begin() + K * start[r], hW.begin() + K * (start[r] + cnt[r])));
        dCA[r] = dev_copy(hConstA);
        dCB[r] = dev_copy(std::vector<float>(hConstB.begin() + 400 * cstart[r], hConstB.begin() + 400 * (cstart[r] + ccnt[r])));
        CHECK(cudaMalloc(&dC[r], M * N * sizeof(float)) == cudaSuccess);
        CHECK(cudaMalloc(&dC8[r], M * N * sizeof(float)) == cudaSuccess);
        CHECK(cudaMalloc(&dCC[r], 200 * 800 * sizeof(float)) == cudaSuccess);
        dRed[r] = dev_copy(std::vector<float>(1000, (float)(r + 1)));
    }
    // single-GPU product of the constant matrices (the comparison value of dotMPI == dot)
    OK(cn_context_make_current(ctx[0]));
    float *dFullB = dev_copy(hConstB), *dFullC = nullptr;
    CHECK(cudaMalloc(&dFullC, 200 * 800 * sizeof(float)) == cudaSuccess);
    OK(cn_gemm_f32(ctx[0], 0, 0, 200, 800, 400, dCA[0], 200, dFullB, 400, dFullC, 200, nullptr, CN_GEMM_3XTF32, nullptr));
    CHECK(cudaDeviceSynchronize() == cudaSuccess);
    const std::vector<float> hFull = host_copy(dFullC, 200 * 800);

    // ---- one host thread per rank: every entry point works as with one process per GPU
    {
        std::vector<std::thread> th;
        for (int r = 0; r < G; ++r)
            th.emplace_back([&, r]() {
                OK(cn_context_make_current(ctx[r]));
                OK(cn_dotmpi_f32(ctx[r], M, K, N, dA[r], dW[r], dC[r], nullptr, CN_GEMM_3XTF32, 0, nullptr));
                OK(cn_dotmpi_f32(ctx[r], M, K, N, dA[r], dW[r], dC8[r], nullptr, CN_GEMM_3XTF32, 1, nullptr));
                OK(cn_dotmpi_f32(ctx[r], 200, 400, 800, dCA[r], dCB[r], dCC[r], nullptr, CN_GEMM_3XTF32, 0, nullptr));
                OK(cn_allreduce_sum_f32(ctx[r], dRed[r], 1000, nullptr));
                OK(cn_gemm_check_status(ctx[r], nullptr));
                CHECK(cudaDeviceSynchronize() == cudaSuccess);
            });
        for (auto &t : th) t.join();
    }
    for (int r = 0; r < G; ++r) {
        OK(cn_context_make_current(ctx[r]));
        const std::vector<float> c = host_copy(dC[r], M * N), c8 = host_copy(dC8[r], M * N), cc = host_copy(dCC[r], 200 * 800);
        double err = 0.0;
        for (int64_t i = 0; i < M * N; ++i) err = fmax(err, fabs((double)c[i] - ref[i]));
        CHECK(err / ref_max < 1e-5);
        for (int64_t i = 0; i < 200 * 800; ++i) CHECK(cc[i] == hFull[i]);                    // dotMPI == dot, elementwise
        for (int64_t i = M * start[r]; i < M * (start[r] + cnt[r]); ++i) CHECK(c8[i] == c[i]);   // own block stays exact fp32
        // the peers' blocks went through the 8-bit codec: each equals decompress(compress(block, absmax(block))) computed
        // with the single-GPU entry points (the committed decode of the special codes included)
        for (int q = 0; q < G; ++q) {
            if (q == r) continue;
            const int64_t nblk = M * cnt[q];
            float *d_blk = dev_copy(std::vector<float>(c.begin() + M * start[q], c.begin() + M * (start[q] + cnt[q])));
            float *d_scale = nullptr, *d_back = nullptr;
            uint8_t *d_codes = nullptr;
            CHECK(cudaMalloc(&d_scale, 4) == cudaSuccess && cudaMalloc(&d_back, nblk * 4) == cudaSuccess && cudaMalloc(&d_codes, nblk) == cudaSuccess);
            OK(cn_absmax_f32(ctx[r], d_blk, nblk, d_scale, nullptr));
            OK(cn_compress_8bit_dp(ctx[r], d_blk, d_scale, nblk, d_codes, nullptr));
            OK(cn_decompress_8bit_dp(ctx[r], d_codes, d_scale, nblk, d_back, nullptr));
            CHECK(cudaDeviceSynchronize() == cudaSuccess);
            const std::vector<float> want = host_copy(d_back, nblk);
            for (int64_t i = 0; i < nblk; ++i) CHECK(c8[M * start[q] + i] == want[i]);
            cudaFree(d_blk); cudaFree(d_scale); cudaFree(d_back); cudaFree(d_codes);
        }
        const std::vector<float> red = host_copy(dRed[r], 1000);
        CHECK(red[0] == (float)(G * (G + 1) / 2) && red[999] == red[0]);
    }

    // ---- one thread drives all ranks: the per-rank calls of a collective inside a group
    std::vector<std::vector<float>> threaded(G);
    for (int r = 0; r < G; ++r) {
        OK(cn_context_make_current(ctx[r]));
        threaded[r] = host_copy(dC[r], M * N);
        CHECK(cudaMemset(dC[r], 0, M * N * sizeof(float)) == cudaSuccess);
        CHECK(cudaMemcpy(dRed[r], std::vector<float>(1000, (float)(r + 1)).data(), 1000 * sizeof(float), cudaMemcpyHostToDevice) == cudaSuccess);
    }
    OK(cn_group_start());
    for (int r = 0; r < G; ++r) {
        OK(cn_context_make_current(ctx[r]));
        OK(cn_dotmpi_f32(ctx[r], M, K, N, dA[r], dW[r], dC[r], nullptr, CN_GEMM_3XTF32, 0, nullptr));
    }
    OK(cn_group_end());
    OK(cn_group_start());
    for (int r = 0; r < G; ++r) {
        OK(cn_context_make_current(ctx[r]));
        OK(cn_allreduce_sum_f32(ctx[r], dRed[r], 1000, nullptr));
    }
    OK(cn_group_end());
    for (int r = 0; r < G; ++r) {
        OK(cn_context_make_current(ctx[r]));
        CHECK(cudaDeviceSynchronize() == cudaSuccess);
        const std::vector<float> c = host_copy(dC[r], M * N);
        for (int64_t i = 0; i < M * N; ++i) CHECK(c[i] == threaded[r][i]);
        CHECK(host_copy(dRed[r], 1000)[5] == (float)(G * (G + 1) / 2));
        // symmetric buffers need one process per GPU: a clear refusal, not a crash
        void *p = nullptr;
        CHECK(cn_sym_alloc(ctx[r], 4096, &p) == CN_ERR_UNSUPPORTED);
    }
    for (int r = 0; r < G; ++r) {
        OK(cn_comm_destroy(ctx[r]));
        OK(cn_context_destroy(ctx[r]));
    }
    printf("All tests passed (%d GPUs in one process)\n", G);
    return 0;
}
