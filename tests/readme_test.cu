// The reference's README snippets and the dotMPI / free-function checks of its own suites, written against the facade:
// runs as one process, or as one process per GPU with RANK / WORLD_SIZE / LOCAL_RANK / CN_NCCL_ID_FILE set.
//   README.md:8-31                      dot / dotMPI, the batch loop, the two-layer distributed-weight example
//   tests/clusterNet_test.cu:257-394    dotMPI == dot on constants; shard shapes; 8783 / 317 / 17 on all-ones operands
//   tests/basicOps_test.cu              slice / stack / elementwise / activation / softmax / maxout free functions
// usage: readme_test <scratch dir>      (codebook from CN_CODEBOOK)
#include <math.h>
#include <cmath>
#include <stdio.h>

#include <string>
#include <vector>

#include "../clusternet_b200/cpp/clusternet.hpp"

#define CHECK(cond)                                                     \
    do {                                                                \
        if (!(cond)) {                                                  \
            printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);    \
            return 1;                                                   \
        }                                                               \
    } while (0)

static bool all_equal(Matrix *host, float v)
{
    for (int64_t i = 0; i < host->size; ++i)
        if (host->data[i] != v) return false;
    return true;
}
static bool shape_is(Matrix *m, int64_t rows, int64_t cols) { return m->rows == rows && m->cols == cols && m->size == rows * cols; }
static Matrix *host_matrix(int64_t rows, int64_t cols, float (*f)(int64_t, int64_t))
{
    Matrix *m = empty_cpu(rows, cols);
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) m->data[r * cols + c] = f(r, c);
    return m;
}

int main(int argc, char **argv)
{
    setvbuf(stdout, nullptr, _IONBF, 0);
    try {
        ClusterNet gpus = ClusterNet(argc, argv, 12346);
        const int G = gpus.MPI_SIZE, me = gpus.MYRANK;
        const std::string dir = argc > 1 ? argv[1] : ".";

        // ---- dotMPI == dot for a weight every rank holds in full
        Matrix *m1 = scalarMul(ones(200, 400), 0.3f);
        Matrix *m2 = scalarAdd(ones(400, 800), 0.1748345f);
        Matrix *m3 = to_host(gpus.dot(m1, m2));
        Matrix *m4 = to_host(gpus.dotMPI(m1, m2));
        CHECK(shape_is(m3, 200, 800) && shape_is(m4, 200, 800));
        const float expect = 400.0f * 0.3f * 1.1748345f;
        for (int64_t i = 0; i < m3->size; ++i) {
            CHECK(fabsf(m3->data[i] - m4->data[i]) <= 4e-6f * expect);   // the shard's K split may differ from the full product's
            CHECK(fabsf(m3->data[i] - expect) < 1e-3f);
        }

        // ---- shard shapes and value ranges of distributed weights
        const int64_t shapes[3][2] = {{10000, 1000}, {100, 10}, {7833, 83}};
        for (auto &sh : shapes) {
            const int64_t rows = sh[0], cols = sh[1];
            const int64_t mine = me < G - 1 ? cols / G : cols - (cols / G) * (G - 1);
            Matrix *w = gpus.distributed_uniformSqrtWeight(rows, cols);
            CHECK(shape_is(w, rows, mine) && w->isDistributed == 1 && w->cols_distributed == cols);
            Matrix *wh = to_host(w);
            const float lim = 4.0f * sqrtf(6.0f / (float)(rows + cols));
            int zero_count = 0;
            for (int64_t i = 0; i < wh->size; ++i) {
                CHECK(wh->data[i] >= -lim && wh->data[i] <= lim);   // u in (0, 1]: the upper limit itself can be drawn
                zero_count += wh->data[i] == 0.0f;
            }
            CHECK(zero_count < 10);
            Matrix *z = to_host(gpus.distributed_zeros(rows, cols));
            CHECK(shape_is(z, rows, mine) && all_equal(z, 0.0f));
        }

        // ---- all-ones products through a sharded weight: forward, backward through the weight, weight gradient
        for (int epoch = 0; epoch < 3; ++epoch) {
            Matrix *w = gpus.distributed_zeros(8783, 317);
            scalarAdd(w, 1.0f, w);
            CHECK(all_equal(to_host(w), 1.0f));
            Matrix *a = ones(111, 8783), *e = ones(17, 317), *at = ones(8783, 17);
            Matrix *fwd = to_host(gpus.dot(a, w));              // routed to dotMPI because w is distributed
            CHECK(shape_is(fwd, 111, 317) && all_equal(fwd, 8783.0f));
            Matrix *bwd = to_host(gpus.dotTMPI(e, w));
            CHECK(shape_is(bwd, 17, 8783) && all_equal(bwd, 317.0f));
            gpus.dot(at, e, w);                                  // sharded output: every rank fills its own columns
            CHECK(all_equal(to_host(w), 17.0f));
            Matrix *w2 = gpus.distributed_ones(8783, 317);
            CHECK(all_equal(to_host(gpus.dotMPI(a, w2)), 8783.0f));
            gpus.dotMPI(at, e, w2);
            CHECK(all_equal(to_host(w2), 17.0f));
        }

        // ---- the README's two-layer example at a size a test can afford, against the single-GPU product of the same data
        {
            Matrix *batch = gpus.rand_same_seed_MPI(128, 4096);
            Matrix *W1 = gpus.distributed_uniformSqrtWeight(4096, 2048);
            Matrix *W2 = gpus.distributed_uniformSqrtWeight(2048, 1024);
            Matrix *out1 = empty(128, 2048), *out2 = empty(128, 1024);
            gpus.tick("Time taken");
            gpus.dotMPI(batch, W1, out1);
            gpus.dotMPI(out1, W2, out2);
            const float ms = gpus.tock("Time taken");
            CHECK(ms > 0.0f);
            // my columns of out1 must equal batch . W1_shard computed locally
            Matrix *local = to_host(gpus.dot(batch, W1));        // W1 distributed -> the same gathered product again
            Matrix *o1 = to_host(out1);
            for (int64_t i = 0; i < o1->size; ++i) CHECK(o1->data[i] == local->data[i]);
            Matrix *o2 = to_host(out2);
            double norm = 0.0;
            for (int64_t i = 0; i < o2->size; ++i) norm += (double)o2->data[i] * o2->data[i];
            CHECK(norm > 0.0 && std::isfinite(norm));
        }

        // ---- free functions (column-major device matrices, row-major host matrices)
        {
            Matrix *h = host_matrix(5, 7, [](int64_t r, int64_t c) { return (float)(r * 7 + c) - 12.0f; });
            Matrix *d = to_gpu(h);
            Matrix *back = to_host(d);
            for (int64_t i = 0; i < h->size; ++i) CHECK(back->data[i] == h->data[i]);
            Matrix *t = to_host(T(d));
            CHECK(shape_is(t, 7, 5));
            for (int64_t r = 0; r < 5; ++r)
                for (int64_t c = 0; c < 7; ++c) CHECK(t->data[c * 5 + r] == h->data[r * 7 + c]);
            Matrix *sc = to_host(slice_cols(d, 2, 4));
            CHECK(shape_is(sc, 5, 3));
            for (int64_t r = 0; r < 5; ++r)
                for (int64_t c = 0; c < 3; ++c) CHECK(sc->data[r * 3 + c] == h->data[r * 7 + c + 2]);
            Matrix *sr = to_host(slice_rows(d, 1, 3));
            CHECK(shape_is(sr, 3, 7));
            for (int64_t r = 0; r < 3; ++r)
                for (int64_t c = 0; c < 7; ++c) CHECK(sr->data[r * 7 + c] == h->data[(r + 1) * 7 + c]);
            Matrix *parts[3] = {slice_cols(d, 0, 1), slice_cols(d, 2, 3), slice_cols(d, 4, 6)};   // 2 + 2 + remainder 3
            Matrix *stacked = empty(5, 7);
            hStackN(parts, 10, stacked, 3);
            Matrix *sh = to_host(stacked);
            for (int64_t i = 0; i < h->size; ++i) CHECK(sh->data[i] == h->data[i]);
            Matrix *hs = to_host(hStack(parts[0], parts[1]));
            CHECK(shape_is(hs, 5, 4) && hs->data[0] == h->data[0] && hs->data[3] == h->data[3]);

            Matrix *ab = to_host(abs(d)), *sq = to_host(square(d)), *rl = to_host(rectified_linear(d));
            Matrix *dr = to_host(doubleRectifiedLinear(scalarMul(d, 0.1f))), *lg = to_host(logistic(d)), *lu = to_host(LinearUnit(d));
            Matrix *rd = to_host(rectified_linear_derivative(d)), *lgg = to_host(logisticGrad(logistic(d)));
            Matrix *s2 = to_host(sub(add(d, d), d)), *ml = to_host(mul(d, d)), *dv = to_host(div(d, scalarAdd(abs(d), 1.0f)));
            for (int64_t i = 0; i < h->size; ++i) {
                const float x = h->data[i];
                CHECK(ab->data[i] == fabsf(x) && sq->data[i] == x * x && rl->data[i] == (x > 0.f ? x : 0.f) && lu->data[i] == x);
                const float x10 = x * 0.1f;
                CHECK(dr->data[i] == (x10 < 0.f ? 0.f : (x10 > 1.f ? 1.f : x10)));
                CHECK(fabsf(lg->data[i] - 1.0f / (1.0f + expf(-x))) < 1e-6f);
                CHECK(rd->data[i] == (x > 0.f ? 1.f : 0.f));
                CHECK(fabsf(lgg->data[i] - lg->data[i] * (1.0f - lg->data[i])) < 1e-6f);
                CHECK(s2->data[i] == x && ml->data[i] == x * x);
                CHECK(fabsf(dv->data[i] - x / (fabsf(x) + 1.0f)) < 1e-6f);
            }
            CHECK(max(d) == 22.0f);                                   // largest element of h
            CHECK(max(scalarAdd(zeros(3, 3), -5.0f)) == -1.0f);       // the reduction is seeded with -1
            Matrix *bias = to_gpu(host_matrix(1, 7, [](int64_t, int64_t c) { return 100.0f * (float)c; }));
            Matrix *av = to_host(addMatrixVector(d, bias));
            for (int64_t r = 0; r < 5; ++r)
                for (int64_t c = 0; c < 7; ++c) CHECK(av->data[r * 7 + c] == h->data[r * 7 + c] + 100.0f * (float)c);

            Matrix *sm = to_host(softmax(d));
            for (int64_t r = 0; r < 5; ++r) {
                float sum = 0.f;
                for (int64_t c = 0; c < 7; ++c) sum += sm->data[r * 7 + c];
                CHECK(fabsf(sum - 1.0f) < 1e-5f && sm->data[r * 7 + 6] > sm->data[r * 7 + 5]);
            }
            Matrix *labels = to_gpu(host_matrix(6, 1, [](int64_t r, int64_t) { return (float)((r * 3) % 4); }));
            Matrix *onehot = to_host(create_t_matrix(labels, 4));
            for (int64_t r = 0; r < 6; ++r)
                for (int64_t c = 0; c < 4; ++c) CHECK(onehot->data[r * 4 + c] == (c == (r * 3) % 4 ? 1.0f : 0.0f));

            // maxout over groups of 4 consecutive columns: value and the winning column's index
            Matrix *mh = host_matrix(3, 8, [](int64_t r, int64_t c) { return (float)((c * 5 + r * 3) % 8); });
            Matrix **mo = maxout(to_gpu(mh), 4);
            Matrix *mv = to_host(mo[0]), *mi = to_host(mo[1]);
            CHECK(shape_is(mv, 3, 2));
            for (int64_t r = 0; r < 3; ++r)
                for (int64_t g = 0; g < 2; ++g) {
                    float best = -1.f;
                    int64_t arg = -1;
                    for (int64_t c = g * 4; c < g * 4 + 4; ++c)
                        if (mh->data[r * 8 + c] > best) { best = mh->data[r * 8 + c]; arg = c; }
                    CHECK(mv->data[r * 2 + g] == best && mi->data[r * 2 + g] == (float)arg);
                }

            // optimiser steps against the formulas of the reference's kernels
            Matrix *w = to_gpu(host_matrix(4, 4, [](int64_t r, int64_t c) { return 0.5f + 0.01f * (float)(r * 4 + c); }));
            Matrix *g = to_gpu(host_matrix(4, 4, [](int64_t r, int64_t c) { return 0.25f - 0.03f * (float)(r * 4 + c); }));
            Matrix *rms = zeros(4, 4), *mom = zeros(4, 4);
            Matrix *w0 = to_host(w), *g0 = to_host(g);
            RMSprop_with_weight_update(rms, g, w, mom, 0.9f, 0.003f, 128, 0.5f);
            Matrix *w1 = to_host(w), *r1 = to_host(rms);
            for (int64_t i = 0; i < 16; ++i) {
                const float r = 0.1f * g0->data[i] * g0->data[i];
                CHECK(fabsf(r1->data[i] - r) < 1e-7f);
                CHECK(fabsf(w1->data[i] - (w0->data[i] - 0.003f * g0->data[i] / (sqrtf(r) + 1e-8f))) < 1e-6f);
            }
            Nesterov_weight_update(rms, g, w, mom, 0.9f, 0.1f, 4, 0.5f);
            Matrix *w2 = to_host(w), *mm = to_host(mom);
            for (int64_t i = 0; i < 16; ++i) {
                const float step = 0.1f * g0->data[i] / 4.0f;
                CHECK(fabsf(mm->data[i] + step) < 1e-7f && fabsf(w2->data[i] - (w1->data[i] - step)) < 1e-6f);
            }

            // codec through the free functions: same codes as through the ClusterNet methods
            Matrix *x = gpus.randn(64, 64);
            Matrix *c1 = empty_char(64, 64), *c2 = gpus.compression_8bit(x, 4.0f);
            compression_8bit(nullptr, x, 4.0f, c1);
            std::vector<unsigned char> b1(4096), b2(4096);
            cn_detail::cuda(cudaMemcpy(b1.data(), c1->char_data, 4096, cudaMemcpyDefault));
            cn_detail::cuda(cudaMemcpy(b2.data(), c2->char_data, 4096, cudaMemcpyDefault));
            CHECK(b1 == b2);
            Matrix *y1 = empty(64, 64);
            decompression_8bit(nullptr, c1, 4.0f, y1);
            Matrix *y1h = to_host(y1), *y2h = to_host(gpus.decompression_8bit(c2, 4.0f));
            for (int64_t i = 0; i < 4096; ++i) CHECK(y1h->data[i] == y2h->data[i]);
        }

        // ---- the README's batch loop
        {
            const int64_t rows = 1000, cols = 32;
            Matrix *X = empty_pinned(rows, cols), *y = empty_pinned(rows, 1);
            for (int64_t i = 0; i < rows * cols; ++i) X->data[i] = (float)(i % 977) * 0.001f;
            for (int64_t i = 0; i < rows; ++i) y->data[i] = (float)(i % 10);
            Matrix *w1 = gpus.uniformSqrtWeight(cols, 16);
            Matrix *w1h = to_host(w1);
            gpus.init_batch_allocator(X, y, 128);
            CHECK(gpus.m_total_batches == 8);
            int64_t row0 = 0;
            for (int i = 0; i < gpus.m_total_batches; i++) {
                gpus.allocate_next_batch_async();
                Matrix *result = to_host(gpus.dot(gpus.m_current_batch_X, w1));
                const int64_t n = gpus.m_current_batch_X->rows;
                CHECK(n == (i < 7 ? 128 : 1000 - 7 * 128) && result->rows == n);
                for (int64_t r = 0; r < n; r += 17) {   // spot rows against a host dot product
                    double acc = 0.0;
                    for (int64_t k = 0; k < cols; ++k) acc += (double)X->data[(row0 + r) * cols + k] * w1h->data[k * 16 + 3];
                    CHECK(fabs(acc - result->data[r * 16 + 3]) < 1e-4);
                }
                row0 += n;
                gpus.replace_current_batch_with_next();
            }
            CHECK(row0 == rows);
        }

        gpus.shutdown_MPI();
        printf("rank %d of %d: All tests passed\n", me, G);
        return 0;
    } catch (const char *msg) {
        printf("exception: %s\n", msg);
        return 2;
    }
}
