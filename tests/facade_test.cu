// Drives the C++ facade the way the reference's own suites drive ClusterNet / BatchAllocator
// (tests/clusterNet_test.cu:16-84,106-129,158-165,257-276,279-314; tests/batchAllocator_test.cu:22-114) and prints
// "All tests passed" (tests/testSuite.cu:24).  Built and run by tests/test_facade_gpu.py.
#include <assert.h>
#include <stdio.h>

#include <vector>

#include "../clusternet_b200/cpp/clusternet.hpp"

#define CHECK(cond)                                                        \
    do {                                                                   \
        if (!(cond)) {                                                     \
            printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);       \
            return 1;                                                      \
        }                                                                  \
    } while (0)

static Matrix *host_matrix(int64_t rows, int64_t cols, const float *data)
{
    Matrix *m = empty_cpu(rows, cols);
    memcpy(m->data, data, m->bytes);
    return m;
}

int main(int argc, char **argv)
{
    try {
        ClusterNet gpu(132456, argc > 1 ? argv[1] : nullptr);
        gpu.tick();
        // ---- dot / Tdot / dotT known answers, float equality as in the reference
        float m1_data[6] = {0, 2, 3, 0, 0.83f, 59.1387f};
        float m2_data[6] = {17, 0, 3, 4, 0, 0};
        Matrix *m1 = gpu.to_gpu(host_matrix(2, 3, m1_data)), *m2 = gpu.to_gpu(host_matrix(3, 2, m2_data));
        Matrix *h = gpu.to_host(gpu.dot(m1, m2));
        CHECK(h->rows == 2 && h->cols == 2 && h->data[0] == 6.0f && h->data[1] == 8.0f && h->data[2] == 2.49f && h->data[3] == 3.32f);
        Matrix *out = gpu.zeros(3, 3);
        gpu.Tdot(m1, m1, out);
        h = gpu.to_host(out);
        CHECK(h->data[0] == 0.0f && h->data[4] == 4.6889f && h->data[5] == 55.085117f && h->data[7] == 55.085117f && h->data[8] == 3506.385742f);
        out = gpu.zeros(2, 2);
        gpu.dotT(m1, m1, out);
        h = gpu.to_host(out);
        CHECK(h->data[0] == 13.0f && h->data[1] == 179.0761f && h->data[2] == 179.0761f && h->data[3] == 3498.074463f);
        bool threw = false;
        try { gpu.dot(m1, m1); } catch (const char *) { threw = true; }
        CHECK(threw);

        // ---- dotMPI == dot, elementwise exact (single rank here; multi-rank is covered by tests/test_dist.py)
        Matrix *A = gpu.fill(200, 400, 0.3f), *B = gpu.fill(400, 800, 1.1748345f);
        Matrix *Bd = gpu.distributed_ones(400, 800);
        cn_fill_f32(gpu.context(), Bd->data, Bd->size, 1.1748345f, nullptr);
        Matrix *c1 = gpu.to_host(gpu.dot(A, B)), *c2 = gpu.to_host(gpu.dot(A, Bd));   // dot routes to dotMPI
        for (int64_t i = 0; i < c1->size; ++i) CHECK(c1->data[i] == c2->data[i]);
        CHECK(fabsf(c1->data[0] - 140.98014f) < 1e-3f);

        // ---- distributed weights: shard shape and the +-4*sqrt(6/(in+out)) range
        Matrix *W = gpu.distributed_uniformSqrtWeight(784, 1200);
        CHECK(W->isDistributed == 1 && W->cols_distributed == 1200 && W->rows == 784 && W->cols == 1200 / gpu.MPI_SIZE);
        Matrix *Wh = gpu.to_host(W);
        float lim = 4.0f * sqrtf(6.0f / (784.0f + 1200.0f)), mx = 0.f;
        for (int64_t i = 0; i < Wh->size; ++i) { CHECK(fabsf(Wh->data[i]) <= lim); mx = fmaxf(mx, fabsf(Wh->data[i])); }
        CHECK(mx > 0.99f * lim);

        // ---- codec: absmax -> compress -> decompress
        Matrix *g = gpu.randn(512, 300, 0.0f, 0.1f);
        float p = gpu.absmax(g);
        Matrix *codes = gpu.compression_8bit(g, p), *back = gpu.to_host(gpu.decompression_8bit(codes, p)), *gh = gpu.to_host(g);
        float worst = 0.f;
        // values below 1.5e-6 * precision take code 254, which the reference's decoder maps to +precision: leave them out
        for (int64_t i = 0; i < gh->size; ++i)
            if (fabsf(gh->data[i]) > 2e-6f * p) worst = fmaxf(worst, fabsf(gh->data[i] - back->data[i]));
        CHECK(worst <= 0.0175f * p + 1.6e-6f * p);

        // ---- BatchAllocator: arange data, running counter over two epochs, short last batch
        const int64_t rows = 1000, cols = 16;
        Matrix *X = empty_pinned(rows, cols), *y = empty_pinned(rows, 1);
        for (int64_t i = 0; i < rows * cols; ++i) X->data[i] = (float)i;
        for (int64_t i = 0; i < rows; ++i) y->data[i] = (float)i;
        BatchAllocator b;
        b.init(X, y, 0.2f, 128, 64, &gpu, Single_GPU);
        CHECK(b.TRAIN_SET_ROWS == 800 && b.CV_SET_ROWS == 200 && b.TOTAL_BATCHES == 7 && b.TOTAL_BATCHES_CV == 4);
        for (int epoch = 0; epoch < 2; ++epoch) {
            int64_t counter = 0;
            for (int64_t i = 0; i < b.TOTAL_BATCHES; ++i) {
                b.broadcast_batch_to_processes();
                b.allocate_next_batch_async();
                CHECK(b.CURRENT_BATCH->rows == (i < 6 ? 128 : 800 % 128));
                Matrix *hb = gpu.to_host(b.CURRENT_BATCH);
                for (int64_t e = 0; e < hb->size; ++e) CHECK(hb->data[e] == (float)(counter + e));
                counter += hb->size;
                b.replace_current_batch_with_next();
            }
            CHECK(counter == 800 * cols);
        }
        Matrix *hcv = gpu.to_host(b.CURRENT_BATCH_CV);
        CHECK(hcv->rows == 64 && hcv->data[0] == (float)(800 * cols));

        // ---- the same data set through files: write_hdf5, then BatchAllocator::init(path_X, path_y, ...)
        if (argc > 3) {
            // the reference's own fixture and check (tests/util_test.cu:18-20): element i of the h5py file is i
            Matrix *F = read_hdf5(argv[3]);
            CHECK(F->rows == 10 && F->cols == 50);
            for (int64_t i = 0; i < F->size; ++i) CHECK(F->data[i] == (float)i);
            if (argc > 4) {   // CSR fixture of the reference (tests/util_test.cu:22-44)
                Matrix *S = read_sparse_hdf5(argv[4]);
                CHECK(S->isSparse == 1 && S->rows == 10 && S->cols == 50 && S->size == 499 && S->ptr_bytes == 11 * sizeof(int));
                for (int64_t i = 0; i < S->size; ++i) CHECK(S->data[i] == (float)(i + 1) && S->idx_cols[i] == (int)((i + 1) % 50));
                for (int r = 0; r <= 10; ++r) CHECK(S->ptr_rows[r] == (r == 0 ? 0 : 50 * r - 1));
            }
            const std::string px = std::string(argv[2]) + "/X.hdf5", py = std::string(argv[2]) + "/y.hdf5";
            write_hdf5(px.c_str(), X);
            write_hdf5(py.c_str(), y);
            BatchAllocator fb;
            fb.init(px, py, 0.2f, 128, 64, &gpu, Single_GPU);
            CHECK(fb.TRAIN_SET_ROWS == 800 && fb.TOTAL_BATCHES == 7);
            fb.broadcast_batch_to_processes();
            fb.allocate_next_batch_async();
            fb.replace_current_batch_with_next();
            Matrix *hb = gpu.to_host(fb.CURRENT_BATCH), *hy = gpu.to_host(fb.CURRENT_BATCH_Y);
            CHECK(hb->rows == 128 && hb->cols == cols && hy->rows == 128);
            for (int64_t e = 0; e < hb->size; ++e) CHECK(hb->data[e] == (float)(128 * cols + e));
            for (int64_t e = 0; e < hy->size; ++e) CHECK(hy->data[e] == (float)(128 + e));
            bool threw = false;
            try { fb.init(std::string("X.bin"), py, 0.2f, 128, 64, &gpu, Single_GPU); } catch (const char *) { threw = true; }
            CHECK(threw);
        }
        CHECK(gpu.tock() > 0.0f);
        printf("All tests passed\n");
        return 0;
    } catch (const char *msg) {
        printf("exception: %s\n", msg);
        return 2;
    }
}
