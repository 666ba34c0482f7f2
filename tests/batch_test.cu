// The reference's batch allocator suite (tests/batchAllocator_test.cu:12-207) at its own sizes, written against the
// facade: arange data sets of 10000 x 784 (+ 10000 x 1 labels) and 70000 x 784 (+ 70000 x 10), 20 % held out, so that
// every element of every batch equals a running counter; two epochs; short last batches; the counters must end at
// 6 272 000 / 8 000 / 7 840 000 / 10 000 and 43 904 000 / 560 000 / 54 880 000 / 700 000.  One allocator serves its
// own process (5-argument init), the other is in Distributed_weights mode, once in each of its two forms: only rank 0's
// data are used and every batch reaches the other GPUs by broadcast; or every process holds the data set (as the
// processes of the reference's own test do), uploads its share of the rows of each batch and the GPUs exchange the
// blocks (EVERY_RANK_HOLDS_DATA).
// Runs as one process, or one per GPU with RANK / WORLD_SIZE / LOCAL_RANK / CN_NCCL_ID_FILE / CN_CODEBOOK set.
#include <stdio.h>

#include "../clusternet_b200/cpp/clusternet.hpp"

#define CHECK(cond)                                                     \
    do {                                                                \
        if (!(cond)) {                                                  \
            printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);    \
            return 1;                                                   \
        }                                                               \
    } while (0)

static bool shape_is(Matrix *m, int64_t rows, int64_t cols) { return m->rows == rows && m->cols == cols; }
static void release(Matrix *host)
{
    free(host->data);
    free(host);
}

// walks `batches` batches of both allocators and advances the two counters; returns false on the first mismatch
static bool walk(BatchAllocator &b, BatchAllocator &b_dist, bool cv, int64_t full, int64_t rest, int64_t cols_y, int64_t &value, int64_t &value_y)
{
    const int64_t batches = cv ? b.TOTAL_BATCHES_CV : b.TOTAL_BATCHES;
    for (int64_t batchno = 0; batchno < batches; ++batchno) {
        Matrix *cur = cv ? b.CURRENT_BATCH_CV : b.CURRENT_BATCH, *cur_y = cv ? b.CURRENT_BATCH_CV_Y : b.CURRENT_BATCH_Y;
        Matrix *dcur = cv ? b_dist.CURRENT_BATCH_CV : b_dist.CURRENT_BATCH, *dcur_y = cv ? b_dist.CURRENT_BATCH_CV_Y : b_dist.CURRENT_BATCH_Y;
        const int64_t want_rows = (batchno + 1 < batches || rest == 0) ? full : rest;
        if (cur->rows != want_rows || dcur->rows != want_rows || cur->cols != 784 || dcur_y->cols != cols_y) return false;
        Matrix *h = to_host(cur), *h2 = to_host(cur_y), *hd = to_host(dcur), *hd2 = to_host(dcur_y);
        if (cv) { b.broadcast_batch_cv_to_processes(); b_dist.broadcast_batch_cv_to_processes(); }
        else { b.broadcast_batch_to_processes(); b_dist.broadcast_batch_to_processes(); }
        for (int64_t i = 0; i < cur->rows * 784; ++i, ++value)
            if (h->data[i] != (float)value || hd->data[i] != (float)value) return false;
        if (cv) { b.allocate_next_cv_batch_async(); b_dist.allocate_next_cv_batch_async(); }
        else { b.allocate_next_batch_async(); b_dist.allocate_next_batch_async(); }
        for (int64_t i = 0; i < cur->rows * cols_y; ++i, ++value_y)
            if (h2->data[i] != (float)value_y || hd2->data[i] != (float)value_y) return false;
        if (cv) { b.replace_current_cv_batch_with_next(); b_dist.replace_current_cv_batch_with_next(); }
        else { b.replace_current_batch_with_next(); b_dist.replace_current_batch_with_next(); }
        release(h); release(h2); release(hd); release(hd2);
    }
    return true;
}

int main(int argc, char **argv)
{
    setvbuf(stdout, nullptr, _IONBF, 0);
    try {
        ClusterNet gpus = ClusterNet(argc, argv, 12345);
        struct Case { int64_t rows, cols_y, batch, cv_batch, train_total, train_total_y, all_total, all_total_y; };
        const Case cases[2] = {{10000, 1, 128, 256, 6272000, 8000, 7840000, 10000}, {70000, 10, 128, 512, 43904000, 560000, 54880000, 700000}};
        for (int form = 0; form < 4; ++form) {
            const Case &c = cases[form & 1];
            const bool every_rank_holds = form >= 2;
            // every rank builds the data for its own allocator; the broadcasting form only looks at rank 0's copy
            Matrix *m1 = to_host(arange(c.rows, 784)), *m2 = to_host(arange(c.rows, c.cols_y));
            Matrix *junk1 = empty_cpu(1, 1), *junk2 = empty_cpu(1, 1);
            const bool other = gpus.MYRANK != 0 && !every_rank_holds;
            BatchAllocator b = BatchAllocator();
            b.init(m1, m2, 0.20f, c.batch, c.cv_batch);
            BatchAllocator b_dist = BatchAllocator();
            b_dist.EVERY_RANK_HOLDS_DATA = every_rank_holds;
            b_dist.init(other ? junk1 : m1, other ? junk2 : m2, 0.2f, c.batch, c.cv_batch, &gpus, Distributed_weights);
            const int64_t train = c.rows * 8 / 10, held = c.rows - train;
            CHECK(b.TRAIN_SET_ROWS == train && b_dist.TRAIN_SET_ROWS == train && b_dist.CV_SET_ROWS == held);
            CHECK(shape_is(b.CURRENT_BATCH, c.batch, 784) && shape_is(b.CURRENT_BATCH_Y, c.batch, c.cols_y));
            CHECK(shape_is(b.CURRENT_BATCH_CV, c.cv_batch, 784) && shape_is(b.CURRENT_BATCH_CV_Y, c.cv_batch, c.cols_y));
            CHECK(shape_is(b_dist.CURRENT_BATCH, c.batch, 784) && shape_is(b_dist.CURRENT_BATCH_Y, c.batch, c.cols_y));
            CHECK(shape_is(b_dist.CURRENT_BATCH_CV, c.cv_batch, 784) && shape_is(b_dist.CURRENT_BATCH_CV_Y, c.cv_batch, c.cols_y));
            int64_t value = 0, value_y = 0;
            for (int epoch = 0; epoch < 2; ++epoch) {
                value = 0;
                value_y = 0;
                CHECK(walk(b, b_dist, false, c.batch, train % c.batch, c.cols_y, value, value_y));
                CHECK(value == c.train_total && value_y == c.train_total_y);
                CHECK(walk(b, b_dist, true, c.cv_batch, held % c.cv_batch, c.cols_y, value, value_y));
            }
            CHECK(value == c.all_total && value_y == c.all_total_y);
        }
        gpus.shutdown_MPI();
        printf("rank %d of %d: All tests passed\n", gpus.MYRANK, gpus.MPI_SIZE);
        return 0;
    } catch (const char *msg) {
        printf("exception: %s\n", msg);
        return 2;
    }
}
