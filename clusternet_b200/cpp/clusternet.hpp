// Header-only C++ facade with the reference's names over the C ABI (include/clusternet_b200.h).
//
// Mirrors, for the dot / dotMPI / codec / batch path only:
//   struct Matrix + empty / zeros / ones / empty_char / empty_pinned / to_gpu / to_host   source/basicOps.cuh:25-42,44-90
//   class ClusterNet   dot, Tdot, dotT, dotMPI, rand, randn, dropout, uniformSqrtWeight, distributed_uniformSqrtWeight,
//                      distributed_zeros / ones, compression_8bit, decompression_8bit, tick, tock, shutdown_MPI,
//                      MYRANK / MPI_SIZE / MYGPUID / NODES / GPU_COUNT                    source/clusterNet.h:77-266
//   class BatchAllocator  init, broadcast_batch_to_processes, allocate_next_batch_async,
//                      replace_current_batch_with_next, CURRENT_BATCH(_Y), TOTAL_BATCHES  source/batchAllocator.h:23-108
// Conventions kept from the reference: host matrices are row-major, device matrices column-major (ld = rows);
// returning functions malloc the descriptor and cudaMalloc the payload, the caller frees with
// cudaFree(m->data); free(m); `out` overloads never allocate; errors are thrown as `const char*`.
// Differences: sizes are 64-bit; the communicator is NCCL (one process per GPU: RANK / WORLD_SIZE / LOCAL_RANK in the
// environment and a 128-byte id handed over by the launcher) instead of MPI.
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <memory>
#include <string>

#include "../../include/clusternet_b200.h"

typedef struct Matrix {
    int64_t rows;
    int64_t cols;
    size_t bytes;
    int64_t size;
    float *data;
    int isDistributed;
    int64_t cols_distributed;
    unsigned char *char_data;
} Matrix;

namespace cn_detail {
inline void check(int status)
{
    if (status != CN_OK) throw cn_last_error();
}
inline void cuda(cudaError_t e)
{
    if (e != cudaSuccess) throw cudaGetErrorString(e);
}
inline Matrix *header(int64_t rows, int64_t cols)
{
    Matrix *m = (Matrix *)malloc(sizeof(Matrix));
    memset(m, 0, sizeof(Matrix));
    m->rows = rows;
    m->cols = cols;
    m->size = rows * cols;
    m->bytes = (size_t)rows * cols * sizeof(float);
    return m;
}
}  // namespace cn_detail

inline Matrix *empty(int64_t rows, int64_t cols)
{
    Matrix *m = cn_detail::header(rows, cols);
    cn_detail::cuda(cudaMalloc((void **)&m->data, m->bytes ? m->bytes : 4));
    return m;
}
inline Matrix *empty_char(int64_t rows, int64_t cols)
{
    Matrix *m = cn_detail::header(rows, cols);
    m->bytes = (size_t)rows * cols;
    cn_detail::cuda(cudaMalloc((void **)&m->char_data, m->bytes ? m->bytes : 4));
    return m;
}
inline Matrix *empty_pinned(int64_t rows, int64_t cols)
{
    Matrix *m = cn_detail::header(rows, cols);
    cn_detail::cuda(cudaHostAlloc((void **)&m->data, m->bytes ? m->bytes : 4, cudaHostAllocPortable));
    return m;
}
inline Matrix *empty_cpu(int64_t rows, int64_t cols)
{
    Matrix *m = cn_detail::header(rows, cols);
    m->data = (float *)malloc(m->bytes ? m->bytes : 4);
    return m;
}

// read_hdf5 / write_hdf5 (source/util.cu:100-131,202-216) without libhdf5: pinned host matrix, row-major, dataset "/Default"
inline Matrix *read_hdf5(const char *filepath, const char *tag)
{
    float *data = nullptr;
    int64_t rows = 0, cols = 0;
    cn_detail::check(cn_hdf5_read_f32(filepath, tag, &data, &rows, &cols));
    Matrix *out = empty_pinned(rows, cols);
    memcpy(out->data, data, out->bytes);
    cn_host_free(data);
    return out;
}
inline Matrix *read_hdf5(const char *filepath) { return read_hdf5(filepath, "/Default"); }
inline void write_hdf5(const char *filepath, Matrix *A) { cn_detail::check(cn_hdf5_write_f32(filepath, "/Default", A->data, A->rows, A->cols)); }

class ClusterNet {
public:
    int MYRANK = 0, NODES = 1, MYGPUID = 0, MPI_SIZE = 1, GPU_COUNT = 1;
    int GEMM_MODE = CN_GEMM_3XTF32;

    // seed as in ClusterNet(int argc, char*[], int seed): per-rank stream = seed + 10000*rank + 12345
    explicit ClusterNet(int seed = 1234, const char *codebook_path = nullptr, const void *nccl_id128 = nullptr)
    {
        const char *r = getenv("RANK"), *w = getenv("WORLD_SIZE"), *l = getenv("LOCAL_RANK");
        MYRANK = r ? atoi(r) : 0;
        MPI_SIZE = w ? atoi(w) : 1;
        MYGPUID = l ? atoi(l) : 0;
        cn_detail::cuda(cudaGetDeviceCount(&GPU_COUNT));
        float tbl[126];
        const char *path = codebook_path ? codebook_path : getenv("CN_CODEBOOK");
        if (!path) throw "ClusterNet: no codebook (pass a path or set CN_CODEBOOK)";
        cn_detail::check(cn_codebook_load(path, tbl));
        cn_context *c = nullptr;
        cn_detail::check(cn_context_create(MYGPUID, tbl, &c));
        ctx_ = std::shared_ptr<cn_context>(c, [](cn_context *p) { cn_context_destroy(p); });
        if (nccl_id128 && MPI_SIZE > 1) cn_detail::check(cn_comm_init_rank(c, nccl_id128, MYRANK, MPI_SIZE));
        seed_ = (uint64_t)seed + 10000ull * MYRANK + 12345ull;
        same_seed_ = 12345ull;
    }

    cn_context *context() const { return ctx_.get(); }
    void shutdown_MPI() { cn_comm_destroy(ctx_.get()); }

    // ---- layout boundary (to_gpu / to_host)
    Matrix *to_gpu(const Matrix *host)
    {
        Matrix *out = empty(host->rows, host->cols), *stage = empty(host->rows, host->cols);
        cn_detail::check(cn_upload_row_major(ctx_.get(), host->data, stage->data, out->data, host->rows, host->cols, nullptr));
        cn_detail::cuda(cudaStreamSynchronize(nullptr));
        cudaFree(stage->data);
        free(stage);
        return out;
    }
    Matrix *to_host(const Matrix *dev)
    {
        Matrix *out = empty_cpu(dev->rows, dev->cols), *stage = empty(dev->rows, dev->cols);
        cn_detail::check(cn_download_row_major(ctx_.get(), dev->data, stage->data, out->data, dev->rows, dev->cols, nullptr));
        cn_detail::cuda(cudaStreamSynchronize(nullptr));
        cudaFree(stage->data);
        free(stage);
        return out;
    }
    Matrix *zeros(int64_t rows, int64_t cols) { return fill(rows, cols, 0.0f); }
    Matrix *ones(int64_t rows, int64_t cols) { return fill(rows, cols, 1.0f); }
    Matrix *fill(int64_t rows, int64_t cols, float v)
    {
        Matrix *m = empty(rows, cols);
        cn_detail::check(cn_fill_f32(ctx_.get(), m->data, m->size, v, nullptr));
        return m;
    }

    // ---- dot family (source/clusterNet.cpp:230-298): distributed operands route to dotMPI
    Matrix *dot(Matrix *A, Matrix *B) { Matrix *out = empty(A->rows, B->isDistributed ? B->cols_distributed : B->cols); dot(A, B, out); return out; }
    Matrix *Tdot(Matrix *A, Matrix *B) { Matrix *out = empty(A->cols, B->cols); Tdot(A, B, out); return out; }
    Matrix *dotT(Matrix *A, Matrix *B) { Matrix *out = empty(A->rows, B->rows); dotT(A, B, out); return out; }
    void dot(Matrix *A, Matrix *B, Matrix *out)
    {
        if (B->isDistributed == 1 || out->isDistributed == 1) { dotMPI(A, B, out); return; }
        gemm(A, B, out, 0, 0, nullptr);
    }
    // backward through a sharded weight: out = A . B^T summed over the ranks (source/clusterNet.cpp:511)
    Matrix *dotTMPI(Matrix *A, Matrix *B) { Matrix *out = empty(A->rows, B->rows); dotTMPI(A, B, out); return out; }
    void dotTMPI(Matrix *A, Matrix *B, Matrix *out)
    {
        if (B->isDistributed != 1) throw "dotTMPI: B must be a distributed (column-sharded) matrix";
        if (A->cols != B->cols_distributed || out->rows != A->rows || out->cols != B->rows) throw "Matrix *size* error";
        cn_detail::check(cn_dottmpi_f32(ctx_.get(), A->rows, B->cols_distributed, B->rows, A->data, B->data, out->data, GEMM_MODE, nullptr));
    }
    // gradient of a sharded weight: out_shard = A^T . B[:, shard] (source/clusterNet.cpp:510)
    void TdotMPI(Matrix *A, Matrix *B, Matrix *out)
    {
        if (out->isDistributed != 1) throw "TdotMPI: out must be a distributed (column-sharded) matrix";
        if (A->rows != B->rows || out->rows != A->cols || out->cols_distributed != B->cols) throw "Matrix *size* error";
        cn_detail::check(cn_dot_sharded_out_f32(ctx_.get(), 1, A->cols, A->rows, B->cols, A->data, B->data, out->data, GEMM_MODE, nullptr));
    }
    void Tdot(Matrix *A, Matrix *B, Matrix *out) { gemm(A, B, out, 1, 0, nullptr); }
    void dotT(Matrix *A, Matrix *B, Matrix *out) { gemm(A, B, out, 0, 1, nullptr); }
    // fused form: out = act(A.B + bias), optional maxout
    void dot(Matrix *A, Matrix *B, Matrix *out, const cn_epilogue &epi) { gemm(A, B, out, 0, 0, &epi); }

    Matrix *dotMPI(Matrix *A, Matrix *B) { Matrix *out = empty(A->rows, B->cols_distributed); dotMPI(A, B, out); return out; }
    void dotMPI(Matrix *A, Matrix *B, Matrix *out, int exchange_8bit = 0)
    {
        if (out->isDistributed == 1 && B->isDistributed != 1) {   // full B, sharded out: local product, no exchange
            if (A->cols != B->rows || out->rows != A->rows || out->cols_distributed != B->cols) throw "Matrix *size* error";
            cn_detail::check(cn_dot_sharded_out_f32(ctx_.get(), 0, A->rows, A->cols, B->cols, A->data, B->data, out->data, GEMM_MODE, nullptr));
            return;
        }
        if (B->isDistributed != 1) throw "dotMPI: B must be a distributed (column-sharded) matrix";
        if (A->cols != B->rows || out->rows != A->rows || out->cols != B->cols_distributed) throw "Matrix *size* error";
        cn_detail::check(cn_dotmpi_f32(ctx_.get(), A->rows, A->cols, B->cols_distributed, A->data, B->data, out->data, nullptr,
                                      GEMM_MODE, exchange_8bit, nullptr));
    }

    // ---- random numbers and weights
    Matrix *rand(int64_t rows, int64_t cols)
    {
        Matrix *m = empty(rows, cols);
        cn_detail::check(cn_rand_uniform(ctx_.get(), m->data, m->size, seed_, next_offset(m->size), nullptr));
        return m;
    }
    Matrix *rand_int(int64_t rows, int64_t cols, int low, int high)
    {
        Matrix *m = empty(rows, cols);
        cn_detail::check(cn_rand_int(ctx_.get(), m->data, m->size, low, high, seed_, next_offset(m->size), nullptr));
        return m;
    }
    // same numbers on every rank (the reference's second generator, seeded with 12345 everywhere)
    Matrix *rand_same_seed_MPI(int64_t rows, int64_t cols)
    {
        Matrix *m = empty(rows, cols);
        cn_detail::check(cn_rand_uniform(ctx_.get(), m->data, m->size, same_seed_, same_offset_, nullptr));
        same_offset_ += (uint64_t)(m->size + 3) / 4;
        return m;
    }
    Matrix *randn(int64_t rows, int64_t cols, float mean = 0.0f, float std = 1.0f)
    {
        Matrix *m = empty(rows, cols);
        cn_detail::check(cn_rand_normal(ctx_.get(), m->data, m->size, mean, std, seed_, next_offset(m->size), nullptr));
        return m;
    }
    Matrix *dropout(Matrix *A, float dropout_rate)
    {
        Matrix *m = empty(A->rows, A->cols);
        cn_detail::check(cn_dropout(ctx_.get(), A->data, m->data, A->size, dropout_rate, seed_, next_offset(A->size), nullptr));
        return m;
    }
    Matrix *uniformSqrtWeight(int64_t rows, int64_t cols)
    {
        Matrix *m = empty(rows, cols);
        cn_detail::check(cn_uniform_sqrt_weight(ctx_.get(), m->data, m->size, rows, cols, seed_, next_offset(m->size), nullptr));
        return m;
    }
    Matrix *uniformSqrtWeight_sameSeed(int64_t rows, int64_t cols)
    {
        Matrix *m = empty(rows, cols);
        cn_detail::check(cn_uniform_sqrt_weight(ctx_.get(), m->data, m->size, rows, cols, same_seed_, same_offset_, nullptr));
        same_offset_ += (uint64_t)(m->size + 3) / 4;
        return m;
    }
    // source/clusterNet.cpp:916-938: local shard, limits from the TOTAL column count, cols == 1 falls back to same-seed
    Matrix *distributed_uniformSqrtWeight(int64_t rows, int64_t cols)
    {
        if (cols == 1) return uniformSqrtWeight_sameSeed(rows, cols);
        int64_t start = 0, cnt = 0;
        cn_detail::check(cn_shard_cols(cols, MYRANK, MPI_SIZE, &start, &cnt));
        Matrix *m = empty(rows, cnt);
        cn_detail::check(cn_uniform_sqrt_weight(ctx_.get(), m->data, m->size, rows, cols, seed_, next_offset(m->size), nullptr));
        m->isDistributed = 1;
        m->cols_distributed = cols;
        return m;
    }
    Matrix *distributed_zeros(int64_t rows, int64_t cols) { return distributed_fill(rows, cols, 0.0f); }
    Matrix *distributed_ones(int64_t rows, int64_t cols) { return distributed_fill(rows, cols, 1.0f); }

    // ---- 8-bit codec (source/clusterNet.cpp:1384-1406)
    Matrix *compression_8bit(Matrix *A, float precision) { Matrix *out = empty_char(A->rows, A->cols); compression_8bit(A, precision, out); return out; }
    void compression_8bit(Matrix *A, float precision, Matrix *out)
    {
        cn_detail::check(cn_compress_8bit(ctx_.get(), A->data, precision, A->size, out->char_data, nullptr));
    }
    Matrix *decompression_8bit(Matrix *A, float precision) { Matrix *out = empty(A->rows, A->cols); decompression_8bit(A, precision, out); return out; }
    void decompression_8bit(Matrix *A, float precision, Matrix *out)
    {
        cn_detail::check(cn_decompress_8bit(ctx_.get(), A->char_data, precision, A->size, out->data, nullptr));
    }
    // abs() + max() of the reference in one pass; synchronises like thrust::reduce does
    float absmax(Matrix *A)
    {
        float *d = nullptr, h = 0.f;
        cn_detail::cuda(cudaMalloc((void **)&d, 4));
        cn_detail::check(cn_absmax_f32(ctx_.get(), A->data, A->size, d, nullptr));
        cn_detail::cuda(cudaMemcpy(&h, d, 4, cudaMemcpyDeviceToHost));
        cudaFree(d);
        return h;
    }

    // ---- timers
    void tick(const std::string &name = "default") { cn_detail::check(cn_tick(ctx_.get(), name.c_str(), nullptr)); }
    float tock(const std::string &name = "default")
    {
        float ms = 0.f;
        cn_detail::check(cn_tock(ctx_.get(), name.c_str(), nullptr, &ms));
        return ms;
    }

private:
    std::shared_ptr<cn_context> ctx_;   // ClusterNet objects are copied by value all over the reference's code
    uint64_t seed_ = 0, offset_ = 0, same_seed_ = 12345, same_offset_ = 0;

    uint64_t next_offset(int64_t n)
    {
        uint64_t o = offset_;
        offset_ += (uint64_t)(n + 3) / 4;   // one Philox counter yields four values
        return o;
    }
    Matrix *distributed_fill(int64_t rows, int64_t cols, float v)
    {
        int64_t start = 0, cnt = 0;
        cn_detail::check(cn_shard_cols(cols, MYRANK, MPI_SIZE, &start, &cnt));
        Matrix *m = fill(rows, cnt, v);
        m->isDistributed = 1;
        m->cols_distributed = cols;
        return m;
    }
    void gemm(Matrix *A, Matrix *B, Matrix *out, int tA, int tB, const cn_epilogue *epi)
    {
        const int64_t M = tA ? A->cols : A->rows, K = tA ? A->rows : A->cols;
        const int64_t K2 = tB ? B->cols : B->rows, N = tB ? B->rows : B->cols;
        const int64_t L = (epi && epi->maxout_level > 1) ? epi->maxout_level : 1;
        // checkMatrixOperation (source/basicOps.cu:839-933) throws on a shape mismatch before any work is queued
        if (K != K2 || out->rows != M || out->cols * L != N) throw "Matrix *size* error";
        cn_detail::check(cn_gemm_f32(ctx_.get(), tA, tB, M, N, K, A->data, A->rows, B->data, B->rows, out->data, out->rows, epi,
                                    GEMM_MODE, nullptr));
    }
};

typedef enum BatchAllocationMethod_t { Single_GPU = 0, Batch_split = 1, Distributed_weights = 2 } BatchAllocationMethod_t;

class BatchAllocator {
public:
    Matrix *CURRENT_BATCH = nullptr, *CURRENT_BATCH_Y = nullptr, *CURRENT_BATCH_CV = nullptr, *CURRENT_BATCH_CV_Y = nullptr;
    int64_t TOTAL_BATCHES = 0, TOTAL_BATCHES_CV = 0, BATCH_SIZE = 0, BATCH_SIZE_CV = 0, TRAIN_SET_ROWS = 0, CV_SET_ROWS = 0;
    bool SKIP_LAST_BATCH = false;

    // data set read from two HDF5 files (source/batchAllocator.cpp:62-99; the csv branch of the reference is not built)
    void init(std::string path_X, std::string path_y, float cross_validation_size, int64_t batch_size, int64_t cv_batch_size,
              ClusterNet *cluster, BatchAllocationMethod_t method = Single_GPU)
    {
        if (path_X.find("hdf5") == std::string::npos) throw "Only the cvs and hdf5 formats are supported!";
        init(read_hdf5(path_X.c_str()), read_hdf5(path_y.c_str()), cross_validation_size, batch_size, cv_batch_size, cluster, method);
    }

    // X, y: HOST row-major matrices holding the whole data set (source/batchAllocator.cpp:21-30,101-139)
    void init(Matrix *X, Matrix *y, float cross_validation_size, int64_t batch_size, int64_t cv_batch_size, ClusterNet *cluster,
              BatchAllocationMethod_t = Single_GPU)
    {
        BATCH_SIZE = batch_size;
        BATCH_SIZE_CV = cv_batch_size;
        TRAIN_SET_ROWS = (int64_t)ceilf(X->rows * (1.0f - cross_validation_size));
        CV_SET_ROWS = X->rows - TRAIN_SET_ROWS;
        if (BATCH_SIZE_CV > X->rows * cross_validation_size) throw "Cross validation batch size must be smaller than the cross validation set.";
        if (BATCH_SIZE > TRAIN_SET_ROWS) throw "ERROR: Batch size must be smaller than the training set.";
        cn_batch *t = nullptr, *c = nullptr;
        cn_detail::check(cn_batch_create(cluster->context(), X->data, y->data, TRAIN_SET_ROWS, X->cols, y->cols, batch_size, 0, &t));
        train_ = std::shared_ptr<cn_batch>(t, [](cn_batch *p) { cn_batch_destroy(p); });
        if (CV_SET_ROWS > 0) {
            cn_detail::check(cn_batch_create(cluster->context(), X->data + (size_t)TRAIN_SET_ROWS * X->cols,
                                            y->data + (size_t)TRAIN_SET_ROWS * y->cols, CV_SET_ROWS, X->cols, y->cols, cv_batch_size, 0, &c));
            cv_ = std::shared_ptr<cn_batch>(c, [](cn_batch *p) { cn_batch_destroy(p); });
        }
        TOTAL_BATCHES = cn_batch_total_batches(t);
        TOTAL_BATCHES_CV = c ? cn_batch_total_batches(c) : 0;
        cols_x_ = X->cols;
        cols_y_ = y->cols;
        CURRENT_BATCH = cn_detail::header(0, 0);
        CURRENT_BATCH_Y = cn_detail::header(0, 0);
        CURRENT_BATCH_CV = cn_detail::header(0, 0);
        CURRENT_BATCH_CV_Y = cn_detail::header(0, 0);
        float *dx, *dy;
        int64_t n;
        cn_detail::check(cn_batch_current(t, &dx, &dy, &n));
        publish(CURRENT_BATCH, CURRENT_BATCH_Y, dx, dy, n);
        if (c) {
            cn_detail::check(cn_batch_current(c, &dx, &dy, &n));
            publish(CURRENT_BATCH_CV, CURRENT_BATCH_CV_Y, dx, dy, n);
        }
    }
    // The host-side staging memcpy and the asynchronous copies are one step here; the first call is kept so that
    // the reference's loop (source/tests/batchAllocator_test.cu:44-76) compiles unchanged.
    void broadcast_batch_to_processes() {}
    void broadcast_batch_cv_to_processes() {}
    void allocate_next_batch_async() { cn_detail::check(cn_batch_copy_next_async(train_.get())); }
    void allocate_next_cv_batch_async() { cn_detail::check(cn_batch_copy_next_async(cv_.get())); }
    void replace_current_batch_with_next() { swap(train_.get(), CURRENT_BATCH, CURRENT_BATCH_Y, SKIP_LAST_BATCH); }
    void replace_current_cv_batch_with_next() { swap(cv_.get(), CURRENT_BATCH_CV, CURRENT_BATCH_CV_Y, false); }

private:
    std::shared_ptr<cn_batch> train_, cv_;
    int64_t cols_x_ = 0, cols_y_ = 0;

    void publish(Matrix *X, Matrix *Y, float *dx, float *dy, int64_t n)
    {
        X->rows = n; X->cols = cols_x_; X->size = n * cols_x_; X->bytes = (size_t)X->size * 4; X->data = dx;
        Y->rows = n; Y->cols = cols_y_; Y->size = n * cols_y_; Y->bytes = (size_t)Y->size * 4; Y->data = dy;
    }
    void swap(cn_batch *b, Matrix *X, Matrix *Y, bool skip_last)
    {
        float *dx, *dy;
        int64_t n;
        cn_detail::check(cn_batch_set_skip_last(b, skip_last ? 1 : 0));
        cn_detail::check(cn_batch_swap(b, nullptr, &dx, &dy, &n));
        publish(X, Y, dx, dy, n);
    }
};


// ------------------------------------------------------------------------------------------------------------
// Layer: the reference's data-parallel MLP layer (source/Layer.h, source/Layer.cpp), dense path.
//   forward           source/Layer.cpp:250-261 (+ unit_activation :147-178)   dot + bias + activation fused in one GEMM
//   backward_errors   :314-330      softmax output: out - onehot(target); hidden: dotT(next->error, w) * f'(activation)
//   backward_grads    :332-339      Tdot(activation, next->error), then the gradient exchange
//   MPI_synchronization_async + wait_for_synchronization :341-437   -> cn_grad_sync_8bit (compress, gather, decode-sum)
//   weight_update     :439-471      RMSprop_with_weight_update on the summed gradient
// As in the reference the bias is never updated (its update is commented out there), the gradient is summed over the
// ranks and not averaged, and with useDropout == false the activation is scaled by (1 - DROPOUT) instead.
// ------------------------------------------------------------------------------------------------------------
typedef enum Unittype_t { Logistic = 0, Rectified_Linear = 1, Softmax = 2, Linear = 4, Double_Rectified_Linear = 8, Input = 16 } Unittype_t;
typedef enum ParallelismType_t { None = 0, DataParallelism = 1, ModelParallelism = 2 } ParallelismType_t;
typedef enum Compression_t { bits_32 = 0, bits_8 = 1 } Compression_t;

class Layer {
public:
    Matrix *out = nullptr, *activation = nullptr, *error = nullptr, *target = nullptr, *target_matrix = nullptr;
    Matrix *w_next = nullptr, *b_next = nullptr, *w_rms_next = nullptr, *w_grad_next = nullptr;
    Layer *next = nullptr, *prev = nullptr;
    float LEARNING_RATE = 0.006f, RMSPROP_MOMENTUM = 0.9f, DROPOUT = 0.5f, MAX_GRAD_VALUE = 1.0f;
    float RUNNING_ERROR = 0.0f, RUNNING_SAMPLE_SIZE = 0.0f;
    int64_t UNITCOUNT = 0, BATCH_SIZE = 0;
    Unittype_t UNIT_TYPE = Rectified_Linear;
    ParallelismType_t PARALLELISM = None;
    Compression_t compression = bits_8;
    bool GATHER_SCALES = false;   // false: the reference's fixed MAX_GRAD_VALUE; true: per-rank absmax, gathered with the codes
    ClusterNet *GPU = nullptr;

    Layer(int64_t unitcount, int64_t start_batch_size, Unittype_t unit, ClusterNet *gpu) { init(unitcount, start_batch_size, unit, gpu); }
    Layer(int64_t unitcount, Unittype_t unit) { init(unitcount, 0, unit, nullptr); }

    void link_with_next_layer(Layer *next_layer)
    {
        next = next_layer;
        if (next->BATCH_SIZE == 0) next->BATCH_SIZE = BATCH_SIZE;
        if (!next->GPU) next->GPU = GPU;
        next->PARALLELISM = PARALLELISM;
        w_next = GPU->uniformSqrtWeight(UNITCOUNT, next->UNITCOUNT);
        w_rms_next = GPU->zeros(UNITCOUNT, next->UNITCOUNT);
        w_grad_next = GPU->zeros(UNITCOUNT, next->UNITCOUNT);
        b_next = GPU->zeros(1, next->UNITCOUNT);
        next->out = GPU->zeros(BATCH_SIZE, next->UNITCOUNT);
        next->activation = GPU->zeros(BATCH_SIZE, next->UNITCOUNT);
        next->error = GPU->zeros(BATCH_SIZE, next->UNITCOUNT);
        next->prev = this;
    }

    void forward(bool useDropout = true)
    {
        if (!prev) {   // input layer: `activation` holds the batch
            unit_activation(useDropout);
            next->forward(useDropout);
            return;
        }
        if (PARALLELISM == DataParallelism && useDropout) { prev->wait_for_synchronization(); prev->weight_update(); }
        // dot + addMatrixVector + activation: one fused GEMM; softmax and dropout follow as in unit_activation
        cn_epilogue epi;
        epi.bias = prev->b_next->data;
        epi.activation = UNIT_TYPE == Rectified_Linear ? CN_ACT_RELU : UNIT_TYPE == Logistic ? CN_ACT_LOGISTIC
                         : UNIT_TYPE == Double_Rectified_Linear ? CN_ACT_DOUBLE_RELU : CN_ACT_LINEAR;
        epi.maxout_level = 0;
        epi.argmax_out = nullptr;
        GPU->dot(prev->out, prev->w_next, UNIT_TYPE == Softmax ? out : activation, epi);
        unit_activation(useDropout);
        if (next) next->forward(useDropout);
    }

    void backward_errors()
    {
        if (!target) next->backward_errors();
        if (target) {
            if (out->cols != target->cols) {
                if (!target_matrix) target_matrix = GPU->zeros(BATCH_SIZE, out->cols);
                cn_detail::check(cn_create_t_matrix(GPU->context(), target->data, target_matrix->data, out->rows, out->cols, nullptr));
                cn_detail::check(cn_sub(GPU->context(), out->data, target_matrix->data, error->data, out->size, nullptr));
            } else {
                cn_detail::check(cn_sub(GPU->context(), activation->data, target->data, error->data, out->size, nullptr));
            }
            return;
        }
        if (UNIT_TYPE == Input) { backward_grads(); return; }
        int act = UNIT_TYPE == Rectified_Linear ? CN_ACT_RELU : UNIT_TYPE == Logistic ? CN_ACT_LOGISTIC
                  : UNIT_TYPE == Double_Rectified_Linear ? CN_ACT_DOUBLE_RELU : -1;
        if (act < 0) throw "Unknown unit";
        cn_detail::check(cn_activation_gradient(GPU->context(), activation->data, act, out->data, out->size, nullptr));
        GPU->dotT(next->error, w_next, error);
        cn_detail::check(cn_mul(GPU->context(), error->data, out->data, error->data, out->size, nullptr));
    }

    void backward_grads()
    {
        GPU->Tdot(activation, next->error, w_grad_next);
        MPI_synchronization_async();
        if (!next->target) next->backward_grads();
    }

    void MPI_synchronization_async()
    {
        if (PARALLELISM != DataParallelism) return;
        isSynchronizing = true;   // the exchange itself is queued in wait_for_synchronization, stream-ordered
    }

    void wait_for_synchronization()
    {
        if (target || !isSynchronizing || PARALLELISM != DataParallelism) return;
        if (compression == bits_8)
            cn_detail::check(cn_grad_sync_8bit(GPU->context(), w_grad_next->data, w_grad_next->size, GATHER_SCALES ? 0.0f : MAX_GRAD_VALUE, nullptr));
        else
            cn_detail::check(cn_allreduce_sum_f32(GPU->context(), w_grad_next->data, w_grad_next->size, nullptr));
        isSynchronizing = false;
    }

    void weight_update()
    {
        if (target) return;
        if (PARALLELISM != DataParallelism && next) next->weight_update();
        cn_detail::check(cn_rmsprop_update(GPU->context(), w_rms_next->data, w_grad_next->data, w_next->data, RMSPROP_MOMENTUM, LEARNING_RATE,
                                          w_next->size, nullptr));
    }

private:
    bool isSynchronizing = false;

    void init(int64_t unitcount, int64_t start_batch_size, Unittype_t unit, ClusterNet *gpu)
    {
        UNITCOUNT = unitcount;
        BATCH_SIZE = start_batch_size;
        UNIT_TYPE = unit;
        GPU = gpu;
        if (BATCH_SIZE > 0 && gpu) {
            out = gpu->zeros(BATCH_SIZE, UNITCOUNT);
            activation = gpu->zeros(BATCH_SIZE, UNITCOUNT);
        }
    }

    void unit_activation(bool useDropout)
    {
        if (UNIT_TYPE == Softmax) {
            cn_detail::check(cn_softmax(GPU->context(), out->data, out->data, out->rows, out->cols, nullptr));
            return;
        }
        if (useDropout) {
            Matrix *d = GPU->dropout(activation, DROPOUT);
            cn_detail::cuda(cudaMemcpyAsync(out->data, d->data, out->bytes, cudaMemcpyDeviceToDevice, nullptr));
            cn_detail::cuda(cudaStreamSynchronize(nullptr));
            cudaFree(d->data);
            free(d);
        } else {
            cn_detail::check(cn_scalar_mul(GPU->context(), activation->data, 1.0f - DROPOUT, out->data, out->size, nullptr));
        }
    }
};
