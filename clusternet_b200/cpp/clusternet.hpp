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

#include <stdio.h>
#include <unistd.h>

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
    // CSR fields of the reference's descriptor (source/basicOps.cuh:25-42); only read_sparse_hdf5 fills them here, every
    // compute function takes dense matrices (isSparse == 0)
    int isSparse;
    size_t ptr_bytes;
    size_t idx_bytes;
    int *ptr_rows;
    int *idx_cols;
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
// The reference's free functions (zeros, to_gpu, add, ...) work on "the current device" without naming an object; here
// they use the context of the most recently constructed ClusterNet, or one made on first use from CN_CODEBOOK.
inline std::shared_ptr<cn_context> &current_slot()
{
    static std::shared_ptr<cn_context> slot;
    return slot;
}
inline cn_context *current()
{
    std::shared_ptr<cn_context> &slot = current_slot();
    if (!slot) {
        const char *path = getenv("CN_CODEBOOK");
        if (!path) throw "clusternet: construct a ClusterNet or set CN_CODEBOOK before calling the free functions";
        float tbl[126];
        check(cn_codebook_load(path, tbl));
        int dev = 0;
        cuda(cudaGetDevice(&dev));
        cn_context *c = nullptr;
        check(cn_context_create(dev, tbl, &c));
        slot = std::shared_ptr<cn_context>(c, [](cn_context *p) { cn_context_destroy(p); });
    }
    return slot.get();
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
    int64_t rows = 0, cols = 0;
    cn_detail::check(cn_hdf5_dims(filepath, tag, &rows, &cols));
    Matrix *out = empty_pinned(rows, cols);
    cn_detail::check(cn_hdf5_read_f32_into(filepath, tag, out->data, out->size));
    return out;
}
inline Matrix *read_hdf5(const char *filepath) { return read_hdf5(filepath, "/Default"); }
// read_sparse_hdf5 (source/util.cu:133-198): CSR matrix from /data, /indices, /indptr, /shape into pinned host memory
inline Matrix *read_sparse_hdf5(const char *filepath)
{
    float *data = nullptr;
    int32_t *idx = nullptr, *ptr = nullptr, *shape = nullptr;
    int64_t n = 0, nidx = 0, nptr = 0, nshape = 0, one = 0;
    cn_detail::check(cn_hdf5_read_f32(filepath, "/data", &data, &n, &one));
    cn_detail::check(cn_hdf5_read_i32(filepath, "/indices", &idx, &nidx, &one));
    cn_detail::check(cn_hdf5_read_i32(filepath, "/indptr", &ptr, &nptr, &one));
    cn_detail::check(cn_hdf5_read_i32(filepath, "/shape", &shape, &nshape, &one));
    if (nshape != 2 || nidx != n || nptr != shape[0] + 1) throw "read_sparse_hdf5: inconsistent CSR datasets";
    Matrix *out = cn_detail::header(shape[0], shape[1]);
    out->isSparse = 1;
    out->size = n;
    out->bytes = (size_t)n * sizeof(float);
    out->idx_bytes = (size_t)nidx * sizeof(int);
    out->ptr_bytes = (size_t)nptr * sizeof(int);
    cn_detail::cuda(cudaHostAlloc((void **)&out->data, out->bytes ? out->bytes : 4, cudaHostAllocPortable));
    cn_detail::cuda(cudaHostAlloc((void **)&out->idx_cols, out->idx_bytes ? out->idx_bytes : 4, cudaHostAllocPortable));
    cn_detail::cuda(cudaHostAlloc((void **)&out->ptr_rows, out->ptr_bytes, cudaHostAllocPortable));
    memcpy(out->data, data, out->bytes);
    memcpy(out->idx_cols, idx, out->idx_bytes);
    memcpy(out->ptr_rows, ptr, out->ptr_bytes);
    cn_host_free(data);
    cn_host_free(idx);
    cn_host_free(ptr);
    cn_host_free(shape);
    return out;
}
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
        cn_detail::current_slot() = ctx_;
        if (nccl_id128 && MPI_SIZE > 1) cn_detail::check(cn_comm_init_rank(c, nccl_id128, MYRANK, MPI_SIZE));
        seed_ = (uint64_t)seed + 10000ull * MYRANK + 12345ull;
        same_seed_ = 12345ull;
    }
    // ClusterNet(argc, argv, seed) / ClusterNet(argc, argv) of the reference (source/clusterNet.cpp:11-36), which call
    // init_MPI: here one process per GPU with RANK / WORLD_SIZE / LOCAL_RANK in the environment (as torchrun or mpirun
    // wrappers set them), the codebook from CN_CODEBOOK, and the communicator id handed from rank 0 to the others
    // through the file named by CN_NCCL_ID_FILE (a path all ranks of the node can reach; written once, atomically).
    ClusterNet(int /*argc*/, char ** /*argv*/, int seed = 1234) : ClusterNet(seed, nullptr, nullptr)
    {
        if (MPI_SIZE > 1) init_comm_from_file();
    }

    cn_context *context() const { return ctx_.get(); }
    void shutdown_MPI() { cn_comm_destroy(ctx_.get()); }

    // ---- batch allocator spelled as in the reference's README (gpu.init_batch_allocator(X, y, 128); gpu.m_total_batches;
    //      gpu.allocate_next_batch_async(); gpu.m_current_batch_X; gpu.replace_current_batch_with_next()); bodies below
    Matrix *m_current_batch_X = nullptr, *m_current_batch_y = nullptr;
    int64_t m_total_batches = 0;
    inline void init_batch_allocator(Matrix *X, Matrix *y, int64_t batch_size);
    inline void allocate_next_batch_async();
    inline void replace_current_batch_with_next();

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

    Matrix *dotMPI(Matrix *A, Matrix *B) { Matrix *out = empty(A->rows, B->isDistributed == 1 ? B->cols_distributed : B->cols); dotMPI(A, B, out); return out; }
    void dotMPI(Matrix *A, Matrix *B, Matrix *out, int exchange_8bit = 0)
    {
        if (out->isDistributed == 1 && B->isDistributed != 1) {   // full B, sharded out: local product, no exchange
            if (A->cols != B->rows || out->rows != A->rows || out->cols_distributed != B->cols) throw "Matrix *size* error";
            cn_detail::check(cn_dot_sharded_out_f32(ctx_.get(), 0, A->rows, A->cols, B->cols, A->data, B->data, out->data, GEMM_MODE, nullptr));
            return;
        }
        if (B->isDistributed != 1) {   // full B on every rank: each rank multiplies its own column block of it (:612-619)
            if (A->cols != B->rows || out->rows != A->rows || out->cols != B->cols) throw "Matrix *size* error";
            int64_t start = 0, cnt = 0;
            cn_detail::check(cn_shard_cols(B->cols, MYRANK, MPI_SIZE, &start, &cnt));
            cn_detail::check(cn_dotmpi_f32(ctx_.get(), A->rows, A->cols, B->cols, A->data, B->data + start * B->rows, out->data, nullptr,
                                          GEMM_MODE, exchange_8bit, nullptr));
            return;
        }
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
    std::shared_ptr<class BatchAllocator> batches_;
    uint64_t seed_ = 0, offset_ = 0, same_seed_ = 12345, same_offset_ = 0;

    // The file carries the 128-byte NCCL id followed by a launch tag ($CN_NCCL_ID_NONCE, else $MASTER_PORT, else the
    // launcher's process id, which the ranks of one launch share).  A file left behind by an earlier launch carries
    // another tag and is ignored; rank 0 removes the file once every rank has joined (ncclCommInitRank returns only then).
    static void launch_tag(char tag[32])
    {
        memset(tag, 0, 32);
        const char *t = getenv("CN_NCCL_ID_NONCE");
        if (!t) t = getenv("MASTER_PORT");
        if (t) snprintf(tag, 32, "%s", t);
        else snprintf(tag, 32, "ppid%ld", (long)getppid());
    }

    void init_comm_from_file()
    {
        const char *path = getenv("CN_NCCL_ID_FILE");
        if (!path) throw "ClusterNet: WORLD_SIZE > 1 needs CN_NCCL_ID_FILE (a file path shared by the ranks)";
        unsigned char id[128];
        char tag[32];
        launch_tag(tag);
        if (MYRANK == 0) {
            cn_detail::check(cn_comm_get_unique_id(id));
            const std::string tmp = std::string(path) + ".tmp";
            FILE *f = fopen(tmp.c_str(), "wb");
            if (!f || fwrite(id, 1, 128, f) != 128 || fwrite(tag, 1, 32, f) != 32 || fclose(f) != 0) throw "ClusterNet: cannot write CN_NCCL_ID_FILE";
            if (rename(tmp.c_str(), path) != 0) throw "ClusterNet: cannot publish CN_NCCL_ID_FILE";
        } else {
            bool got = false;
            for (int tries = 0; tries < 1200 && !got; ++tries) {   // up to two minutes
                FILE *f = fopen(path, "rb");
                if (f) {
                    char seen[32];
                    got = fread(id, 1, 128, f) == 128 && fread(seen, 1, 32, f) == 32 && memcmp(seen, tag, 32) == 0;
                    fclose(f);
                }
                if (!got) usleep(100000);
            }
            if (!got) throw "ClusterNet: rank 0 never published CN_NCCL_ID_FILE for this launch";
        }
        cn_detail::check(cn_comm_init_rank(ctx_.get(), id, MYRANK, MPI_SIZE));
        if (MYRANK == 0) remove(path);
    }

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
    BatchAllocationMethod_t BATCH_METHOD = Single_GPU;
    // Set before init: with Batch_split / Distributed_weights every process passes the whole data set (as in
    // tests/batchAllocator_test.cu:22-114, where each process makes its own X, y) and uploads only its 1/G of the rows of
    // each batch over its own PCIe link; the blocks are exchanged over NVLink (CN_BATCH_SHARDED_UPLOAD).  Default: only
    // rank 0's data set is used and every batch is broadcast from it.
    bool EVERY_RANK_HOLDS_DATA = false;

    // data set read from two HDF5 files (source/batchAllocator.cpp:62-99; the csv branch of the reference is not built).
    // As in the reference only rank 0 reads the files unless every process serves itself (Single_GPU).
    void init(std::string path_X, std::string path_y, float cross_validation_size, int64_t batch_size, int64_t cv_batch_size,
              ClusterNet *cluster, BatchAllocationMethod_t method = Single_GPU)
    {
        if (path_X.find("hdf5") == std::string::npos) throw "Only the cvs and hdf5 formats are supported!";
        const bool reads = method == Single_GPU || cluster->MPI_SIZE == 1 || cluster->MYRANK == 0;
        Matrix *X = reads ? read_hdf5(path_X.c_str()) : empty_cpu(1, 1);
        Matrix *y = reads ? read_hdf5(path_y.c_str()) : empty_cpu(1, 1);
        init(X, y, cross_validation_size, batch_size, cv_batch_size, cluster, method);
    }

    // without a ClusterNet (source/batchAllocator.cpp:21-30): one GPU, the context of the free functions
    void init(Matrix *X, Matrix *y, float cross_validation_size, int64_t batch_size, int64_t cv_batch_size)
    {
        init_impl(X, y, cross_validation_size, batch_size, cv_batch_size, cn_detail::current(), 0, 1, Single_GPU);
    }

    // X, y: HOST row-major matrices holding the whole data set (source/batchAllocator.cpp:31-60,101-139).  With
    // Single_GPU every process serves its own X, y.  With Batch_split / Distributed_weights and several processes only
    // rank 0's X, y are used (the others may pass anything): the data set's dimensions and then every batch travel from
    // rank 0 to the other GPUs (MPI_get_dataset_dimensions and the MPI sends of broadcast_batch_to_processes there,
    // one NCCL broadcast over NVLink per batch here).
    void init(Matrix *X, Matrix *y, float cross_validation_size, int64_t batch_size, int64_t cv_batch_size, ClusterNet *cluster,
              BatchAllocationMethod_t method = Single_GPU)
    {
        init_impl(X, y, cross_validation_size, batch_size, cv_batch_size, cluster->context(), cluster->MYRANK, cluster->MPI_SIZE, method);
    }

    // The host-side staging memcpy and the asynchronous copies are one step here, and the broadcast to the other
    // processes happens when the batch becomes current; these calls are kept so that the reference's loop
    // (tests/batchAllocator_test.cu:44-76) compiles unchanged.
    void broadcast_batch_to_processes() {}
    void broadcast_batch_cv_to_processes() {}
    void allocate_next_batch_async() { if (root_) cn_detail::check(cn_batch_copy_next_async(train_.get())); }
    void allocate_next_cv_batch_async() { if (root_) cn_detail::check(cn_batch_copy_next_async(cv_.get())); }
    void replace_current_batch_with_next() { swap(train_.get(), CURRENT_BATCH, CURRENT_BATCH_Y, recv_x_, recv_y_, SKIP_LAST_BATCH); }
    void replace_current_cv_batch_with_next() { swap(cv_.get(), CURRENT_BATCH_CV, CURRENT_BATCH_CV_Y, recv_cv_x_, recv_cv_y_, false); }

private:
    std::shared_ptr<cn_batch> train_, cv_;
    cn_context *ctx_ = nullptr;
    int64_t cols_x_ = 0, cols_y_ = 0;
    bool root_ = true, bcast_ = false;
    Matrix *recv_x_ = nullptr, *recv_y_ = nullptr, *recv_cv_x_ = nullptr, *recv_cv_y_ = nullptr;   // receive buffers of the other ranks
    float *d_hdr_ = nullptr;

    void init_impl(Matrix *X, Matrix *y, float cross_validation_size, int64_t batch_size, int64_t cv_batch_size, cn_context *ctx, int rank,
                   int nranks, BatchAllocationMethod_t method)
    {
        ctx_ = ctx;
        BATCH_METHOD = method;
        const bool sharded = EVERY_RANK_HOLDS_DATA && method != Single_GPU && nranks > 1;
        bcast_ = method != Single_GPU && nranks > 1 && !sharded;
        root_ = !bcast_ || rank == 0;
        // two uploads in flight: with many ranks one upload's exchanges can outlast a short step
        const int flags = sharded ? (CN_BATCH_SHARDED_UPLOAD | CN_BATCH_LOOKAHEAD) : 0;
        BATCH_SIZE = batch_size;
        BATCH_SIZE_CV = cv_batch_size;
        cn_detail::cuda(cudaMalloc((void **)&d_hdr_, 8 * sizeof(float)));
        // data set dimensions from rank 0; rows as two 16-bit halves so that they stay exact as floats
        float meta[4] = {(float)(X->rows >> 16), (float)(X->rows & 0xffff), (float)X->cols, (float)y->cols};
        if (bcast_) {
            cn_detail::cuda(cudaMemcpy(d_hdr_, meta, sizeof(meta), cudaMemcpyHostToDevice));
            cn_detail::check(cn_bcast_f32(ctx_, d_hdr_, 4, 0, nullptr));
            cn_detail::cuda(cudaMemcpy(meta, d_hdr_, sizeof(meta), cudaMemcpyDeviceToHost));
        }
        const int64_t rows = ((int64_t)meta[0] << 16) + (int64_t)meta[1];
        cols_x_ = (int64_t)meta[2];
        cols_y_ = (int64_t)meta[3];
        TRAIN_SET_ROWS = (int64_t)ceilf(rows * (1.0f - cross_validation_size));
        CV_SET_ROWS = rows - TRAIN_SET_ROWS;
        if (BATCH_SIZE_CV > rows * cross_validation_size) throw "Cross validation batch size must be smaller than the cross validation set.";
        if (BATCH_SIZE > TRAIN_SET_ROWS) throw "ERROR: Batch size must be smaller than the training set.";
        TOTAL_BATCHES = (TRAIN_SET_ROWS + batch_size - 1) / batch_size;
        TOTAL_BATCHES_CV = (CV_SET_ROWS > 0 && cv_batch_size > 0) ? (CV_SET_ROWS + cv_batch_size - 1) / cv_batch_size : 0;
        CURRENT_BATCH = cn_detail::header(0, 0);
        CURRENT_BATCH_Y = cn_detail::header(0, 0);
        CURRENT_BATCH_CV = cn_detail::header(0, 0);
        CURRENT_BATCH_CV_Y = cn_detail::header(0, 0);
        cn_batch *t = nullptr, *c = nullptr;
        if (root_) {
            cn_detail::check(cn_batch_create_ex(ctx_, X->data, y->data, TRAIN_SET_ROWS, cols_x_, cols_y_, batch_size, 0, flags, &t));
            train_ = std::shared_ptr<cn_batch>(t, [](cn_batch *p) { cn_batch_destroy(p); });
            if (TOTAL_BATCHES_CV > 0) {
                cn_detail::check(cn_batch_create_ex(ctx_, X->data + (size_t)TRAIN_SET_ROWS * cols_x_, y->data + (size_t)TRAIN_SET_ROWS * cols_y_,
                                                   CV_SET_ROWS, cols_x_, cols_y_, cv_batch_size, 0, flags, &c));
                cv_ = std::shared_ptr<cn_batch>(c, [](cn_batch *p) { cn_batch_destroy(p); });
            }
        } else {
            recv_x_ = empty(batch_size, cols_x_);
            recv_y_ = empty(batch_size, cols_y_);
            if (TOTAL_BATCHES_CV > 0) {
                recv_cv_x_ = empty(cv_batch_size, cols_x_);
                recv_cv_y_ = empty(cv_batch_size, cols_y_);
            }
        }
        float *dx = nullptr, *dy = nullptr;
        int64_t n = 0;
        if (root_) cn_detail::check(cn_batch_current(t, &dx, &dy, &n));
        share(CURRENT_BATCH, CURRENT_BATCH_Y, recv_x_, recv_y_, dx, dy, n);
        if (TOTAL_BATCHES_CV > 0) {
            if (root_) cn_detail::check(cn_batch_current(c, &dx, &dy, &n));
            share(CURRENT_BATCH_CV, CURRENT_BATCH_CV_Y, recv_cv_x_, recv_cv_y_, dx, dy, n);
        }
    }
    void publish(Matrix *X, Matrix *Y, float *dx, float *dy, int64_t n)
    {
        X->rows = n; X->cols = cols_x_; X->size = n * cols_x_; X->bytes = (size_t)X->size * 4; X->data = dx;
        Y->rows = n; Y->cols = cols_y_; Y->size = n * cols_y_; Y->bytes = (size_t)Y->size * 4; Y->data = dy;
    }
    // makes (dx, dy, n) of rank 0 the current batch everywhere: row count first, then the two blocks
    void share(Matrix *X, Matrix *Y, Matrix *rx, Matrix *ry, float *dx, float *dy, int64_t n)
    {
        if (bcast_) {
            float nf = (float)n;
            if (root_) cn_detail::cuda(cudaMemcpy(d_hdr_, &nf, sizeof(float), cudaMemcpyHostToDevice));
            cn_detail::check(cn_bcast_f32(ctx_, d_hdr_, 1, 0, nullptr));
            if (!root_) {
                cn_detail::cuda(cudaMemcpy(&nf, d_hdr_, sizeof(float), cudaMemcpyDeviceToHost));
                n = (int64_t)nf;
                dx = rx->data;
                dy = ry->data;
            }
        }
        publish(X, Y, dx, dy, n);
        if (bcast_) {
            cn_detail::check(cn_bcast_f32(ctx_, dx, n * cols_x_, 0, nullptr));
            cn_detail::check(cn_bcast_f32(ctx_, dy, n * cols_y_, 0, nullptr));
        }
    }
    void swap(cn_batch *b, Matrix *X, Matrix *Y, Matrix *rx, Matrix *ry, bool skip_last)
    {
        float *dx = nullptr, *dy = nullptr;
        int64_t n = 0;
        if (root_) {
            cn_detail::check(cn_batch_set_skip_last(b, skip_last ? 1 : 0));
            cn_detail::check(cn_batch_swap(b, nullptr, &dx, &dy, &n));
        }
        share(X, Y, rx, ry, dx, dy, n);
    }
};

inline void ClusterNet::init_batch_allocator(Matrix *X, Matrix *y, int64_t batch_size)
{
    batches_ = std::make_shared<BatchAllocator>();
    batches_->init(X, y, 0.0f, batch_size, 0, this, Single_GPU);
    m_total_batches = batches_->TOTAL_BATCHES;
    m_current_batch_X = batches_->CURRENT_BATCH;
    m_current_batch_y = batches_->CURRENT_BATCH_Y;
}
inline void ClusterNet::allocate_next_batch_async() { batches_->allocate_next_batch_async(); }
inline void ClusterNet::replace_current_batch_with_next() { batches_->replace_current_batch_with_next(); }

// ------------------------------------------------------------------------------------------------------------
// Free functions of source/basicOps.cuh that sit on the dot / codec / training-step path, same names and argument
// order; device matrices are column-major, everything runs on the NULL stream as in the reference.
// ------------------------------------------------------------------------------------------------------------
inline Matrix *fill_matrix(int64_t rows, int64_t cols, float v)
{
    Matrix *m = empty(rows, cols);
    cn_detail::check(cn_fill_f32(cn_detail::current(), m->data, m->size, v, nullptr));
    return m;
}
inline void fill_matrix(Matrix *A, const float v) { cn_detail::check(cn_fill_f32(cn_detail::current(), A->data, A->size, v, nullptr)); }
inline Matrix *zeros(int64_t rows, int64_t cols) { return fill_matrix(rows, cols, 0.0f); }
// to_host(arange(rows, cols)) reads start, start + 1, ... in row-major order (source/basicOps.cu:205-212)
inline Matrix *arange(int64_t start, int64_t rows, int64_t cols)
{
    Matrix *m = empty(rows, cols);
    cn_detail::check(cn_arange_f32(cn_detail::current(), m->data, start, rows, cols, nullptr));
    return m;
}
inline Matrix *arange(int64_t rows, int64_t cols) { return arange(0, rows, cols); }
inline Matrix *ones(int64_t rows, int64_t cols) { return fill_matrix(rows, cols, 1.0f); }

// layout boundary (source/basicOps.cu:14-137)
inline void to_col_major(Matrix *A, Matrix *out) { cn_detail::check(cn_to_col_major(cn_detail::current(), A->data, out->data, A->rows, A->cols, nullptr)); }
inline Matrix *to_col_major(Matrix *A) { Matrix *out = empty(A->rows, A->cols); to_col_major(A, out); return out; }
inline Matrix *to_row_major(Matrix *A)
{
    Matrix *out = empty(A->rows, A->cols);
    cn_detail::check(cn_to_row_major(cn_detail::current(), A->data, out->data, A->rows, A->cols, nullptr));
    return out;
}
// transpose of a column-major matrix: its row-major image read as a column-major cols x rows matrix
inline Matrix *T(Matrix *A)
{
    Matrix *out = to_row_major(A);
    out->rows = A->cols;
    out->cols = A->rows;
    return out;
}
inline Matrix *to_gpu(Matrix *A, int is_col_major)
{
    Matrix *raw = empty(A->rows, A->cols);
    cn_detail::cuda(cudaMemcpy(raw->data, A->data, A->bytes, cudaMemcpyDefault));
    if (is_col_major) return raw;
    Matrix *out = to_col_major(raw);
    cn_detail::cuda(cudaStreamSynchronize(nullptr));
    cudaFree(raw->data);
    free(raw);
    return out;
}
inline Matrix *to_gpu(Matrix *A) { return to_gpu(A, 0); }
inline Matrix *to_host(Matrix *A, int is_row_major)
{
    Matrix *src = is_row_major ? A : to_row_major(A);
    Matrix *out = empty_cpu(A->rows, A->cols);
    cn_detail::cuda(cudaMemcpy(out->data, src->data, A->bytes, cudaMemcpyDefault));
    if (!is_row_major) {
        cudaFree(src->data);
        free(src);
    }
    return out;
}
inline Matrix *to_host(Matrix *A) { return to_host(A, 0); }

// slices and stacks of column-major matrices are plain copies (source/basicOps.cu:153-160,499-523,562-572)
inline Matrix *slice_cols(Matrix *A, int64_t start, int64_t end)   // columns start..end, both included
{
    if (start < 0 || end < start || end >= A->cols) throw "slice_cols: range outside the matrix";
    Matrix *out = empty(A->rows, end - start + 1);
    cn_detail::cuda(cudaMemcpyAsync(out->data, A->data + start * A->rows, out->bytes, cudaMemcpyDeviceToDevice, nullptr));
    return out;
}
inline Matrix *slice_rows(Matrix *A, int64_t start, int64_t end)   // rows start..end, both included
{
    if (start < 0 || end < start || end >= A->rows) throw "slice_rows: range outside the matrix";
    Matrix *out = empty(end - start + 1, A->cols);
    cn_detail::cuda(cudaMemcpy2DAsync(out->data, (size_t)out->rows * 4, A->data + start, (size_t)A->rows * 4, (size_t)out->rows * 4,
                                      (size_t)A->cols, cudaMemcpyDeviceToDevice, nullptr));
    return out;
}
inline void hStack(Matrix *A, Matrix *B, Matrix *out)
{
    if (A->rows != B->rows || out->rows != A->rows || out->cols != A->cols + B->cols) throw "Wrong merge sizes!";
    cn_detail::cuda(cudaMemcpyAsync(out->data, A->data, A->bytes, cudaMemcpyDeviceToDevice, nullptr));
    cn_detail::cuda(cudaMemcpyAsync(out->data + A->size, B->data, B->bytes, cudaMemcpyDeviceToDevice, nullptr));
}
inline Matrix *hStack(Matrix *A, Matrix *B) { Matrix *out = empty(A->rows, A->cols + B->cols); hStack(A, B, out); return out; }
// the first matrices_count - 1 blocks hold general_size elements each, the last one the rest (the remainder shard)
inline void hStackN(Matrix **arrA, int64_t general_size, Matrix *out, int matrices_count)
{
    int64_t done = 0;
    for (int i = 0; i < matrices_count; ++i) {
        const int64_t n = i + 1 < matrices_count ? general_size : out->size - done;
        if (n < 0 || n > arrA[i]->size) throw "hStackN: block larger than its source";
        cn_detail::cuda(cudaMemcpyAsync(out->data + done, arrA[i]->data, (size_t)n * 4, cudaMemcpyDeviceToDevice, nullptr));
        done += n;
    }
}

// elementwise (source/basicOps.cu:574-760)
#define CN_FACADE_BINARY(name, fn)                                                                                         \
    inline void name(Matrix *A, Matrix *B, Matrix *out)                                                                   \
    {                                                                                                                     \
        if (A->rows != B->rows || A->cols != B->cols || out->rows != A->rows || out->cols != A->cols) throw "Matrix *size* error"; \
        cn_detail::check(fn(cn_detail::current(), A->data, B->data, out->data, A->size, nullptr));                       \
    }                                                                                                                     \
    inline Matrix *name(Matrix *A, Matrix *B) { Matrix *out = empty(A->rows, A->cols); name(A, B, out); return out; }
CN_FACADE_BINARY(add, cn_add)
CN_FACADE_BINARY(sub, cn_sub)
CN_FACADE_BINARY(mul, cn_mul)
CN_FACADE_BINARY(div, cn_div)
#undef CN_FACADE_BINARY
#define CN_FACADE_UNARY(name, call)                                                                  \
    inline void name(Matrix *A, Matrix *out) { cn_detail::check(call); }                             \
    inline Matrix *name(Matrix *A) { Matrix *out = empty(A->rows, A->cols); name(A, out); return out; }
CN_FACADE_UNARY(abs, cn_abs(cn_detail::current(), A->data, out->data, A->size, nullptr))
CN_FACADE_UNARY(square, cn_square(cn_detail::current(), A->data, out->data, A->size, nullptr))
CN_FACADE_UNARY(logistic, cn_bias_activation(cn_detail::current(), A->data, nullptr, CN_ACT_LOGISTIC, out->data, A->rows, A->cols, nullptr))
CN_FACADE_UNARY(rectified_linear, cn_bias_activation(cn_detail::current(), A->data, nullptr, CN_ACT_RELU, out->data, A->rows, A->cols, nullptr))
CN_FACADE_UNARY(doubleRectifiedLinear, cn_bias_activation(cn_detail::current(), A->data, nullptr, CN_ACT_DOUBLE_RELU, out->data, A->rows, A->cols, nullptr))
CN_FACADE_UNARY(LinearUnit, cn_bias_activation(cn_detail::current(), A->data, nullptr, CN_ACT_LINEAR, out->data, A->rows, A->cols, nullptr))
CN_FACADE_UNARY(logisticGrad, cn_activation_gradient(cn_detail::current(), A->data, CN_ACT_LOGISTIC, out->data, A->size, nullptr))
CN_FACADE_UNARY(rectified_linear_derivative, cn_activation_gradient(cn_detail::current(), A->data, CN_ACT_RELU, out->data, A->size, nullptr))
CN_FACADE_UNARY(double_rectified_linear_derivative, cn_activation_gradient(cn_detail::current(), A->data, CN_ACT_DOUBLE_RELU, out->data, A->size, nullptr))
CN_FACADE_UNARY(softmax, cn_softmax(cn_detail::current(), A->data, out->data, A->rows, A->cols, nullptr))
#undef CN_FACADE_UNARY
inline void scalarMul(Matrix *A, float a, Matrix *out) { cn_detail::check(cn_scalar_mul(cn_detail::current(), A->data, a, out->data, A->size, nullptr)); }
inline Matrix *scalarMul(Matrix *A, float a) { Matrix *out = empty(A->rows, A->cols); scalarMul(A, a, out); return out; }
inline void scalarAdd(Matrix *A, float a, Matrix *out) { cn_detail::check(cn_scalar_add(cn_detail::current(), A->data, a, out->data, A->size, nullptr)); }
inline Matrix *scalarAdd(Matrix *A, float a) { Matrix *out = empty(A->rows, A->cols); scalarAdd(A, a, out); return out; }
// max() seeds its reduction with -1.0f and blocks until the value is on the host, as thrust::reduce does
inline float max(Matrix *A)
{
    float *d = nullptr, h = 0.f;
    cn_detail::cuda(cudaMalloc((void **)&d, 4));
    cn_detail::check(cn_max_f32(cn_detail::current(), A->data, A->size, d, nullptr));
    cn_detail::cuda(cudaMemcpy(&h, d, 4, cudaMemcpyDeviceToHost));
    cudaFree(d);
    return h;
}
// bias row vector v (1 x cols) added to every row of A (source/basicOps.cu:966-974)
inline void addMatrixVector(Matrix *A, Matrix *v, Matrix *out)
{
    if (A->cols != v->cols) throw "Error dimensions do not match";
    cn_detail::check(cn_bias_activation(cn_detail::current(), A->data, v->data, CN_ACT_LINEAR, out->data, A->rows, A->cols, nullptr));
}
inline Matrix *addMatrixVector(Matrix *A, Matrix *v) { Matrix *out = empty(A->rows, A->cols); addMatrixVector(A, v, out); return out; }
// maximum over groups of maxout_level consecutive columns, plus the winning column index as a float (:1272-1299)
inline void maxout(Matrix *A, Matrix *out, Matrix *outargmax, int maxout_level)
{
    if (maxout_level <= 0 || A->cols % maxout_level != 0) throw "maxout: columns must be a multiple of the maxout level";
    cn_detail::check(cn_maxout(cn_detail::current(), A->data, out->data, outargmax->data, A->rows, A->cols, maxout_level, nullptr));
}
inline Matrix **maxout(Matrix *A, int maxout_level)
{
    if (maxout_level <= 0 || A->cols % maxout_level != 0) throw "maxout: columns must be a multiple of the maxout level";
    Matrix **pair = (Matrix **)malloc(sizeof(Matrix *) * 2);
    pair[0] = empty(A->rows, A->cols / maxout_level);
    pair[1] = empty(A->rows, A->cols / maxout_level);
    maxout(A, pair[0], pair[1], maxout_level);
    return pair;
}
inline void create_t_matrix(Matrix *labels, Matrix *out) { cn_detail::check(cn_create_t_matrix(cn_detail::current(), labels->data, out->data, out->rows, out->cols, nullptr)); }
inline Matrix *create_t_matrix(Matrix *labels, int max_label) { Matrix *out = empty(labels->rows, max_label); create_t_matrix(labels, out); return out; }
// optimiser steps with the reference's full argument lists (:1185-1197); RMS_multiplier etc. unused by a kernel stay unused
inline void RMSprop_with_weight_update(Matrix *RMS, Matrix *grad, Matrix *w, Matrix * /*m*/, float RMS_multiplier, float learning_rate,
                                       int /*batch_size*/, float /*momentum*/)
{
    cn_detail::check(cn_rmsprop_update(cn_detail::current(), RMS->data, grad->data, w->data, RMS_multiplier, learning_rate, RMS->size, nullptr));
}
inline void Nesterov_weight_update(Matrix *RMS, Matrix *grad, Matrix *w, Matrix *m, float /*RMS_multiplier*/, float learning_rate, int batch_size,
                                   float momentum)
{
    cn_detail::check(cn_nesterov_update(cn_detail::current(), grad->data, w->data, m->data, learning_rate, batch_size, momentum, RMS->size, nullptr));
}
// codec with an explicit table argument, as ::compression_8bit / ::decompression_8bit take it (:1163-1176); the table the
// context was created with is the one used, tbl_flt is accepted for source compatibility
inline void compression_8bit(Matrix * /*tbl_flt*/, Matrix *A, float precision, Matrix *out)
{
    cn_detail::check(cn_compress_8bit(cn_detail::current(), A->data, precision, A->size, out->char_data, nullptr));
}
inline void decompression_8bit(Matrix * /*tbl_flt*/, Matrix *A, float precision, Matrix *out)
{
    cn_detail::check(cn_decompress_8bit(cn_detail::current(), A->char_data, precision, A->size, out->data, nullptr));
}


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
