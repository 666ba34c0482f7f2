/*
 * clusternet_b200 — C ABI of the B200-native dot / dotMPI / 8-bit codec / batch path.
 *
 * Every entry point is `extern "C"`, takes plain pointers and 64-bit sizes, and returns a cn_status.
 * Device pointers are ordinary CUDA device addresses; `stream` is a cudaStream_t passed as void*
 * (NULL = the legacy default stream, which is what the reference uses everywhere).
 * All matrices on the device are dense fp32, COLUMN-major with leading dimension = rows, exactly as
 * the reference keeps them (source/basicOps.cu:14-33: to_gpu transposes on upload).
 *
 * Each declaration cites the reference interface (file:line, relative to the reference tree) whose
 * job it takes over.
 *
 * Threading and streams.  One context per host thread.  Calls on one context must be serialised on ONE stream: the
 * scratch buffers the kernels use (activation planes and split-K partials of the products, exchange codes, partial
 * maxima) belong to the context, and the first call that needs a larger buffer grows it with a device synchronisation -
 * make that call before a stream capture.  The codec / gradient-exchange entry points and the product entry points use
 * disjoint scratch, so one stream for each is allowed.
 */
#ifndef CLUSTERNET_B200_H
#define CLUSTERNET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cn_context cn_context;

typedef enum cn_status {
    CN_OK = 0,
    CN_ERR_ARG = 1,         /* null pointer, negative size, misaligned buffer */
    CN_ERR_SHAPE = 2,       /* operand shapes do not match (the reference throws "Matrix *size* error") */
    CN_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed; cn_last_error() has the text */
    CN_ERR_NCCL = 4,
    CN_ERR_TIMEOUT = 5,     /* a bounded device-side or host-side wait ran out */
    CN_ERR_UNSUPPORTED = 6, /* valid request that this build has no kernel for */
    CN_ERR_NOMEM = 7
} cn_status;

/* Text of the last error raised on the calling thread ("" when none). */
const char *cn_last_error(void);
const char *cn_status_string(int status);
/* Library version, and the compute capability it was compiled for (100 for sm_100a). */
int cn_version(void);
/* Number of CUDA kernels this library has launched in the calling process so far (all contexts). */
uint64_t cn_kernel_launches(void);
int cn_compiled_arch(void);

/* ---------------------------------------------------------------------------------------------
 * Context.  Replaces ClusterNet::init (source/clusterNet.cpp:40-146): binds a device, uploads the
 * 126-entry codebook (source/clusterNet.cpp:73, file source/8bit_floats.hdf5), derives the codec's
 * decision thresholds from it and allocates the small scratch buffers the kernels need.
 * codebook126 is a HOST pointer to 126 strictly increasing floats in (0,1).
 * ------------------------------------------------------------------------------------------- */
int cn_context_create(int device, const float *codebook126, cn_context **out);
int cn_context_destroy(cn_context *ctx);
int cn_context_device(const cn_context *ctx);

/* Host-only helper (no GPU needed): reads the codebook from the reference's HDF5 file or from a raw
 * 504-byte dump (replaces read_hdf5 of "/Default", source/util.cu:100-131). */
int cn_codebook_load(const char *path, float *codebook126);

/* Host-only (no GPU needed): reads a dense dataset of an HDF5 file into a malloc'd row-major float array; replaces
 * read_hdf5 (source/util.cu:100-131, libhdf5) for the files numpy / h5py write: version-0 superblock, contiguous or
 * compact layout, rank 1 or 2, little-endian 4- or 8-byte float or integer data (converted to float, as
 * H5T_NATIVE_FLOAT does).  Release the array with cn_host_free. */
int cn_hdf5_read_f32(const char *path, const char *dataset, float **data_out, int64_t *rows, int64_t *cols);
/* Shape of a dataset, and conversion straight into a caller's buffer of `capacity` floats (e.g. pinned memory, as the
 * reference's read_hdf5 allocates it with cudaHostAlloc, source/util.cu:112-116). */
int cn_hdf5_dims(const char *path, const char *dataset, int64_t *rows, int64_t *cols);
int cn_hdf5_read_f32_into(const char *path, const char *dataset, float *dst, int64_t capacity);
/* The same with 32-bit integer output, for the index datasets of the CSR files (/indices, /indptr, /shape of
 * read_sparse_hdf5, source/util.cu:133-198). */
int cn_hdf5_read_i32(const char *path, const char *dataset, int32_t **data_out, int64_t *rows, int64_t *cols);
void cn_host_free(void *p);
/* Host-only: writes one rank-2 float32 dataset (row-major `data`) into a new version-0 HDF5 file; replaces write_hdf5
 * (source/util.cu:202-216).  cn_hdf5_read_f32 reads it back bit for bit. */
int cn_hdf5_write_f32(const char *path, const char *dataset, const float *data, int64_t rows, int64_t cols);

/* Host-only helper (no GPU needed): derives, from the codebook, the 127 ascending magnitude
 * thresholds (fp32 bit patterns) at which kCompression_8bit's answer changes, and the 128 codes of
 * the levels they separate (254, 0..125, 127).  code(|a|) = level_codes[#{j : thr[j] <= bits(|a|)}].
 * This is an exact re-expression of the search-and-pick of source/clusterKernels.cu:1193-1229. */
int cn_codec_build_thresholds(const float *codebook126, uint32_t *thr127, uint8_t *level_codes128);

/* ---------------------------------------------------------------------------------------------
 * 8-bit dynamic-float codec.
 * ------------------------------------------------------------------------------------------- */

/* absmax: replaces abs() + max() (source/basicOps.cu:810-822,1076-1081; kAbs
 * source/clusterKernels.cu:429-436).  Writes max_i |A[i]| (or -1.0f when n == 0, the reference's
 * reduce seed) to the DEVICE scalar d_out.  One pass, no temporary matrix. */
int cn_absmax_f32(cn_context *ctx, const float *d_A, int64_t n, float *d_out, void *stream);

/* absmax without any allocation and without a context, for callers that cannot call cudaMalloc where they need the
 * scale: callbacks that must not take the allocator's lock (cudaMalloc may block and synchronise the device),
 * processes whose device memory is already owned by another allocator, recovery paths that run when device memory is
 * exhausted.  Same kernel and same result as
 * cn_absmax_f32; the per-CTA partial maxima live in a fixed 4352-byte array inside the library image instead of in
 * context scratch.  Limits: n <= 2^32 elements (larger inputs return CN_ERR_ARG); all calls on a device share the
 * array, so calls that overlap on the GPU race — keep them on one stream; the first call on a device looks the
 * array's device address up and should be made before any stream capture starts.  Uses the current device.
 * This entry point has no counterpart in the reference. */
int cn_absmax_f32_noalloc(const float *d_A, int64_t n, float *d_out, void *stream);

/* compression_8bit: replaces ::compression_8bit (source/basicOps.cu:1163-1168) and kCompression_8bit
 * (source/clusterKernels.cu:1163-1232).  codes[i] is bit-identical to the reference kernel's output
 * for every input for which the reference's answer is defined. */
int cn_compress_8bit(cn_context *ctx, const float *d_A, float precision, int64_t n, uint8_t *d_codes, void *stream);
/* Same, with `precision` read from a device scalar (e.g. the output of cn_absmax_f32) so that the
 * absmax -> compress chain needs no host synchronisation. */
int cn_compress_8bit_dp(cn_context *ctx, const float *d_A, const float *d_precision, int64_t n, uint8_t *d_codes, void *stream);

/* scale = max |A|, then compression_8bit(A, scale) - the pair of calls the reference makes when the scale is not known
 * beforehand (source/test.cu:1964-1968,2108-2109: max(abs(A)) followed by compression_8bit).  Up to 4 Mi elements it is ONE
 * cooperative kernel launch: pass 1 reduces, a bounded grid-wide barrier publishes the maximum, pass 2 codes the tensor
 * out of L2; larger tensors, for which launch latency no longer matters, take two pipelined launches.
 * d_scale_out (device) receives the scale; the codes equal
 * cn_absmax_f32 + cn_compress_8bit_dp bit for bit.  Uses context scratch: calls on one context must be serialised on
 * one stream.  A barrier wait that runs out (it cannot unless the GPU is shared with a kernel that blocks half of it)
 * is reported by cn_gemm_check_status as CN_ERR_TIMEOUT. */
int cn_absmax_compress_8bit(cn_context *ctx, const float *d_A, int64_t n, float *d_scale_out, uint8_t *d_codes, void *stream);

/* decompression_8bit: replaces ::decompression_8bit (source/basicOps.cu:1172-1176) and
 * kDecompression_8bit (source/clusterKernels.cu:1135-1160), including its committed decoding of the
 * special codes (126, 127, 254 -> +precision; 255 -> -precision). */
int cn_decompress_8bit(cn_context *ctx, const uint8_t *d_codes, float precision, int64_t n, float *d_out, void *stream);
int cn_decompress_8bit_dp(cn_context *ctx, const uint8_t *d_codes, const float *d_precision, int64_t n, float *d_out, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Layout boundary: host row-major <-> device column-major.
 * Replaces to_gpu / to_host / to_col_major / to_row_major / kTranspose
 * (source/basicOps.cu:14-33,35-88,108-127; source/clusterKernels.cu:457-482).
 * ------------------------------------------------------------------------------------------- */
/* d_dst (col-major rows x cols) <- d_src (row-major rows x cols); both on the device. */
int cn_to_col_major(cn_context *ctx, const float *d_src, float *d_dst, int64_t rows, int64_t cols, void *stream);
/* d_dst (row-major rows x cols) <- d_src (col-major rows x cols). */
int cn_to_row_major(cn_context *ctx, const float *d_src, float *d_dst, int64_t rows, int64_t cols, void *stream);
/* Upload: h_src is a HOST row-major rows x cols buffer (pinned for an asynchronous copy), d_stage a
 * device staging buffer of the same size, d_dst the col-major result. */
int cn_upload_row_major(cn_context *ctx, const float *h_src, float *d_stage, float *d_dst, int64_t rows, int64_t cols, void *stream);
/* Download: the inverse; h_dst receives row-major data once the stream has drained. */
int cn_download_row_major(cn_context *ctx, const float *d_src, float *d_stage, float *h_dst, int64_t rows, int64_t cols, void *stream);
int cn_fill_f32(cn_context *ctx, float *d_A, int64_t n, float value, void *stream);
/* arange (source/basicOps.cu:205-212, kArange source/clusterKernels.cu:925-937): col-major rows x cols matrix whose
 * row-major reading is start, start+1, ... */
int cn_arange_f32(cn_context *ctx, float *d_A, int64_t start, int64_t rows, int64_t cols, void *stream);

/* ---------------------------------------------------------------------------------------------
 * GEMM.  Replaces the cublasSgemm call of ClusterNet::dot (source/clusterNet.cpp:404-487) and the
 * elementwise passes that follow it in the reference's layers (addMatrixVector, rectified_linear,
 * logistic, doubleRectifiedLinear, LinearUnit, maxout: source/basicOps.cu:966-974,1212-1216,672-676,
 * 728-732,742-746,1287-1299), which are fused into the tile store.
 *
 * C(M x N) = act(op(A)(M x K) . op(B)(K x N) + bias), all column-major.  lda/ldb/ldc are leading
 * dimensions of the stored (untransposed) arrays, as in the reference's call
 * (lda = A->rows, ldb = B->rows, ldc = out->rows).
 * ------------------------------------------------------------------------------------------- */
typedef enum cn_gemm_mode {
    CN_GEMM_3XTF32 = 0,  /* fp32-accurate: hi/lo TF32 split, three tensor-core products per tile */
    CN_GEMM_TF32 = 1,    /* single TF32 product (10-bit mantissa operands), reported separately */
    CN_GEMM_FP32_SIMT = 2 /* plain fp32 FMA kernel; also chosen automatically for shapes the tensor path cannot take */
} cn_gemm_mode;

typedef enum cn_activation {
    CN_ACT_LINEAR = 0,          /* LinearUnit: copy */
    CN_ACT_RELU = 1,            /* rectified_linear: x > 0 ? x : 0 */
    CN_ACT_LOGISTIC = 2,        /* logistic: 1/(1+expf(-x)) */
    CN_ACT_DOUBLE_RELU = 3      /* doubleRectifiedLinear: clamp to [0,1] */
} cn_activation;

typedef struct cn_epilogue {
    const float *bias;     /* device, N floats, added to every row (kAddMatrixVector: v[i / rows]); NULL = none */
    int activation;        /* cn_activation */
    int maxout_level;      /* 0/1 = off; L>1: C becomes M x N/L, each entry the max over L consecutive columns (kMaxout) */
    float *argmax_out;     /* device, M x N/L col-major, absolute column of the max as float; NULL = not wanted */
} cn_epilogue;

int cn_gemm_f32(cn_context *ctx, int transA, int transB, int64_t M, int64_t N, int64_t K,
                const float *d_A, int64_t lda, const float *d_B, int64_t ldb, float *d_C, int64_t ldc,
                const cn_epilogue *epi, int mode, void *stream);
/* Name of the kernel family the last cn_gemm_f32 call on this context dispatched to
 * ("tcgen05_3xtf32", "tcgen05_tf32", "simt_fp32"); for tests and reports. */
const char *cn_gemm_last_path(const cn_context *ctx);
/* The tensor-core kernel bounds every wait of its internal pipeline; a wait that runs out makes the kernel
 * return early and set a device status word.  This call drains `stream`, reads the word and returns
 * CN_ERR_TIMEOUT if any launch since the last check gave up (the output of that launch is then undefined),
 * CN_OK otherwise.  No counterpart in the reference (cublasSgemm reports nothing). */
int cn_gemm_check_status(cn_context *ctx, void *stream);
/* Diagnostics for failure handling: queues a one-thread kernel that waits, like the cross-GPU flag barrier of the fused
 * gather, for a signal that never comes, gives up after `limit_cycles` SM clock cycles and records the time-out; the
 * next cn_gemm_check_status then returns CN_ERR_TIMEOUT.  Shows (and lets tests assert) that a rank that never signals
 * becomes a host-visible error and not a hang.  The reference has no counterpart: its MPI waits are unbounded. */
int cn_diag_wait_probe(cn_context *ctx, int64_t limit_cycles, void *stream);
/* Timing of the tensor-core product without its activation pre-pass: while enabled, every launch of the main GEMM
 * kernel together with the split-K reduction kernel that follows it (when K is split) is bracketed by CUDA events on
 * the launching stream.  cn_gemm_profile_read waits for the recorded launches, writes up to `max` durations in
 * milliseconds, in launch order, and clears the record.
 * Takes the place of the reference's tick/tock around a dot call (source/clusterNet.cpp:798-840). */
int cn_gemm_profile_enable(cn_context *ctx, int enable);
int cn_gemm_profile_read(cn_context *ctx, float *ms_out, int max, int *count);

/* Test and sweep knobs of the tensor-core kernel, per context; 0 leaves the library's own choice.  tiles_per_cta: 1 or 2
 * weight tiles of 128 columns per CTA; k_splits: number of K ranges the product is cut into (split-K); chain_k_blocks:
 * K blocks of 32 accumulated in tensor memory before the sum is folded into fp32 registers.  The environment
 * variables CN_GEMM_NT / CN_GEMM_SPLITS / CN_GEMM_CHAIN give the initial values, read once per context.  No counterpart
 * in the reference (cuBLAS picks its kernels itself). */
int cn_gemm_set_tuning(cn_context *ctx, int tiles_per_cta, int k_splits, int chain_k_blocks);

/* The same elementwise ops as stand-alone kernels over an existing col-major matrix (the reference's
 * un-fused call sites, e.g. source/Layer.cpp:257-259). */
int cn_bias_activation(cn_context *ctx, const float *d_A, const float *d_bias, int activation,
                       float *d_out, int64_t rows, int64_t cols, void *stream);
int cn_maxout(cn_context *ctx, const float *d_A, float *d_out, float *d_argmax, int64_t rows, int64_t cols,
              int maxout_level, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Random numbers and weight creation.  Replaces ClusterNet::rand / uniformSqrtWeight /
 * distributed_uniformSqrtWeight (source/clusterNet.cpp:746-769,874-894,916-938) and
 * kCreateRdmSqrtWeight_Logistic (source/clusterKernels.cu:126-138).  The generator is a counter-based
 * Philox-4x32-10 written here, not cuRAND's XORWOW, so streams differ from the reference's; ranges
 * and statistics are the same (uniform in (0,1]; weights in +-4*sqrtf(6/(in+out_total))).
 * ------------------------------------------------------------------------------------------- */
int cn_rand_uniform(cn_context *ctx, float *d_A, int64_t n, uint64_t seed, uint64_t offset, void *stream);
int cn_rand_normal(cn_context *ctx, float *d_A, int64_t n, float mean, float std, uint64_t seed, uint64_t offset, void *stream);
/* rand_int (source/clusterNet.cpp:790-796; kRandInt source/clusterKernels.cu:159-170): integers low..high stored as floats. */
int cn_rand_int(cn_context *ctx, float *d_A, int64_t n, int low, int high, uint64_t seed, uint64_t offset, void *stream);
int cn_uniform_sqrt_weight(cn_context *ctx, float *d_A, int64_t n, int64_t fan_in, int64_t fan_out_total,
                           uint64_t seed, uint64_t offset, void *stream);
/* dropout (source/clusterNet.cpp:842-872, kDropout source/clusterKernels.cu:939-947):
 * out[i] = u[i] > rate ? A[i] : 0, u uniform in (0,1]; no rescale. */
int cn_dropout(cn_context *ctx, const float *d_A, float *d_out, int64_t n, float rate, uint64_t seed, uint64_t offset, void *stream);

/* dropout with its seed in device memory and a call that advances that seed on the stream: a training step recorded
 * once (CUDA graph) then draws fresh masks on every replay.  No counterpart in the reference (cuRAND host generator). */
int cn_dropout_dp(cn_context *ctx, const float *d_A, float *d_out, int64_t n, float rate, const uint64_t *d_seed, uint64_t offset, void *stream);
int cn_seed_advance(cn_context *ctx, uint64_t *d_seed, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Communicator (one process per GPU).  Replaces ClusterNet::init_MPI / shutdown_MPI
 * (source/clusterNet.cpp:148-183,223-228) with NCCL over NVLink.  The 128-byte id is produced on one
 * rank and handed to the others by the host program (torch.distributed store, a file, ...).
 * ------------------------------------------------------------------------------------------- */
int cn_comm_get_unique_id(void *id128);
int cn_comm_init_rank(cn_context *ctx, const void *id128, int rank, int nranks);
/* Single-process form of the bootstrap (several GPUs driven from one process): the n contexts, each on its own device,
 * become ranks 0 .. n-1 of one communicator (ncclCommInitAll).  Either every rank is then driven by its own host thread
 * (each thread makes its context's device current once: cn_context_make_current), and every entry point works as with
 * one process per GPU; or one thread drives all ranks and brackets the per-rank calls of one collective with
 * cn_group_start / cn_group_end (making each context current before its call) - that form covers the entry points that
 * end in a single collective (cn_bcast_f32, cn_allgather_*, cn_allreduce_sum_f32, cn_dotmpi_f32 / cn_tdotmpi_f32 with
 * exchange = 0, cn_dottmpi_f32), not the 8-bit exchanges, which launch kernels after their gather.  Symmetric buffers
 * (cn_sym_alloc, CN_BATCH_SHARDED_UPLOAD) need one process per GPU.  The reference's own bootstrap is one process per
 * GPU (source/clusterNet.cpp:148-183); its single-process "PCIe" mode (source/clusterNet.cpp:1137-1370) keeps arrays of
 * per-device matrices instead. */
int cn_comm_init_all(cn_context **ctxs, int n);
int cn_group_start(void);
int cn_group_end(void);
int cn_context_make_current(const cn_context *ctx);
/* Host-side wait with a limit, for loops in which a peer may have died: returns CN_OK when everything queued on
 * `stream` has finished; on an asynchronous NCCL error (CN_ERR_NCCL) or after timeout_ms with the stream still busy
 * (CN_ERR_TIMEOUT) it aborts the communicator so that the collectives in flight end; afterwards every collective call
 * on the context fails until cn_comm_destroy + cn_comm_init_rank.  Without a communicator it is a plain bounded wait.
 * The reference has no counterpart: its MPI_Barrier / MPI_Wait (source/clusterNet.cpp:663-690) block forever. */
int cn_comm_sync(cn_context *ctx, void *stream, int timeout_ms);
int cn_comm_destroy(cn_context *ctx);
int cn_comm_rank(const cn_context *ctx);
int cn_comm_size(const cn_context *ctx);
/* Shard of an N-column matrix owned by `rank`: floor(N/G) columns, the last rank also takes the
 * remainder (source/clusterNet.cpp:515-516,926-931). Host-only. */
int cn_shard_cols(int64_t n_total, int rank, int nranks, int64_t *col_start, int64_t *col_count);
/* Broadcast of the activations ("A is broadcast"): n floats from root to every rank, in place. */
int cn_bcast_f32(cn_context *ctx, float *d_buf, int64_t n, int root, void *stream);
/* In-place all-gather of column shards of a col-major M x N_total matrix: rank r has already written
 * its own columns; on return every rank holds all of C.  Replaces the MPI ring + hStackN
 * (source/clusterNet.cpp:663-694; source/clusterKernels.cu:225-238). */
int cn_allgather_cols_f32(cn_context *ctx, float *d_C, int64_t M, int64_t n_total, void *stream);
int cn_allgather_cols_u8(cn_context *ctx, uint8_t *d_codes, int64_t M, int64_t n_total, void *stream);
/* All-gather of one float per rank (the per-rank codec scales; the commented intent of
 * source/Layer.cpp:354-358). d_vals holds nranks floats; entry [rank] is this rank's input. */
int cn_allgather_scalar_f32(cn_context *ctx, float *d_vals, void *stream);
int cn_allreduce_sum_f32(cn_context *ctx, float *d_buf, int64_t n, void *stream);

/* Symmetric buffers.  A collective call: every rank allocates `bytes` and maps the allocation of every peer (CUDA IPC
 * over NVLink).  When the output of cn_dotmpi_f32 lies in such a buffer, the all-gather is fused into the GEMM: the
 * kernel's epilogue stores each finished tile straight into every peer's copy of C, framed by two flag exchanges, and
 * no gather kernel runs.  This takes the place of the per-shape receive slots that dotMPI keeps in m_matrixCache
 * (source/clusterNet.cpp:523-556).  With one rank the call is an ordinary allocation. */
int cn_sym_alloc(cn_context *ctx, size_t bytes, void **ptr);
int cn_sym_free(cn_context *ctx, void *ptr);

/* dotMPI: replaces ClusterNet::dotMPI (source/clusterNet.cpp:512-697) for a column-sharded B.
 * A is M x K and already resident on every rank; Wshard is this rank's K x cols_local block of the
 * K x n_total weight; C is the full M x n_total col-major output on every rank.
 * exchange = 0: fp32 all-gather; 1: the slice is absmax-scaled, 8-bit compressed, gathered as codes
 * and decoded on arrival (the reference's commented 8-bit ring, source/clusterNet.cpp:670-677). */
int cn_dotmpi_f32(cn_context *ctx, int64_t M, int64_t K, int64_t n_total, const float *d_A,
                  const float *d_Wshard, float *d_C, const cn_epilogue *epi, int mode, int exchange, void *stream);

/* TdotMPI with a column-sharded B (source/clusterNet.cpp:510: dotMPI with the first operand transposed): the same
 * product and exchange as cn_dotmpi_f32, with A given transposed - d_At is the column-major K x M array (leading
 * dimension lda >= K), which is also what a row-major M x K matrix, e.g. the batch as the host holds it, looks like. */
int cn_tdotmpi_f32(cn_context *ctx, int64_t M, int64_t K, int64_t n_total, const float *d_At, int64_t lda,
                   const float *d_Wshard, float *d_C, const cn_epilogue *epi, int mode, int exchange, void *stream);

/* The 8-bit exchange with the decode moved into the consumer (the reference's commented 8-bit ring,
 * source/clusterNet.cpp:670-677, decompresses every received slot before hStackN; here the codes stay codes until the
 * next product reads them).  cn_coded describes a gathered M x n_total matrix held as codes: column block r (the
 * columns rank r owns) was coded with scale scales[r]; own_fp32 holds this rank's own block in exact fp32.
 * All buffers belong to the caller: codes M*n_total bytes, scales nranks floats, own_fp32 M*cols_local floats. */
typedef struct cn_coded {
    uint8_t *codes;
    float *scales;
    float *own_fp32;
    int64_t rows, cols;   /* M, n_total */
} cn_coded;
/* Producer: local GEMM into out->own_fp32 (with the fused epilogue), absmax -> scale, compress, all-gather of codes
 * and scales.  No decode, no fp32 copy of the peers' blocks. */
int cn_dotmpi_to_coded_f32(cn_context *ctx, int64_t M, int64_t K, int64_t n_total, const float *d_A, const float *d_Wshard,
                           cn_coded *out, const cn_epilogue *epi, int mode, void *stream);
/* Consumer: C = act(A . W + bias) with A given as codes; the GEMM's activation pre-pass decodes them (own block from
 * own_fp32) while it transposes and splits.  exchange as in cn_dotmpi_f32 (0: fp32 gather of C, 1: 8-bit gather). */
int cn_dotmpi_from_coded_f32(cn_context *ctx, const cn_coded *A, int64_t n_total, const float *d_Wshard, float *d_C,
                             const cn_epilogue *epi, int mode, int exchange, void *stream);

/* Activation planes made ahead of the product.  The tensor-core kernel reads the activation operand as K-major TF32
 * hi / lo planes, which every product call otherwise makes first (one pass over A: 12 bytes per element).  Where A is
 * known before the product can start - the next batch, while the current step still multiplies - the planes can be made
 * then, on another stream, and the product starts with its first tile:
 *   cn_gemm_prepare_create  allocates planes for an M x K operand and a mode (CN_GEMM_3XTF32 / CN_GEMM_TF32);
 *   cn_gemm_prepare         fills them from A (transA = 0: column-major M x K, lda >= M; transA = 1: the row-major batch,
 *                           K x M column-major, lda >= K, as cn_tdotmpi_f32 takes it) on `stream`;
 *   cn_dotmpi_prepared_f32  = cn_dotmpi_f32 / cn_tdotmpi_f32 on that operand, bit for bit, without the pre-pass.
 * The caller orders the streams (an event after cn_gemm_prepare, waited for by the product's stream) and keeps a handle
 * untouched while a product that reads it may run.  The reference has no counterpart (cuBLAS reads A as it is). */
typedef struct cn_prepared cn_prepared;
int cn_gemm_prepare_create(cn_context *ctx, int64_t M, int64_t K, int mode, cn_prepared **out);
int cn_gemm_prepare(cn_context *ctx, cn_prepared *p, int transA, const float *d_A, int64_t lda, void *stream);
int cn_dotmpi_prepared_f32(cn_context *ctx, const cn_prepared *p, int64_t n_total, const float *d_Wshard, float *d_C,
                           const cn_epilogue *epi, int exchange, void *stream);
int cn_gemm_prepare_destroy(cn_prepared *p);

/* dotTMPI: replaces ClusterNet::dotTMPI (source/clusterNet.cpp:511,628-642,698-727), the backward product through a
 * column-sharded weight: out (M x R) = A (M x n_total) . B^T, where this rank holds the R x cols_local block of the
 * R x n_total matrix B.  Each rank multiplies its column slice of A with its shard (transposed) and the full-size
 * partial products are summed over the ranks (all-reduce in place of the reference's ring of partials + add loop). */
int cn_dottmpi_f32(cn_context *ctx, int64_t M, int64_t n_total, int64_t R, const float *d_A, const float *d_Bshard,
                   float *d_out, int mode, void *stream);
/* dot / TdotMPI into a column-sharded output (source/clusterNet.cpp:510,612-625,729-730): out_shard (M x cols_local)
 * = op(A) . B[:, shard], B being a full K x n_total matrix on every rank; no communication.  transA = 1 gives
 * TdotMPI (A stored K x M). */
int cn_dot_sharded_out_f32(cn_context *ctx, int transA, int64_t M, int64_t K, int64_t n_total, const float *d_A,
                           const float *d_B, float *d_out_shard, int mode, void *stream);

/* ---------------------------------------------------------------------------------------------
 * Data-parallel training step (the reference's Layer class, source/Layer.cpp): elementwise pieces and the 8-bit
 * gradient exchange.
 * ------------------------------------------------------------------------------------------- */
/* softmax over the columns of each row (kSoftMax, source/clusterKernels.cu:651-688; same order, same __expf). */
int cn_softmax(cn_context *ctx, const float *d_A, float *d_out, int64_t rows, int64_t cols, void *stream);
/* one-hot target matrix from a rows x 1 label vector stored as floats (kCreate_t_matrix, :775-790; zero fill included). */
int cn_create_t_matrix(cn_context *ctx, const float *d_labels, float *d_out, int64_t rows, int64_t cols, void *stream);
/* add / sub / mul / scalarMul (kAdd :313-320, kSub :332-339, kMul :323-330). */
int cn_add(cn_context *ctx, const float *d_a, const float *d_b, float *d_out, int64_t n, void *stream);
int cn_sub(cn_context *ctx, const float *d_a, const float *d_b, float *d_out, int64_t n, void *stream);
int cn_mul(cn_context *ctx, const float *d_a, const float *d_b, float *d_out, int64_t n, void *stream);
int cn_scalar_mul(cn_context *ctx, const float *d_a, float s, float *d_out, int64_t n, void *stream);
/* div (kDiv :341-348, fdividef), scalarAdd (kScalarAdd), abs (kAbs :429-436), square (kSquare :420-427, powf(x,2)). */
int cn_div(cn_context *ctx, const float *d_a, const float *d_b, float *d_out, int64_t n, void *stream);
int cn_scalar_add(cn_context *ctx, const float *d_a, float s, float *d_out, int64_t n, void *stream);
int cn_abs(cn_context *ctx, const float *d_a, float *d_out, int64_t n, void *stream);
int cn_square(cn_context *ctx, const float *d_a, float *d_out, int64_t n, void *stream);
/* max (source/basicOps.cu:1076-1081): thrust::reduce with maximum, seeded with -1.0f, into *d_out (device). */
int cn_max_f32(cn_context *ctx, const float *d_A, int64_t n, float *d_out, void *stream);
/* Nesterov_weight_update (kNesterov_weight_update, :1064-1077): g = lr grad / batch_size; m = momentum m - g; w -= g. */
int cn_nesterov_update(cn_context *ctx, const float *d_grad, float *d_w, float *d_m, float learning_rate, int64_t batch_size,
                       float momentum, int64_t n, void *stream);
/* derivative of the unit from its activation (Layer::activation_gradient, source/Layer.cpp:180-200): ReLU x>0?1:0
 * (kRectifiedLinear_Derivative :813-821), logistic a(1-a), double ReLU 0<a<1?1:0. */
int cn_activation_gradient(cn_context *ctx, const float *d_activation, int activation, float *d_out, int64_t n, void *stream);
/* The same derivative multiplied into an error matrix in one pass: error_out = error_in * f'(activation); when
 * d_gradient_out is not NULL it also receives f'(activation) (the reference stores it in the layer's `out` matrix and
 * multiplies with a second kernel, source/Layer.cpp:323-329).  Bit-identical to cn_activation_gradient + cn_mul. */
int cn_mul_activation_gradient(cn_context *ctx, const float *d_error_in, const float *d_activation, int activation,
                               float *d_gradient_out, float *d_error_out, int64_t n, void *stream);
/* Output layer in one pass: softmax over the columns of each row (as cn_softmax) and error = softmax - onehot(label)
 * (softmax, create_t_matrix and sub of the reference's step, source/Layer.cpp:163-165,318-322).  d_softmax_out may be
 * d_A.  Bit-identical to the three calls. */
int cn_softmax_error(cn_context *ctx, const float *d_A, const float *d_labels, float *d_softmax_out, float *d_error_out,
                     int64_t rows, int64_t cols, void *stream);
/* RMSprop_with_weight_update (kRMSprop_with_weight_update, :1306-1325): RMS = m RMS + (1-m) g^2; w -= lr g / (sqrt(RMS)+1e-8). */
int cn_rmsprop_update(cn_context *ctx, float *d_rms, const float *d_grad, float *d_w, float rms_multiplier, float learning_rate,
                      int64_t n, void *stream);
/* Layer::MPI_synchronization_async + wait_for_synchronization (source/Layer.cpp:341-437) in one call: the rank's
 * gradient is 8-bit compressed, codes (and scales) are all-gathered, and the peers' decoded gradients are added to
 * d_grad in rank order — one fused decode-and-sum pass instead of a decompression_8bit + add pair per peer.
 * fixed_precision > 0 uses that scale on every rank (the reference's MAX_GRAD_VALUE = 1.0f); fixed_precision <= 0 uses
 * each rank's absmax and gathers the scales (what the reference's commented-out code intended; as committed it decodes
 * with an uninitialised array). */
int cn_grad_sync_8bit(cn_context *ctx, float *d_grad, int64_t n, float fixed_precision, void *stream);
/* The same exchange for several tensors that lie back to back in d_grad (segment_sizes is a HOST array of num_segments
 * element counts, e.g. the weight gradients of all layers of a step): every segment is coded with its own scale and the
 * result equals num_segments calls of cn_grad_sync_8bit bit for bit, but there is one all-gather and one decode-and-sum
 * pass per step instead of one per layer (the reference exchanges layer by layer, source/Layer.cpp:341-390). */
int cn_grad_sync_8bit_multi(cn_context *ctx, float *d_grad, const int64_t *segment_sizes, int num_segments,
                            float fixed_precision, void *stream);
/* cn_grad_sync_8bit_multi followed by cn_rmsprop_update(d_rms, d_grad, d_w, ...) over the same elements (the reference's
 * wait_for_synchronization + weight_update pair, source/Layer.cpp:250-261,400-437), with the update done inside the pass
 * that sums the decoded gradients: one launch and one trip of the gradient through memory less; gradient, RMS state
 * and weights come out as from the two calls, bit for bit. */
int cn_grad_sync_8bit_rmsprop(cn_context *ctx, float *d_grad, const int64_t *segment_sizes, int num_segments,
                              float fixed_precision, float *d_rms, float *d_w, float rms_multiplier, float learning_rate,
                              void *stream);
/* How cn_grad_sync_8bit_multi moves its blocks.  on != 0 (the default with one process per GPU): every rank stores its
 * block straight into every peer's memory (one kernel: "your area may be written" / 16-byte stores over NVLink / "my block
 * has arrived", every wait bounded and reported by cn_gemm_check_status as CN_ERR_TIMEOUT) - one NVLink hop instead of
 * the steps of a ring, and no library launch; a single tensor of up to 4 Mi elements with its own absmax is coded and
 * pushed by ONE kernel.  on == 0: ncclAllGather.  The results are identical bit for bit.  Call it
 * on every rank alike.  After a CN_ERR_TIMEOUT (a peer never took part) the ranks' exchange counters no longer agree:
 * re-create the communicator (cn_comm_destroy + cn_comm_init_rank), as after cn_comm_sync gave up on a collective.  The reference sends its codes with MPI_Isend / MPI_Recv, rank to rank (source/Layer.cpp:364-390). */
int cn_comm_set_push_exchange(cn_context *ctx, int on);

/* ---------------------------------------------------------------------------------------------
 * Batch allocator (dense path).  Replaces BatchAllocator::init / init_batch_buffer /
 * broadcast_batch_to_processes / allocate_next_batch_async / replace_current_batch_with_next
 * (source/batchAllocator.cpp:101-251,253-338,399-425,759-864,977-1053).
 * The full data set stays in host memory (row-major); each step stages the next batch's rows in a
 * pinned buffer, copies them on side streams, and the swap transposes them to col-major into the
 * current-batch matrices on the compute stream, ordered by events instead of stream synchronisation.
 * ------------------------------------------------------------------------------------------- */
typedef struct cn_batch cn_batch;
int cn_batch_create(cn_context *ctx, const float *h_X, const float *h_y, int64_t rows, int64_t cols_X, int64_t cols_y,
                    int64_t batch_size, int skip_last_batch, cn_batch **out);
/* cn_batch_create with options (flags, OR-ed):
 *   CN_BATCH_KEEP_ROW_MAJOR  the row-major device copy of the current batch stays valid until the next swap (two buffers
 *       alternate); cn_batch_current_row_major returns it.  Read as a column-major cols_X x rows matrix it is the
 *       transposed operand of cn_tdotmpi_f32 / cn_gemm_f32(transA = 1), so a product that consumes the batch needs no
 *       col-major copy of it (the reference always makes one: to_col_major in replace_current_batch_with_next,
 *       source/batchAllocator.cpp:986-990).
 *   CN_BATCH_NO_COL_MAJOR    X is not transposed at the swap; cn_batch_current / cn_batch_swap return d_X = NULL.
 *   CN_BATCH_SHARDED_UPLOAD  collective over the context's communicator; EVERY rank passes the same host data set (the
 *       Matrix* form of BatchAllocator::init, in which every process holds the data and stages its own batches,
 *       source/batchAllocator.cpp:411-440).  Rank r uploads only its block of floor(batch/G) rows (last rank: plus the
 *       remainder) over its own PCIe link and writes that block into every peer's buffer over NVLink; two bounded
 *       cross-GPU flag exchanges on the copy stream order the writes (a peer that never takes part surfaces as
 *       CN_ERR_TIMEOUT from cn_gemm_check_status).  Ignored with one rank.
 *   CN_BATCH_PUSH_BY_KERNEL  with CN_BATCH_SHARDED_UPLOAD: the block goes to the peers through one kernel's stores
 *       instead of one copy-engine transfer per peer (fewer host calls per step; needs SM time beside the product).
 *   CN_BATCH_LOOKAHEAD       two X copies in flight instead of one (three row-major buffers; implies
 *       CN_BATCH_KEEP_ROW_MAJOR): cn_batch_copy_next_async also starts the copy of the batch AFTER the next one as soon as
 *       its buffer is free, so a copy has two steps to finish in.  For steps shorter than one upload's latency (many
 *       ranks, each waiting for every peer's block).  The order of the batches is unchanged. */
#define CN_BATCH_KEEP_ROW_MAJOR 1
#define CN_BATCH_NO_COL_MAJOR 2
#define CN_BATCH_SHARDED_UPLOAD 4
#define CN_BATCH_PUSH_BY_KERNEL 8
#define CN_BATCH_LOOKAHEAD 16
int cn_batch_create_ex(cn_context *ctx, const float *h_X, const float *h_y, int64_t rows, int64_t cols_X, int64_t cols_y,
                       int64_t batch_size, int skip_last_batch, int flags, cn_batch **out);
/* Row-major device copy (batch_rows x cols_X, leading dimension cols_X) of the current batch; needs CN_BATCH_KEEP_ROW_MAJOR. */
int cn_batch_current_row_major(const cn_batch *b, float **d_X_row_major, int64_t *batch_rows);
/* Measurement aid for the sharded upload (takes the place of the reference's tick/tock around its batch copies):
 * enable != 0 makes the following cn_batch_copy_next_async calls record CUDA events on the copy stream; ms4 receives the
 * phases of the last recorded copy in milliseconds: waiting for the peers' "buffer free" flags, the host-to-device copy of
 * the own block, the push to the peers, waiting for the peers' "arrived" flags. */
int cn_batch_profile(cn_batch *b, int enable, float *ms4);
/* The row-major device copy of the NEXT batch (the one the next cn_batch_swap makes current) and its row count, for work
 * that can start before the swap, e.g. cn_gemm_prepare on another stream: `stream` is made to wait for the batch's copy.
 * Needs CN_BATCH_KEEP_ROW_MAJOR and a copy under way (cn_batch_copy_next_async).  The buffer stays valid until the swap
 * after next. */
int cn_batch_next_row_major(cn_batch *b, void *stream, float **d_X_row_major, int64_t *batch_rows);
int cn_batch_destroy(cn_batch *b);
int64_t cn_batch_total_batches(const cn_batch *b);
/* The batch that is current now (after cn_batch_create: the first batch, as BatchAllocator::init leaves it). */
int cn_batch_current(const cn_batch *b, float **d_X, float **d_y, int64_t *batch_rows);
/* BatchAllocator::SKIP_LAST_BATCH is a public field that callers flip after init (source/batchAllocator.h:37). */
int cn_batch_set_skip_last(cn_batch *b, int skip_last_batch);
/* Stage + asynchronous copy of the next batch (allocate_next_batch_async). */
int cn_batch_copy_next_async(cn_batch *b);
/* Make the next batch current (replace_current_batch_with_next): waits (on the device, through an
 * event) for the copies, transposes into the current-batch buffers on `stream`, advances the counter
 * with wrap-around.  Returns the device pointers and the row count of the batch (the last batch of an
 * epoch may be short). */
int cn_batch_swap(cn_batch *b, void *stream, float **d_X, float **d_y, int64_t *batch_rows);

/* Named cumulative timers: ClusterNet::tick / tock (source/clusterNet.cpp:798-840). */
int cn_tick(cn_context *ctx, const char *name, void *stream);
int cn_tock(cn_context *ctx, const char *name, void *stream, float *cumulative_ms);

#ifdef __cplusplus
}
#endif
#endif /* CLUSTERNET_B200_H */
