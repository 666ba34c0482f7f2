// Internal interface between the GEMM entry point (cn_gemm.cu) and the tensor-core kernel (cn_gemm_tc.cu).
#pragma once
#include "cn_internal.h"

enum {
    CN_GEMM_SLOT_MAXOUT = 0,   // full product ahead of an un-fused maxout
    CN_GEMM_SLOT_ASPLIT = 1,   // activations re-laid K-major as TF32 hi / lo planes
    CN_GEMM_SLOT_SPLITK = 2,   // per-split partial tiles of a split-K launch
    CN_GEMM_SLOT_EXCHANGE = 3, // codes + scales of the 8-bit exchange in dotMPI
    CN_GEMM_SLOTS = 4
};

#define CN_GEMM_MAX_TICKETS 4096

// Activations that exist only as gathered 8-bit codes (plus this rank's own block in fp32): set by
// cn_dotmpi_from_coded_f32 right before the dispatch, consumed by the tensor-core launch, whose pre-pass then decodes
// while it transposes and splits.
struct cn_coded_src {
    const uint8_t *codes = nullptr;
    const float *scales = nullptr;
    const float *own_fp32 = nullptr;
    int nranks = 1, own_rank = 0;
};

// The K-major TF32 hi / lo planes of an activation operand, made ahead of the product that consumes them
// (cn_gemm_prepare): the product's own pre-pass is then skipped.  `hi` holds both planes back to back.
struct cn_prepared {
    cn_context *ctx = nullptr;
    float *hi = nullptr, *lo = nullptr;
    int64_t M = 0, K = 0, Kpad = 0;
    int mode = 0;
    bool filled = false;
};

struct cn_gemm_workspace {
    void *ptr[CN_GEMM_SLOTS] = {nullptr, nullptr, nullptr, nullptr};
    size_t bytes[CN_GEMM_SLOTS] = {0, 0, 0, 0};
    unsigned int *d_status = nullptr;   // word 0: set by a kernel whose bounded wait ran out
    void *encode_fn = nullptr;          // cuTensorMapEncodeTiled, resolved once
    const cn_coded_src *coded_src = nullptr;   // one-shot: see cn_coded_src
    const cn_prepared *prepared = nullptr;   // one-shot: planes made ahead of the launch (cn_gemm_prepare)
    // test and sweep knobs (0 = automatic choice): W tiles per CTA, K splits, K blocks per accumulation chain.  Seeded once,
    // when the workspace is made, from CN_GEMM_NT / CN_GEMM_SPLITS / CN_GEMM_CHAIN; changed with cn_gemm_set_tuning.
    int force_nt = 0, force_splits = 0, force_chain = 0;
    bool profile = false;               // bracket main-kernel launches with events
    std::vector<cudaEvent_t> prof_events;   // start, stop, start, stop, ...
    size_t prof_used = 0;
};

// The only way a workspace is made: reads the environment knobs once.
cn_gemm_workspace *cn_gemm_workspace_new();

// Grow-only scratch buffers owned by the context.
int cn_gemm_scratch(cn_context *ctx, int slot, size_t bytes, void **out);

// Peer windows of the output for the fused all-gather: the tensor-core kernel's epilogue stores each finished tile into
// the same window of every peer's C (plain stores to peer memory over NVLink) in addition to the local C.
#define CN_MAX_PEERS 7
struct cn_peer_out {
    int npeers = 0;
    float *C[CN_MAX_PEERS] = {};          // peer addresses of the window that d_C points to locally
    const unsigned int *ready = nullptr;  // local flags, one per rank, raised by the peers when they may be written to
    unsigned int *const *peer_flags = nullptr;   // device table: flag block of every rank (this kernel raises its own "ready")
    int nranks = 0;
    int my_rank = 0;
    unsigned int epoch = 0;
};

bool cn_gemm_tc_supported(cn_context *ctx, int transA, int transB, int64_t M, int64_t N, int64_t K,
                          const float *A, int64_t lda, const float *B, int64_t ldb, const float *C, int64_t ldc);
bool cn_gemm_tc_can_fuse_maxout(int level);
// the activation pre-pass alone, into caller-owned planes (lo == nullptr in the single-pass mode)
int cn_gemm_tc_split_activations(cn_context *ctx, int transA, int64_t M, int64_t K, const float *A, int64_t lda, float *hi, float *lo,
                                 cudaStream_t s);
int cn_gemm_tc_launch(cn_context *ctx, int64_t M, int64_t N, int64_t K, const float *A, int64_t lda,
                      const float *B, int64_t ldb, float *C, int64_t ldc, const cn_epilogue *epi, int mode, cudaStream_t s,
                      const cn_peer_out *peers = nullptr, int transA = 0, int transB = 0);
// cn_gemm_f32 with optional peer windows; *used_peers tells whether the launch took them (tensor-core path only).
int cn_gemm_dispatch(cn_context *ctx, int transA, int transB, int64_t M, int64_t N, int64_t K, const float *d_A, int64_t lda,
                     const float *d_B, int64_t ldb, float *d_C, int64_t ldc, const cn_epilogue *epi, int mode, void *stream,
                     const cn_peer_out *peers, bool *used_peers);
