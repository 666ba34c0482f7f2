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

struct cn_gemm_workspace {
    void *ptr[CN_GEMM_SLOTS] = {nullptr, nullptr, nullptr, nullptr};
    size_t bytes[CN_GEMM_SLOTS] = {0, 0, 0, 0};
    unsigned int *d_status = nullptr;   // word 0: set by a kernel whose bounded wait ran out; words 16..: split-K tickets
    void *encode_fn = nullptr;          // cuTensorMapEncodeTiled, resolved once
    bool profile = false;               // bracket main-kernel launches with events
    std::vector<cudaEvent_t> prof_events;   // start, stop, start, stop, ...
    size_t prof_used = 0;
};

// Grow-only scratch buffers owned by the context.
int cn_gemm_scratch(cn_context *ctx, int slot, size_t bytes, void **out);

bool cn_gemm_tc_supported(cn_context *ctx, int transA, int transB, int64_t M, int64_t N, int64_t K,
                          const float *A, int64_t lda, const float *B, int64_t ldb, const float *C, int64_t ldc);
bool cn_gemm_tc_can_fuse_maxout(int level);
int cn_gemm_tc_launch(cn_context *ctx, int64_t M, int64_t N, int64_t K, const float *A, int64_t lda,
                      const float *B, int64_t ldb, float *C, int64_t ldc, const cn_epilogue *epi, int mode, cudaStream_t s);
