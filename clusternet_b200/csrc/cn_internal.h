// Shared declarations of the library's translation units (not part of the public C ABI).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <map>
#include <string>
#include <vector>
#include "../../include/clusternet_b200.h"

#define CN_CODEBOOK_N 126
#define CN_NUM_THR 127      // decision thresholds of the compressor
#define CN_NUM_LEVELS 128   // levels they separate: 254, 0..125, 127
#define CN_MAX_PARTIALS 4096

void cn_set_error(const char *fmt, ...);
// every kernel launch of the library is counted (cn_kernel_launches), so that callers can tell library work from fallbacks
void cn_count_launch(void);
int cn_cuda_fail(cudaError_t e, const char *what);

#define CN_CUDA(call)                                         \
    do {                                                      \
        cudaError_t e__ = (call);                             \
        if (e__ != cudaSuccess) return cn_cuda_fail(e__, #call); \
    } while (0)

#define CN_REQUIRE(cond, status, ...)      \
    do {                                   \
        if (!(cond)) {                     \
            cn_set_error(__VA_ARGS__);     \
            return (status);               \
        }                                  \
    } while (0)

struct cn_timer_slot {
    cudaEvent_t start = nullptr, stop = nullptr;
    float cumulative_ms = 0.f;
};

struct cn_gemm_workspace;  // owned by cn_gemm.cu
struct cn_comm_state;      // owned by cn_comm.cu

struct cn_context {
    int device = 0;
    int sm_count = 0;
    // codec tables (device)
    float *d_tbl = nullptr;            // 128 floats: codebook[0..125], +inf, +inf
    uint32_t *d_thr = nullptr;         // 128 words: 127 thresholds (fp32 bit patterns of |x/precision|) + 0xffffffff pad
    uint8_t *d_level_codes = nullptr;  // 128 bytes
    float h_tbl[128];
    uint32_t h_thr[128];
    uint8_t h_level_codes[128];
    // boundaries of the compressor's levels in |x| space for the last host-side scale (cn_compress_8bit), see cn_codec.cu
    bool codec_cache_valid = false, codec_cache_ok = false;
    uint32_t codec_cache_pbits = 0;
    uint32_t codec_cache_X[128];
    // reduction scratch: per-CTA partial maxima + a ticket counter that the last CTA resets
    float *d_partials = nullptr;
    unsigned int *d_ticket = nullptr;   // 64 bytes: word 0 = absmax ticket, words 4 and 5 = grid barrier of the fused compressor (arrivals, generation)
    // GEMM
    cn_gemm_workspace *gemm = nullptr;
    const char *gemm_last_path = "";
    // communicator
    cn_comm_state *comm = nullptr;
    // timers
    std::map<std::string, cn_timer_slot> timers;
};

// cn_gemm.cu
void cn_gemm_workspace_free(cn_context *ctx);
// Device status block of the context (word 0: code of the first bounded wait that ran out, read by cn_gemm_check_status),
// allocated and zeroed on first use.
int cn_status_block(cn_context *ctx, unsigned int **d_status);
// cn_comm.cu
void cn_comm_state_free(cn_context *ctx);
// Addresses of a symmetric buffer on every rank ([nranks] entries, own rank = local); false if `local` is not inside one.
bool cn_comm_sym_peers(cn_context *ctx, const void *local, size_t bytes, void **peers_out);
// Reserves `count` consecutive flag slots of the context's cross-GPU flag block (same call order on every rank).
int cn_comm_flag_slots(cn_context *ctx, int count, int *first_slot);
// Queues the one-warp kernel that raises this rank's flag of `slot` on every peer and waits (bounded) for theirs.
int cn_comm_flag_barrier(cn_context *ctx, int slot, unsigned int epoch, cudaStream_t s);

static inline cudaStream_t cn_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

// Pushed block exchange, seen from the codec: where this rank's codes and scale go in every peer's area, and the flags
// that frame the stores ("your area may be written" = slot, "my block has arrived" = slot + 1; see cn_push_exchange_kernel).
struct cn_codec_push {
    uint8_t *codes_dst[7];
    float *scale_dst[7];
    int ndst;
    unsigned int *const *peer_flags;
    const unsigned int *local_flags;
    int nranks, my_rank, slot;
    unsigned int *state;   // [0] epoch of the last finished exchange
};
// scale = absmax(A); codes = compress(A, scale), the codes and the scale stored locally AND in every peer's area, the two
// flag exchanges included: one cooperative launch.  *done = 0 when the tensor is no case for it (too large, unaligned):
// nothing was launched and the caller takes the separate calls.
int cn_absmax_compress_push(cn_context *ctx, const float *d_A, int64_t n, float *d_scale_out, uint8_t *d_codes, const cn_codec_push *push,
                            void *stream, int *done);
// Fills the destinations for a block of block_bytes whose codes start at the block's first byte and whose scale lies at
// scale_offset; only valid for the area cn_comm_push_area returned for that block size.
int cn_comm_push_params(cn_context *ctx, size_t block_bytes, size_t scale_offset, cn_codec_push *out);
