/*
 * zbal expert-parallel MoE operations (C entry points). A zbal_moe_t owns the receive areas of one
 * communicator in the symmetric heap (token rows, 1x128 scales, origins, combine slots, count table,
 * flags); the operations enqueue kernels on the caller's stream and return.
 *
 *   normal mode:      zbal_dispatch_normal_layout -> zbal_dispatch_normal_notify -> zbal_dispatch_normal
 *                     -> (caller's expert FFN on the received rows) -> zbal_combine_normal
 *   low-latency mode: zbal_dispatch_low_latency -> (FFN) -> zbal_combine_low_latency   (one launch each)
 *   fused:            zbal_fused_deep_moe  (dispatch + grouped fp8 GEMMs + combine)
 *
 * Names follow app/zbal/src/include/zbal_operations.h of the reference; the argument lists differ where the
 * design differs: the receive buffers belong to the zbal_moe_t (peers store straight into them, so they
 * must sit at the same heap offset on every rank), rows travel as block-scaled fp8 e4m3 or raw bf16
 * instead of int8, and there is no load-balance matrix (NVSwitch gives every pair of GPUs full bandwidth).
 * All tensors are device pointers; int32 for indices and counts, fp32 for weights, bf16 for tokens.
 * Members of the communicator must issue the same sequence of dispatch / combine calls.
 */
#ifndef MF_B200_ZBAL_MOE_H
#define MF_B200_ZBAL_MOE_H

#include "zbal_def.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void *zbal_moe_t;

typedef struct {
    uint32_t maxTokens;   /* tokens a rank dispatches per call, at most */
    uint32_t hidden;      /* multiple of 128, at most 7168 */
    uint32_t experts;     /* all experts of the group, a multiple of the group size, at most 1024 */
    uint32_t topk;        /* at most 16 */
    uint32_t maxRecv;     /* rows of the receive buffers; 0 = maxTokens * groupSize * min(topk, experts / groupSize) */
    uint32_t rawBf16;     /* 0: rows travel as fp8 e4m3 with 1x128 scales (quantised in the push kernel); 1: raw bf16 rows */
} zbal_moe_options_t;

/* device views of the receive areas of this rank (valid rows: rowOffsets[localExperts] of the last dispatch) */
typedef struct {
    void *recvTokens;     /* [maxRecv, hidden] fp8 e4m3 (or bf16 when rawBf16 is set) */
    float *recvScales;    /* [maxRecv, hidden / 128] */
    int32_t *recvInfo;    /* [maxRecv, 4]: source rank, token, k slot, routing weight (fp32 bits) */
    uint32_t maxRecv;
    uint32_t localExperts;
} zbal_moe_buffers_t;

/* Collective over the communicator's members. */
int32_t zbal_moe_create(zbal_comm_t comm, const zbal_moe_options_t *options, zbal_moe_t *moe);
int32_t zbal_moe_destroy(zbal_moe_t moe);
int32_t zbal_moe_get_buffers(zbal_moe_t moe, zbal_moe_buffers_t *buffers);
/* 0 = no kernel of this object ever gave up a wait or dropped a row; else the first code recorded */
int32_t zbal_moe_get_status(zbal_moe_t moe, int32_t *status);

/* topkIndex [tokens, topk] -> tokensPerRank [groupSize], tokensPerExpert [experts], sendTokensIndex [tokens * topk]
 * (position of every (token, k) inside its expert, token order), isTokenInRank [tokens, groupSize] (uint8). */
int32_t zbal_dispatch_normal_layout(zbal_moe_t moe, const int32_t *topkIndex, int64_t tokens, int32_t *tokensPerRank,
                                    int32_t *tokensPerExpert, int32_t *sendTokensIndex, uint8_t *isTokenInRank, zbal_stream_t stream);
/* Count exchange. Outputs (device, no host read): recvTokensPerExpert [localExperts], rowOffsets [localExperts + 1]
 * (rowOffsets[localExperts] = rows this rank receives), pushTargetOffset [experts], srcOffsets [localExperts * groupSize]. */
int32_t zbal_dispatch_normal_notify(zbal_moe_t moe, const int32_t *tokensPerExpert, int32_t *recvTokensPerExpert, int32_t *rowOffsets,
                                    int32_t *pushTargetOffset, int32_t *srcOffsets, zbal_stream_t stream);
/* Quantise (unless rawBf16) and push every (token, k) row into the owner's receive buffers, then wait
 * until every peer's rows for this rank have landed. */
int32_t zbal_dispatch_normal(zbal_moe_t moe, const void *srcTokens, int64_t tokens, const int32_t *topkIndex, const float *topkWeights,
                             const int32_t *sendTokensIndex, const int32_t *pushTargetOffset, zbal_stream_t stream);
/* srcTokens: expert outputs [rows, hidden] bf16 in the row order of the receive buffers (leading dimension ld,
 * in elements); rowsDev: device int32 with the number of rows (= &rowOffsets[localExperts]). Rows are multiplied
 * by their routing weight when weighted != 0, pushed home and summed per token into destTokens [tokens, hidden]. */
int32_t zbal_combine_normal(zbal_moe_t moe, const void *srcTokens, int64_t ld, const int32_t *rowsDev, int32_t weighted,
                            const int32_t *topkIndex, int64_t tokens, void *destTokens, zbal_stream_t stream);

/* One cooperative launch; may be captured in a CUDA graph and replayed. Outputs as for layout + notify. */
int32_t zbal_dispatch_low_latency(zbal_moe_t moe, const void *x, int64_t tokens, const int32_t *topkIndex, const float *topkWeights,
                                  int32_t *sendTokensIndex, int32_t *tokensPerExpert, int32_t *recvTokensPerExpert, int32_t *rowOffsets,
                                  int32_t *pushTargetOffset, int32_t *srcOffsets, zbal_stream_t stream);
/* homeWeights: optional [tokens, topk] fp32 applied on the home rank (then pass weighted = 0). */
int32_t zbal_combine_low_latency(zbal_moe_t moe, const void *expandX, int64_t ld, const int32_t *rowsDev, int32_t weighted,
                                 const int32_t *topkIndex, const float *homeWeights, int64_t tokens, void *xOut, zbal_stream_t stream);

/* dispatch + GEMM1 (gate/up, SwiGLU, requantisation to fp8) + GEMM2 with the weighted push home in its epilogue + slot
 * reduce. gmm1Weight [localExperts, 2 * inter, hidden] fp8 with gate/up rows interleaved per
 * zbal_fused_deep_moe_gate_up_tile() rows (128 when hidden is a multiple of 256: the block-scaled tensor-core kernel;
 * else 64), gmm1Scale [localExperts, 2 * inter / 128, hidden / 128]; gmm2Weight [localExperts, hidden, inter], gmm2Scale
 * [.., hidden / 128, inter / 128]. Every scale is a power of two (the smallest with amax / scale <= 448).
 * workspace: device memory of zbal_fused_deep_moe_workspace(moe, inter) bytes. */
uint64_t zbal_fused_deep_moe_workspace(zbal_moe_t moe, uint32_t inter);
int32_t zbal_fused_deep_moe_gate_up_tile(zbal_moe_t moe, uint32_t inter);
int32_t zbal_fused_deep_moe(zbal_moe_t moe, const void *x, int64_t tokens, const int32_t *topkIndex, const float *topkWeights,
                            const void *gmm1Weight, const float *gmm1Scale, const void *gmm2Weight, const float *gmm2Scale, uint32_t inter,
                            void *workspace, void *xOut, zbal_stream_t stream);

/* Smooth quantisation (the reference's SMOOTH_QUANT execution flag): every token row is multiplied by scales[hidden]
 * (device fp32, caller-owned, must stay valid) before the dispatch kernels quantise it; the expert weights carry the
 * inverse factors. NULL switches it off. Applies to normal, low-latency and fused dispatch of this object. */
int32_t zbal_moe_set_smooth_scales(zbal_moe_t moe, const float *scales);

/* Host-side plan of the reference's load balancing (which helper rank pushes which range of which rank's tokens);
 * counts: [ranks, experts] send counts, matrix: [ranks, ranks * 2] int32 out. Not used by the kernels here. */
int32_t zbal_moe_balance_matrix(const int32_t *counts, uint32_t ranks, uint32_t experts, uint32_t topk, float factorHigh, float factorLow,
                                uint32_t minTokens, int32_t *matrix);

#ifdef __cplusplus
}
#endif
#endif
