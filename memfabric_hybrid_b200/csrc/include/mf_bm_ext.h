/*
 * Entry points of the Big Memory API that go beyond the reference's ABI (smem_bm.h). They live in libmf_smem.so.
 */
#ifndef MF_B200_BM_EXT_H
#define MF_B200_BM_EXT_H

#include "smem_bm.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Counters of what the copy paths did since the pool was created, in the order: kernel launches, kernel work chunks,
 * copy-engine copies, host memcpys, process-VM copies, coalesced items. */
int32_t mf_bm_copy_stats(smem_bm_t handle, uint64_t out[6]);

/* Shape of the bulk-copy (TMA) variant of the xcopy kernel for the launches that follow: pipelines per CTA (0: register-copy
 * kernel only), stages per pipeline (>= 4), KiB per stage. */
int32_t mf_xcopy_bulk_config(int pipes, int stages, int pieceKb);

/* Prepared batches: the low-latency submission path for a batch that is sent again and again (the KV blocks of a layout that
 * does not change, the weight shards of a reshard plan).
 *   mf_bm_batch_create   validates every (source, destination, size) triple like smem_bm_copy_batch, merges neighbours, cuts
 *                        the runs into work chunks and stores the descriptors in pinned memory that belongs to the batch.
 *                        Device-to-device copy types only (SMEMB_COPY_L2G, _G2L, _G2G).
 *   mf_bm_batch_launch   ONE kernel launch on the caller's stream; the host touches no descriptor and no shared state, so the
 *                        call may be recorded into a CUDA graph. Asynchronous: order it with the stream.
 *   mf_bm_batch_bytes    bytes one launch moves.
 *   mf_bm_batch_destroy  after the stream has passed the last launch (and after every graph that recorded one is destroyed).
 * A batch names mapped memory of the members that were joined when it was created: after a member leaves, launches are
 * refused with SMEM_NOT_CONNECTED; create it again. */
typedef struct mf_bm_batch *mf_bm_batch_t;
int32_t mf_bm_batch_create(smem_bm_t handle, const smem_batch_copy_params_t *params, smem_bm_copy_type_t t, mf_bm_batch_t *out);
int32_t mf_bm_batch_launch(mf_bm_batch_t batch, void *stream);
uint64_t mf_bm_batch_bytes(mf_bm_batch_t batch);
int32_t mf_bm_batch_destroy(mf_bm_batch_t batch);

#ifdef __cplusplus
}
#endif
#endif
