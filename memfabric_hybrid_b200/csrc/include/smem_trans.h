/*
 * Transfer (TRANS): point-to-point movement between processes identified by "ip:port[_pid]" strings
 * (prefill/decode KV hand-off). A process registers buffers; peers of the opposite role import them
 * and read/write by the owner's *local* addresses.
 * ABI parity: src/smem/include/host/smem_trans.h:30-252, smem_trans_def.h:29-60 of the reference.
 */
#ifndef MF_B200_SMEM_TRANS_H
#define MF_B200_SMEM_TRANS_H

#include "smem.h"
#include "smem_bm_def.h"

#ifdef __cplusplus
extern "C" {
#endif

#define SMEM_TRANS_RANK_COUNT_MAX (512U)
typedef void *smem_trans_t;

typedef enum {
    SMEM_TRANS_NONE = 0,
    SMEM_TRANS_SENDER,
    SMEM_TRANS_RECEIVER,
    SMEM_TRANS_BOTH,
    SMEM_TRANS_BUTT
} smem_trans_role_t;

#define SMEM_TRANS_QUANT_FP8_E4M3 (1u << 0) /* extension: output format of smem_trans_batch_quant_write */

typedef struct {
    smem_trans_role_t role;
    uint32_t initTimeout; /* seconds, default 120 */
    uint32_t deviceId;
    uint32_t flags;
    smem_bm_data_op_type dataOpType;
} smem_trans_config_t;

/* Quantising write: each `unitNum`-element unit of the bf16/fp16 source is scaled to int8 with its own
 * dynamic scale while it is pushed; scale[i] is the remote address receiving the fp32 dequant factors. */
typedef struct {
    const char *remoteUniqueId;
    void **localAddrs;
    void **remoteAddrs;
    size_t *dataSizes;
    float **scale;
    float **offset;
    uint32_t batchSize;
    uint32_t unitNum;
    void *stream;
    uint32_t inputType; /* 0 bf16, 1 fp16 */
    uint32_t flags;     /* SMEM_TRANS_QUANT_FP8_E4M3: fp8 e4m3 with one factor per 128 elements instead of int8 */
} smem_trans_quant_copy_param_t;

typedef void (*smem_trans_peer_down_callback_t)(const char *peerUniqueId, void *userData);

int32_t smem_trans_config_init(smem_trans_config_t *config);
int32_t smem_trans_init(const smem_trans_config_t *config);
void smem_trans_uninit(uint32_t flags);
smem_trans_t smem_trans_create(const char *storeUrl, const char *uniqueId, const smem_trans_config_t *config);
void smem_trans_destroy(smem_trans_t handle, uint32_t flags);
int32_t smem_trans_register_mem(smem_trans_t handle, void *address, size_t capacity, uint32_t flags);
int32_t smem_trans_batch_register_mem(smem_trans_t handle, void *addresses[], size_t capacities[], uint32_t count,
                                      uint32_t flags);
int32_t smem_trans_deregister_mem(smem_trans_t handle, void *address);
int32_t smem_trans_write(smem_trans_t handle, const void *localAddr, const char *remoteUniqueId, void *remoteAddr,
                         size_t dataSize, uint32_t flags);
int32_t smem_trans_batch_write(smem_trans_t handle, const void *localAddrs[], const char *remoteUniqueId,
                               void *remoteAddrs[], size_t dataSizes[], uint32_t batchSize, uint32_t flags);
int32_t smem_trans_read(smem_trans_t handle, void *localAddr, const char *remoteUniqueId, const void *remoteAddr,
                        size_t dataSize, uint32_t flags);
int32_t smem_trans_batch_read(smem_trans_t handle, void *localAddrs[], const char *remoteUniqueId,
                              const void *remoteAddrs[], size_t dataSizes[], uint32_t batchSize, uint32_t flags);
int32_t smem_trans_read_submit(smem_trans_t handle, void *localAddr, const char *remoteUniqueId, const void *remoteAddr,
                               size_t dataSize, void *stream, uint32_t flags);
int32_t smem_trans_write_submit(smem_trans_t handle, const void *localAddr, const char *remoteUniqueId,
                                void *remoteAddr, size_t dataSize, void *stream, uint32_t flags);
int32_t smem_trans_batch_read_submit(smem_trans_t handle, void *localAddrs[], const char *remoteUniqueId,
                                     const void *remoteAddrs[], size_t dataSizes[], uint32_t batchSize,
                                     void *stream, uint32_t flags);
int32_t smem_trans_batch_write_submit(smem_trans_t handle, const void *localAddrs[],
                                      const char *remoteUniqueId, void *remoteAddrs[], size_t dataSizes[],
                                      uint32_t batchSize, void *stream, uint32_t flags);
int32_t smem_trans_batch_quant_write(smem_trans_t handle, smem_trans_quant_copy_param_t *params);
int32_t smem_trans_set_peer_down_callback(smem_trans_t handle, smem_trans_peer_down_callback_t callback,
                                          void *userData);

#ifdef __cplusplus
}
#endif
#endif
