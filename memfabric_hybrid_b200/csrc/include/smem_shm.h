/*
 * Symmetric shared memory (SHM): a fixed-size group in which every rank owns one slice of equal
 * (1 GiB-aligned) stride inside a GVA range, meant to be addressed from kernels as
 *   peer(ptr, r) = ptr + (r - myRank) * symmetricSize
 * plus control-plane barrier / allgather helpers over the config store.
 * ABI parity: src/smem/include/host/smem_shm.h:28-222, smem_shm_def.h of the reference.
 */
#ifndef MF_B200_SMEM_SHM_H
#define MF_B200_SMEM_SHM_H

#include "smem.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef void *smem_shm_t;
#define SMEM_SHM_TIMEOUT_MAX      UINT32_MAX
#define SMEM_SHM_ATOMIC_NUM_LIMIT 1024U

typedef enum {
    SMEMS_DATA_OP_MTE = 1U << 0,  /* load/store from SM kernels */
    SMEMS_DATA_OP_SDMA = 1U << 1, /* copy engines */
    SMEMS_DATA_OP_RDMA = 1U << 2,
} smem_shm_data_op_type;

typedef struct {
    uint32_t shmInitTimeout;          /* seconds, default 120 */
    uint32_t shmCreateTimeout;        /* seconds, default 120 */
    uint32_t controlOperationTimeout; /* seconds, default 120 */
    bool startConfigStoreServer;      /* default true (rank 0 hosts it) */
    uint32_t flags;
} smem_shm_config_t;

int32_t smem_shm_config_init(smem_shm_config_t *config);
int32_t smem_shm_init(const char *configStoreIpPort, uint32_t worldSize, uint32_t rankId, uint16_t deviceId,
                      smem_shm_config_t *config);
void smem_shm_uninit(uint32_t flags);
uint32_t smem_shm_query_support_data_operation(void);
smem_shm_t smem_shm_create(uint32_t id, uint32_t rankSize, uint32_t rankId, uint64_t localSize,
                           smem_shm_data_op_type dataOpType, uint32_t flags, void **gva);
uint64_t smem_shm_get_symmetric_size(smem_shm_t handle);
int32_t smem_shm_destroy(smem_shm_t handle, uint32_t flags);
int32_t smem_shm_set_extra_context(smem_shm_t handle, const void *context, uint32_t size);
uint32_t smem_shm_get_global_rank(smem_shm_t handle);
uint32_t smem_shm_get_global_rank_size(smem_shm_t handle);
int32_t smem_shm_control_barrier(smem_shm_t handle);
int32_t smem_shm_control_allgather(smem_shm_t handle, const char *sendBuf, uint32_t sendSize, char *recvBuf,
                                   uint32_t recvSize);
int32_t smem_shm_subgroup_barrier(smem_shm_t handle, const char *key, uint32_t rankSize, uint32_t rankId);
int32_t smem_shm_subgroup_allgather(smem_shm_t handle, const char *key, uint32_t rankSize, uint32_t rankId,
                                    const char *sendBuf, uint32_t sendSize, char *recvBuf, uint32_t recvSize);
int32_t smem_shm_topology_can_reach(smem_shm_t handle, uint32_t remoteRank, uint32_t *reachInfo);
int32_t smem_shm_atomic_alloc_value(smem_shm_t handle, uint32_t limit, int32_t *value);
int32_t smem_shm_atomic_release_value(smem_shm_t handle, int32_t value);
int32_t smem_shm_register_exit(smem_shm_t handle, void (*exit)(int));
void smem_shm_global_exit(smem_shm_t handle, int status);
/* Fills the block a kernel takes by value to use the device API (smem_shm_device.cuh: smem_shm_device_ctx_t,
 * 40 bytes). The reference publishes the same facts in a meta region at a fixed address instead. */
int32_t smem_shm_get_device_context(smem_shm_t handle, void *ctx, uint32_t ctxSize);

#ifdef __cplusplus
}
#endif
#endif
