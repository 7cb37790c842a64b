/*
 * Big Memory (BM): every member contributes an HBM and/or DRAM slice to one pool laid out as
 *   gva(memType, rank) = base(memType) + maxSize(memType) * rank
 * identical in all processes; copies take raw uint64 addresses inside or outside the pool.
 * ABI parity: src/smem/include/host/smem_bm.h of the reference (all 22 entry points).
 */
#ifndef MF_B200_SMEM_BM_H
#define MF_B200_SMEM_BM_H

#include "smem.h"
#include "smem_bm_def.h"

#ifdef __cplusplus
extern "C" {
#endif

int32_t smem_bm_config_init(smem_bm_config_t *config);
int32_t smem_bm_init(const char *storeURL, uint32_t worldSize, uint16_t deviceId, const smem_bm_config_t *config);
void smem_bm_uninit(uint32_t flags);
uint32_t smem_bm_get_rank_id(void);
smem_bm_t smem_bm_create(uint32_t id, uint32_t memberSize, smem_bm_data_op_type_t dataOpType, uint64_t localDRAMSize,
                         uint64_t localHBMSize, uint32_t flags);
smem_bm_t smem_bm_create2(uint32_t id, const smem_bm_create_option_t *option);
void smem_bm_destroy(smem_bm_t handle);
int32_t smem_bm_join(smem_bm_t handle, uint32_t flags);
int32_t smem_bm_leave(smem_bm_t handle, uint32_t flags);
int32_t smem_bm_extend_local_mem(smem_bm_t handle, smem_bm_mem_type_t memType, uint64_t size);
int32_t smem_bm_set_group_event_handler(smem_bm_t handle, smem_bm_group_event_cb cb, void *context);
uint64_t smem_bm_get_local_mem_size_by_mem_type(smem_bm_t handle, smem_bm_mem_type_t memType);
void *smem_bm_ptr_by_mem_type(smem_bm_t handle, smem_bm_mem_type_t memType, uint16_t peerRankId);
int32_t smem_bm_gva_to_va(smem_bm_t handle, void *gva, smem_bm_mem_type_t vaMemType, void **va);
int32_t smem_bm_copy(smem_bm_t handle, smem_copy_params_t *params, smem_bm_copy_type_t t, uint32_t flags);
int32_t smem_bm_copy_batch(smem_bm_t handle, smem_batch_copy_params_t *params, smem_bm_copy_type_t t, uint32_t flags);
int32_t smem_bm_copy_batch_partial_succeed(smem_bm_t handle, smem_batch_copy_params_t *params, smem_bm_copy_type_t t,
                                           uint32_t flags, smem_batch_copy_result *result);
int32_t smem_bm_wait(smem_bm_t handle);
int32_t smem_bm_register_user_mem(smem_bm_t handle, uint64_t addr, uint64_t size);
int32_t smem_bm_unregister_user_mem(smem_bm_t handle, uint64_t addr);
uint32_t smem_bm_get_rank_id_by_gva(smem_bm_t handle, void *gva);

#ifdef __cplusplus
}
#endif
#endif
