/*
 * hybm C API: init, entities, GVA reservation, slices, export/import/mmap and data copies.
 * ABI parity: src/hybm/include/hybm.h:28-65, hybm_big_mem.h:31-189, hybm_data_op.h:36-65 of the reference.
 */
#ifndef MF_B200_HYBM_H
#define MF_B200_HYBM_H

#include "hybm_def.h"

#ifdef __cplusplus
extern "C" {
#endif

int32_t hybm_init(uint16_t deviceId, uint64_t flags);
void hybm_uninit(void);
void hybm_set_extern_logger(void (*logger)(int level, const char *msg));
void hybm_set_extern_alarm(void (*alarm)(uint16_t code, const char *msg), void (*resume)(uint16_t code));
int32_t hybm_set_log_level(int level);
const char *hybm_get_error_string(int32_t errCode);

hybm_entity_t hybm_create_entity(uint16_t id, const hybm_options *options, uint32_t flags);
void hybm_destroy_entity(hybm_entity_t e, uint32_t flags);
int32_t hybm_reserve_mem_space(hybm_entity_t e, uint32_t flags);
int32_t hybm_unreserve_mem_space(hybm_entity_t e, uint32_t flags);
void *hybm_get_memory_ptr(hybm_entity_t e, hybm_mem_type mType);
hybm_mem_slice_t hybm_alloc_local_memory(hybm_entity_t e, hybm_mem_type mType, uint64_t size, uint32_t flags);
int32_t hybm_free_local_memory(hybm_entity_t e, hybm_mem_slice_t slice, uint32_t count, uint32_t flags);
void *hybm_get_slice_va(hybm_entity_t e, hybm_mem_slice_t slice);
hybm_mem_slice_t hybm_register_local_memory(hybm_entity_t e, const void *ptr, uint64_t size, uint32_t flags);
/* slice == NULL exports the entity itself */
int32_t hybm_export(hybm_entity_t e, hybm_mem_slice_t slice, uint32_t flags, hybm_exchange_info *exInfo);
int32_t hybm_import(hybm_entity_t e, const hybm_exchange_info allExInfo[], uint32_t count, void *addresses[],
                    uint32_t flags);
int32_t hybm_mmap(hybm_entity_t e, uint32_t flags);
void hybm_unmap(hybm_entity_t e, uint32_t flags);
#ifdef __cplusplus
int32_t hybm_entity_reach_types(hybm_entity_t e, uint32_t rank, hybm_data_op_type &reachTypes, uint32_t flags);
#endif
int32_t hybm_remove_imported(hybm_entity_t e, uint32_t rank, uint32_t flags);
int32_t hybm_set_extra_context(hybm_entity_t e, const void *context, uint32_t size);
int32_t hybm_gva_to_va(uint64_t gva, hybm_mem_type vaMemType, uint64_t *va);

int32_t hybm_data_copy(hybm_entity_t e, hybm_copy_params *params, hybm_data_copy_direction direction, void *stream,
                       uint32_t flags);
int32_t hybm_data_batch_copy(hybm_entity_t e, hybm_batch_copy_params *params, hybm_data_copy_direction direction,
                             void *stream, uint32_t flags);
int32_t hybm_wait(hybm_entity_t e);
int32_t hybm_data_quant_copy(hybm_entity_t e, hybm_quant_copy_params *params);

#ifdef __cplusplus
}
#endif
#endif
