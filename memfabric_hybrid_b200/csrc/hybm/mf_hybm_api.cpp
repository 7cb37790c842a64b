// C facade of the memory layer (hybm_* entry points). Handles are raw pointers to heap-held
// shared_ptrs so that a handle stays valid until its destroy call.
// Parity: src/hybm/csrc/hybm_entry.cpp:51-189, src/hybm/csrc/hybm_big_mem_entry.cpp, hybm_data_op_entry.cpp:22-140.
#include "../include/hybm.h"
#include "mf_entity.h"

using namespace mf;
using namespace mf::hybm;

namespace {
int ToBm(int rc)
{
    switch (rc) {
        case OK: return BM_OK;
        case ERR_INVALID_PARAM: return BM_INVALID_PARAM;
        case ERR_MALLOC: return BM_MALLOC_FAILED;
        case ERR_TIMEOUT: return BM_TIMEOUT;
        case ERR_NOT_INIT: return BM_NOT_INITIALIZED;
        case ERR_NOT_CONNECTED: return BM_NOT_CONNECTED;
        default: return rc > -100 ? rc : BM_ERROR;
    }
}
Entity *E(hybm_entity_t e) { return e == nullptr ? nullptr : static_cast<EntityPtr *>(e)->get(); }
}  // namespace

extern "C" {

int32_t hybm_init(uint16_t deviceId, uint64_t flags) { return ToBm(HybmInit(deviceId, flags)); }
void hybm_uninit(void) { HybmUninit(); }
void hybm_set_extern_logger(void (*logger)(int level, const char *msg)) { Logger::Get().SetSink(logger); }
void hybm_set_extern_alarm(void (*alarm)(uint16_t code, const char *msg), void (*resume)(uint16_t code))
{
    Logger::Get().SetAlarm(alarm, resume);
}
int32_t hybm_set_log_level(int level)
{
    if (level < LOG_DEBUG || level > LOG_OFF) return BM_INVALID_PARAM;
    Logger::Get().SetLevel(level);
    return BM_OK;
}
const char *hybm_get_error_string(int32_t errCode) { return ErrorString(errCode); }

hybm_entity_t hybm_create_entity(uint16_t id, const hybm_options *options, uint32_t)
{
    if (options == nullptr) return nullptr;
    auto e = Entity::Create(id, *options);
    if (!e) return nullptr;
    return new EntityPtr(e);
}

void hybm_destroy_entity(hybm_entity_t e, uint32_t)
{
    if (e != nullptr) delete static_cast<EntityPtr *>(e);
}

int32_t hybm_reserve_mem_space(hybm_entity_t e, uint32_t flags)
{
    return E(e) ? ToBm(E(e)->ReserveMemSpace(flags)) : BM_INVALID_PARAM;  // flags carries the attempt number
}
int32_t hybm_unreserve_mem_space(hybm_entity_t e, uint32_t) { return E(e) ? ToBm(E(e)->UnreserveMemSpace()) : BM_INVALID_PARAM; }
void *hybm_get_memory_ptr(hybm_entity_t e, hybm_mem_type mType) { return E(e) ? E(e)->MemoryPtr(mType) : nullptr; }

hybm_mem_slice_t hybm_alloc_local_memory(hybm_entity_t e, hybm_mem_type mType, uint64_t size, uint32_t flags)
{
    MemSlice *s = nullptr;
    if (E(e) == nullptr || E(e)->AllocLocal(mType, size, flags, &s) != OK) return nullptr;
    return s;
}

int32_t hybm_free_local_memory(hybm_entity_t e, hybm_mem_slice_t slice, uint32_t, uint32_t)
{
    return E(e) ? ToBm(E(e)->FreeLocal(static_cast<MemSlice *>(slice))) : BM_INVALID_PARAM;
}

void *hybm_get_slice_va(hybm_entity_t e, hybm_mem_slice_t slice)
{
    auto *s = static_cast<MemSlice *>(slice);
    if (E(e) == nullptr || s == nullptr || !s->Valid()) return nullptr;
    return reinterpret_cast<void *>(s->gva);
}

hybm_mem_slice_t hybm_register_local_memory(hybm_entity_t e, const void *ptr, uint64_t size, uint32_t flags)
{
    MemSlice *s = nullptr;
    if (E(e) == nullptr || E(e)->RegisterLocal(ptr, size, flags, &s) != OK) return nullptr;
    return s;
}

int32_t hybm_export(hybm_entity_t e, hybm_mem_slice_t slice, uint32_t, hybm_exchange_info *exInfo)
{
    return E(e) ? ToBm(E(e)->Export(static_cast<MemSlice *>(slice), exInfo)) : BM_INVALID_PARAM;
}

int32_t hybm_import(hybm_entity_t e, const hybm_exchange_info allExInfo[], uint32_t count, void *addresses[], uint32_t)
{
    if (E(e) == nullptr || allExInfo == nullptr) return BM_INVALID_PARAM;
    return ToBm(E(e)->Import(allExInfo, count, addresses));
}

int32_t hybm_mmap(hybm_entity_t e, uint32_t) { return E(e) ? ToBm(E(e)->Mmap()) : BM_INVALID_PARAM; }
void hybm_unmap(hybm_entity_t e, uint32_t)
{
    if (E(e)) E(e)->Unmap();
}

int32_t hybm_entity_reach_types(hybm_entity_t e, uint32_t rank, hybm_data_op_type &reachTypes, uint32_t)
{
    if (E(e) == nullptr) return BM_INVALID_PARAM;
    uint32_t t = 0;
    int rc = E(e)->ReachTypes(rank, t);
    reachTypes = (hybm_data_op_type)t;
    return ToBm(rc);
}

int32_t hybm_remove_imported(hybm_entity_t e, uint32_t rank, uint32_t) { return E(e) ? ToBm(E(e)->RemoveImported(rank)) : BM_INVALID_PARAM; }

int32_t hybm_set_extra_context(hybm_entity_t e, const void *context, uint32_t size)
{
    return E(e) ? ToBm(E(e)->SetExtraContext(context, size)) : BM_INVALID_PARAM;
}

int32_t hybm_gva_to_va(uint64_t gva, hybm_mem_type, uint64_t *va)
{
    // The pool is mapped at its GVA in every process, so the translation is the identity for any
    // address inside a reserved window.
    if (va == nullptr) return BM_INVALID_PARAM;
    ReservedRange r;
    uint32_t rank = 0;
    if (!VaManager::Get().Locate(gva, r, rank)) return BM_INVALID_PARAM;
    // ... except in a window of 56-bit addresses, whose slots are mapped in a compact window of this process
    *va = r.localSlot == 0 ? gva : r.localBase + (uint64_t)rank * r.localSlot + (gva - r.base - (uint64_t)rank * r.slot);
    if (r.localSlot != 0 && gva - r.base - (uint64_t)rank * r.slot >= r.localSlot) return BM_INVALID_PARAM;
    return BM_OK;
}

int32_t hybm_data_copy(hybm_entity_t e, hybm_copy_params *params, hybm_data_copy_direction direction, void *stream,
                       uint32_t flags)
{
    if (E(e) == nullptr || params == nullptr) return BM_INVALID_PARAM;
    return ToBm(E(e)->CopyData(*params, direction, stream, flags));
}

int32_t hybm_data_batch_copy(hybm_entity_t e, hybm_batch_copy_params *params, hybm_data_copy_direction direction,
                             void *stream, uint32_t flags)
{
    if (E(e) == nullptr || params == nullptr) return BM_INVALID_PARAM;
    return ToBm(E(e)->BatchCopyData(*params, direction, stream, flags));
}

int32_t hybm_wait(hybm_entity_t e) { return E(e) ? ToBm(E(e)->Wait()) : BM_INVALID_PARAM; }

int32_t hybm_data_quant_copy(hybm_entity_t e, hybm_quant_copy_params *params)
{
    if (E(e) == nullptr || params == nullptr) return BM_INVALID_PARAM;
    return ToBm(E(e)->QuantCopy(*params, (params->flags & HYBM_QUANT_FP8_E4M3) ? 1 : 0));
}

}  // extern "C"
