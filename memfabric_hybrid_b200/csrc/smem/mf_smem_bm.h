// Big Memory entry: one pool instance of one process. Owns the dynamic group (join / update / leave /
// link-down driven by the EVENT record in the store), the memory entity and this rank's exported blobs.
// Parity: src/smem/csrc/smem_bm/smem_bm_entry.{h,cpp}:28-124,178-269,271-385,416-457,469-722,774-822,
// src/smem/csrc/smem_bm/smem_bm_entry_manager.cpp:46-155.
#pragma once
#include "../include/smem_bm.h"
#include "mf_smem_common.h"

namespace mf {
namespace smem {

struct BmGlobals {
    std::string storeUrl;
    uint32_t worldSize = 0;
    uint16_t deviceId = 0;
    smem_bm_config_t config{};
    store::StorePtr store;  // prefixed "BM_"
    uint32_t rank = 0;
    bool inited = false;
    bool hybmInited = false;
};

class BmEntry : public std::enable_shared_from_this<BmEntry> {
public:
    BmEntry(uint32_t id, const smem_bm_create_option_t &opt, const BmGlobals &g) : id_(id), opt_(opt), g_(g) {}
    ~BmEntry();
    int Initialize();
    int Join(uint32_t flags);
    int Leave(uint32_t flags);
    int ExtendLocal(smem_bm_mem_type_t t, uint64_t size);
    int SetEventHandler(smem_bm_group_event_cb cb, void *ctx);
    uint64_t LocalSize(smem_bm_mem_type_t t);
    void *PtrOf(smem_bm_mem_type_t t, uint16_t rank);
    int Copy(const smem_copy_params_t &p, smem_bm_copy_type_t t, uint32_t flags);
    int CopyBatch(const smem_batch_copy_params_t &p, smem_bm_copy_type_t t, uint32_t flags, int32_t *perItem);
    int Wait();
    int PrepareBatch(const smem_batch_copy_params_t &p, smem_bm_copy_type_t t, hybm::PreparedBatch &out);
    int RegisterUser(uint64_t addr, uint64_t size);
    int UnregisterUser(uint64_t addr);
    uint32_t RankOfGva(const void *gva);
    bool Joined() const { return group_ && group_->Joined(); }
    hybm::EntityPtr Entity() const { return entity_; }
    uint32_t Id() const { return id_; }

private:
    int CheckConsistency();
    int PublishBlobs();
    int ImportRank(uint32_t rank, uint64_t timeoutMs);
    int OnJoin(uint32_t rank);
    int OnUpdate(uint32_t rank);
    int OnLeave(uint32_t rank);
    int OnLinkDown(uint32_t rank);
    hybm_data_copy_direction DirectionFor(smem_bm_copy_type_t t, const void *src, const void *dst, uint64_t len);
    uint8_t PoolClass(const void *p, uint64_t len);
    void Fire(uint32_t rank, smem_bm_group_event_t ev);

    uint32_t id_;
    smem_bm_create_option_t opt_;
    BmGlobals g_;
    store::StorePtr store_;  // "BM_(<id>)_"
    group::GroupPtr group_;
    hybm::EntityPtr entity_;
    std::mutex mu_;
    std::vector<hybm_exchange_info> blobs_;  // entity + every local slice
    std::vector<hybm::MemSlice *> slices_;
    smem_bm_group_event_cb cb_ = nullptr;
    void *cbCtx_ = nullptr;
    std::set<uint32_t> imported_;
};
using BmEntryPtr = std::shared_ptr<BmEntry>;

}  // namespace smem
}  // namespace mf
