#include "../util/mf_trace.h"
#include "mf_smem_bm.h"

namespace mf {
namespace smem {

using namespace hybm;

namespace {
#pragma pack(push, 1)
struct ConsistencyRecord {
    uint64_t maxDram;
    uint64_t maxHbm;
    uint8_t gva56;
};
#pragma pack(pop)

uint32_t ToHybmOps(uint32_t smemOps)
{
    uint32_t o = 0;
    if (smemOps & SMEMB_DATA_OP_SDMA) o |= HYBM_DOP_TYPE_SDMA | HYBM_DOP_TYPE_MTE;
    if (smemOps & SMEMB_DATA_OP_HOST_RDMA) o |= HYBM_DOP_TYPE_HOST_RDMA;
    if (smemOps & SMEMB_DATA_OP_HOST_TCP) o |= HYBM_DOP_TYPE_HOST_TCP;
    if (smemOps & SMEMB_DATA_OP_DEVICE_RDMA) o |= HYBM_DOP_TYPE_DEVICE_RDMA;
    if (smemOps & SMEMB_DATA_OP_HOST_URMA) o |= HYBM_DOP_TYPE_HOST_URMA;
    if (smemOps & SMEMB_DATA_OP_HOST_SHM) o |= HYBM_DOP_TYPE_HOST_SHM;
    if (smemOps & SMEMB_DATA_OP_DEVICE_URMA) o |= HYBM_DOP_TYPE_DEVICE_URMA;
    return o;
}
}  // namespace

BmEntry::~BmEntry()
{
    if (group_) group_->StopListen();
    if (entity_) entity_->Wait();
    group_.reset();
    entity_.reset();
}

int BmEntry::CheckConsistency()
{
    // Every member must describe the same layout: the first one records it, the others compare.
    ConsistencyRecord mine{opt_.maxDramSize, opt_.maxHbmSize, (uint8_t)(opt_.enable56BitsGva ? 1 : 0)};
    std::string want(reinterpret_cast<const char *>(&mine), sizeof(mine)), existing;
    int rc = store_->Cas("CONFIG", "", want, existing);
    if (rc == OK) return OK;
    if (rc != ERR_IN_USE) return rc;
    if (existing != want) {
        ConsistencyRecord other{};
        if (existing.size() == sizeof(other)) memcpy(&other, existing.data(), sizeof(other));
        return MF_FAIL(ERR_INVALID_PARAM,
                       "pool %u: this rank asks for maxDRAM %lu / maxHBM %lu but the pool was created with %lu / %lu", id_,
                       (unsigned long)mine.maxDram, (unsigned long)mine.maxHbm, (unsigned long)other.maxDram,
                       (unsigned long)other.maxHbm);
    }
    return OK;
}

int BmEntry::Initialize()
{
    MF_TRACE_BEGIN(TP_BM_CREATE);
    store_ = store::StoreFactory::Prefixed(g_.store, "(" + std::to_string(id_) + ")_");
    int rc = CheckConsistency();
    if (rc == OK) {
        group::GroupOption go;
        go.rankSize = g_.worldSize;
        go.rank = g_.rank;
        go.timeoutMs = 1000ULL * g_.config.controlOperationTimeout;
        go.dynamic = true;
        std::weak_ptr<BmEntry> weak = weak_from_this();
        go.joinCb = [weak](uint32_t r) { auto s = weak.lock(); return s ? s->OnJoin(r) : OK; };
        go.updateCb = [weak](uint32_t r) { auto s = weak.lock(); return s ? s->OnUpdate(r) : OK; };
        go.leaveCb = [weak](uint32_t r) { auto s = weak.lock(); return s ? s->OnLeave(r) : OK; };
        go.linkDownCb = [weak](uint32_t r) { auto s = weak.lock(); return s ? s->OnLinkDown(r) : OK; };
        group_ = group::GroupEngine::Create(store_, go);
        if (!group_) rc = ERR_INVALID_PARAM;
        // A store that restarted (a new leader after the old one died) has lost this rank's exchange record; members
        // have imported it long ago, but a rank that joins, or returns, later reads it from the store.
        store_->RegisterReconnectHandler([weak]() -> int {
            auto s = weak.lock();
            if (!s || !s->group_ || !s->Joined()) return OK;
            std::string mine;
            {
                std::lock_guard<std::mutex> g(s->mu_);
                mine = PackInfos(s->blobs_);
            }
            return s->store_->Set("BMEX_" + std::to_string(s->g_.rank), mine);
        });
    }
    if (rc == OK) rc = group_->StartListen();
    if (rc == OK) {
        hybm_options ho{};
        ho.bmType = HYBM_TYPE_HOST_INITIATE;
        uint32_t mt = 0;
        if (opt_.maxHbmSize != 0) mt |= HYBM_MEM_TYPE_DEVICE;
        if (opt_.maxDramSize != 0) mt |= HYBM_MEM_TYPE_HOST;
        ho.memType = (hybm_mem_type)mt;
        ho.bmDataOpType = (hybm_data_op_type)ToHybmOps(opt_.dataOpType);
        ho.rankCount = g_.worldSize;
        ho.rankId = g_.rank;
        ho.devId = g_.deviceId;
        ho.maxHBMSize = opt_.maxHbmSize;
        ho.maxDRAMSize = opt_.maxDramSize;
        ho.scene = HYBM_SCENE_DEFAULT;
        ho.enable56BitsGva = opt_.enable56BitsGva;
        ho.role = HYBM_ROLE_PEER;
        ho.flags = opt_.flags;
        ho.dramShmFd = opt_.dramShmFd;
        snprintf(ho.tag, sizeof(ho.tag), "%s", opt_.tag);
        snprintf(ho.tagOpInfo, sizeof(ho.tagOpInfo), "%s", opt_.tagOpInfo);
        entity_ = Entity::Create((uint16_t)id_, ho);
        if (!entity_) rc = LastError::Code() != 0 ? LastError::Code() : (int)ERR;
    }
    if (rc == OK) {
        // All ranks try the same sequence of windows; a peer that ended on another window is refused at import.
        for (uint32_t attempt = 0; attempt < kReserveAttempts; attempt++) {
            rc = entity_->ReserveMemSpace(attempt);
            if (rc == OK) break;
            MF_WARN("pool %u: GVA window attempt %u failed (%d)", id_, attempt, rc);
        }
    }
    if (rc == OK && opt_.localHBMSize != 0) {
        MemSlice *s = nullptr;
        rc = entity_->AllocLocal(HYBM_MEM_TYPE_DEVICE, opt_.localHBMSize, 0, &s);
        if (rc == OK) slices_.push_back(s);
    }
    if (rc == OK && opt_.localDRAMSize != 0) {
        MemSlice *s = nullptr;
        rc = entity_->AllocLocal(HYBM_MEM_TYPE_HOST, opt_.localDRAMSize, 0, &s);
        if (rc == OK) slices_.push_back(s);
    }
    if (rc == OK) rc = PublishBlobs();
    MF_TRACE_END(TP_BM_CREATE, rc);
    return rc;
}

int BmEntry::PublishBlobs()
{
    std::vector<hybm_exchange_info> v(1 + slices_.size());
    int rc = entity_->Export(nullptr, &v[0]);
    for (size_t i = 0; i < slices_.size() && rc == OK; i++) rc = entity_->Export(slices_[i], &v[i + 1]);
    if (rc != OK) return rc;
    std::lock_guard<std::mutex> g(mu_);
    blobs_.swap(v);
    return OK;
}

int BmEntry::ImportRank(uint32_t rank, uint64_t timeoutMs)
{
    std::string blob;
    int rc = store_->Get("BMEX_" + std::to_string(rank), blob, (int64_t)timeoutMs);
    if (rc != OK) return MF_FAIL(rc, "pool %u: exchange record of rank %u not available (%d)", id_, rank, rc);
    std::vector<hybm_exchange_info> infos;
    if (!UnpackInfos(blob, infos)) return MF_FAIL(ERR, "pool %u: exchange record of rank %u is malformed", id_, rank);
    rc = entity_->Import(infos.data(), (uint32_t)infos.size(), nullptr);
    if (rc == OK) {
        std::lock_guard<std::mutex> g(mu_);
        imported_.insert(rank);
    }
    return rc;
}

void BmEntry::Fire(uint32_t rank, smem_bm_group_event_t ev)
{
    smem_bm_group_event_cb cb;
    void *ctx;
    {
        std::lock_guard<std::mutex> g(mu_);
        cb = cb_;
        ctx = cbCtx_;
    }
    if (cb != nullptr) cb(this, rank, ev, ctx);
}

int BmEntry::OnJoin(uint32_t rank)
{
    uint64_t to = 1000ULL * g_.config.controlOperationTimeout;
    int rc = OK;
    if (rank == g_.rank) {
        std::string mine;
        {
            std::lock_guard<std::mutex> g(mu_);
            mine = PackInfos(blobs_);
        }
        rc = store_->Set("BMEX_" + std::to_string(rank), mine);
        group::GroupInfo info = group_->Info();
        for (uint32_t r = 0; r < g_.worldSize && rc == OK; r++)
            if (r != g_.rank && info.Has(r)) rc = ImportRank(r, to);
    } else {
        rc = ImportRank(rank, to);
    }
    // Everybody reports, so that nobody maps a half-built pool; then map, then meet again.
    int all = group_->EventGatherResult(rc);
    if (all != OK) return rc != OK ? rc : all;
    int32_t mrc = entity_->Mmap();
    all = group_->EventGatherResult(mrc);
    if (all != OK) return mrc != OK ? mrc : all;
    if (rank != g_.rank) Fire(rank, SMEM_GROUP_EVENT_JOIN);
    return OK;
}

int BmEntry::OnUpdate(uint32_t rank)
{
    uint64_t to = 1000ULL * g_.config.controlOperationTimeout;
    int rc = OK;
    if (rank == g_.rank) {
        std::string mine;
        {
            std::lock_guard<std::mutex> g(mu_);
            mine = PackInfos(blobs_);
        }
        rc = store_->Set("BMEX_" + std::to_string(rank), mine);
    }
    int all = group_->EventGatherResult(rc);  // the record is in the store once this returns
    if (all != OK) return rc != OK ? rc : all;
    if (rank != g_.rank) {
        rc = ImportRank(rank, to);
        if (rc == OK) rc = entity_->Mmap();
    }
    all = group_->EventGatherResult(rc);
    return rc != OK ? rc : all;
}

int BmEntry::OnLeave(uint32_t rank)
{
    if (rank != g_.rank) {
        entity_->RemoveImported(rank);
        {
            std::lock_guard<std::mutex> g(mu_);
            imported_.erase(rank);
        }
    }
    int rc = group_->EventBarrier();  // the leaver frees nothing before every member unmapped it
    if (rank == g_.rank) {
        entity_->Wait();
        entity_->Unmap();
        store_->Remove("BMEX_" + std::to_string(rank), true);
        std::lock_guard<std::mutex> g(mu_);
        imported_.clear();
    } else {
        Fire(rank, SMEM_GROUP_EVENT_LEAVE);
    }
    return rc;
}

int BmEntry::OnLinkDown(uint32_t rank)
{
    MF_WARN("pool %u: rank %u lost its link, dropping its memory", id_, rank);
    entity_->RemoveImported(rank);
    {
        std::lock_guard<std::mutex> g(mu_);
        imported_.erase(rank);
    }
    Fire(rank, SMEM_GROUP_EVENT_LEAVE);
    return OK;
}

int BmEntry::Join(uint32_t)
{
    MF_TRACE_BEGIN(TP_BM_JOIN);
    int rc = group_->Join();
    MF_TRACE_END(TP_BM_JOIN, rc);
    return rc;
}

int BmEntry::Leave(uint32_t) { return group_->Leave(); }

int BmEntry::ExtendLocal(smem_bm_mem_type_t t, uint64_t size)
{
    if (!Joined()) return MF_FAIL(ERR_NOT_STARTED, "pool %u: extend_local_mem before join", id_);
    hybm_mem_type mt = (t == SMEM_MEM_TYPE_HOST || t == SMEM_MEM_TYPE_LOCAL_HOST) ? HYBM_MEM_TYPE_HOST : HYBM_MEM_TYPE_DEVICE;
    MemSlice *s = nullptr;
    int rc = entity_->AllocLocal(mt, size, 0, &s);
    if (rc != OK) return rc;
    slices_.push_back(s);
    rc = PublishBlobs();
    if (rc == OK) rc = group_->Update();
    return rc;
}

int BmEntry::SetEventHandler(smem_bm_group_event_cb cb, void *ctx)
{
    std::lock_guard<std::mutex> g(mu_);
    cb_ = cb;
    cbCtx_ = ctx;
    return OK;
}

uint64_t BmEntry::LocalSize(smem_bm_mem_type_t t)
{
    bool host = t == SMEM_MEM_TYPE_HOST || t == SMEM_MEM_TYPE_LOCAL_HOST;
    return entity_->LocalBytes(host ? HYBM_MEM_TYPE_HOST : HYBM_MEM_TYPE_DEVICE);
}

void *BmEntry::PtrOf(smem_bm_mem_type_t t, uint16_t rank)
{
    if (rank >= g_.worldSize) {
        MF_FAIL(ERR_INVALID_PARAM, "peer rank %u outside world %u", rank, g_.worldSize);
        return nullptr;
    }
    hybm_mem_type mt;
    if (t == SMEM_MEM_TYPE_DEVICE) mt = HYBM_MEM_TYPE_DEVICE;
    else if (t == SMEM_MEM_TYPE_HOST) mt = HYBM_MEM_TYPE_HOST;
    else {
        MF_FAIL(ERR_INVALID_PARAM, "memory type %d has no pool address", (int)t);
        return nullptr;
    }
    auto seg = entity_->SegmentOf(mt);
    if (!seg || seg->Base() == 0) {
        MF_FAIL(ERR_NOT_EXIST, "pool %u has no %s space", id_, mt == HYBM_MEM_TYPE_HOST ? "DRAM" : "HBM");
        return nullptr;
    }
    return reinterpret_cast<void *>(seg->PubBase() + seg->PubSlot() * rank);
}

uint32_t BmEntry::RankOfGva(const void *gva)
{
    uint64_t a = reinterpret_cast<uint64_t>(gva);
    for (auto mt : {HYBM_MEM_TYPE_DEVICE, HYBM_MEM_TYPE_HOST}) {
        auto seg = entity_->SegmentOf(mt);
        if (!seg || seg->Base() == 0 || a < seg->PubBase()) continue;
        uint64_t r = (a - seg->PubBase()) / seg->PubSlot();
        if (r < g_.worldSize) return (uint32_t)r;
    }
    return UINT32_MAX;
}

uint8_t BmEntry::PoolClass(const void *p, uint64_t len)
{
    uint64_t a = reinterpret_cast<uint64_t>(p);
    auto in = [&](hybm_mem_type mt) {
        auto seg = entity_->SegmentOf(mt);
        return seg && seg->Base() != 0 && a >= seg->PubBase() && a + len <= seg->PubBase() + seg->PubSlot() * g_.worldSize;
    };
    if (in(HYBM_MEM_TYPE_DEVICE)) return AC_GD;
    if (in(HYBM_MEM_TYPE_HOST)) return AC_GH;
    return AC_NONE;
}

hybm_data_copy_direction BmEntry::DirectionFor(smem_bm_copy_type_t t, const void *src, const void *dst, uint64_t len)
{
    uint8_t s = PoolClass(src, len), d = PoolClass(dst, len);
    switch (t) {
        case SMEMB_COPY_L2G:
        case SMEMB_COPY_L2GH: s = AC_LD; break;
        case SMEMB_COPY_G2L:
        case SMEMB_COPY_GH2L: d = AC_LD; break;
        case SMEMB_COPY_G2H:
        case SMEMB_COPY_GH2H: d = AC_LH; break;
        case SMEMB_COPY_H2G:
        case SMEMB_COPY_H2GH: s = AC_LH; break;
        case SMEMB_COPY_AUTO: return HYBM_DATA_COPY_DIRECTION_AUTO;
        default: break;
    }
    return VaManager::DirectionOf(s, d);
}

int BmEntry::Copy(const smem_copy_params_t &p, smem_bm_copy_type_t t, uint32_t flags)
{
    if (!Joined()) return MF_FAIL(ERR_NOT_STARTED, "pool %u: copy before join", id_);
    MF_TRACE_BEGIN(TP_BM_COPY);
    hybm_data_copy_direction dir = DirectionFor(t, p.src, p.dest, p.dataSize);
    int rc;
    if (dir == HYBM_DATA_COPY_DIRECTION_BUTT) {
        rc = MF_FAIL(ERR_INVALID_PARAM, "copy type %d does not fit addresses %p -> %p", (int)t, p.src, p.dest);
    } else {
        hybm_copy_params hp{const_cast<void *>(p.src), p.dest, p.dataSize};
        void *stream = (flags & SMEM_BM_FLAG_USE_EXTERNAL_STREAM) ? p.stream : nullptr;
        rc = entity_->CopyData(hp, dir, stream, flags);
    }
    MF_TRACE_END(TP_BM_COPY, rc);
    return rc;
}

int BmEntry::CopyBatch(const smem_batch_copy_params_t &p, smem_bm_copy_type_t t, uint32_t flags, int32_t *perItem)
{
    if (!Joined()) return MF_FAIL(ERR_NOT_STARTED, "pool %u: copy before join", id_);
    MF_TRACE_BEGIN(TP_BM_COPY_BATCH);
    // The first item fixes the direction of the whole batch.
    hybm_data_copy_direction dir = DirectionFor(t, p.sources[0], p.destinations[0], p.dataSizes[0]);
    int rc;
    if (dir == HYBM_DATA_COPY_DIRECTION_BUTT) {
        rc = MF_FAIL(ERR_INVALID_PARAM, "copy type %d does not fit addresses %p -> %p", (int)t, p.sources[0], p.destinations[0]);
    } else {
        hybm_batch_copy_params hp{p.sources, p.destinations, p.dataSizes, p.batchSize};
        void *stream = (flags & SMEM_BM_FLAG_USE_EXTERNAL_STREAM) ? p.stream : nullptr;
        rc = entity_->BatchCopyData(hp, dir, stream, flags, perItem);
    }
    MF_TRACE_END(TP_BM_COPY_BATCH, rc);
    return rc;
}

int BmEntry::Wait() { return entity_->Wait(); }

int BmEntry::PrepareBatch(const smem_batch_copy_params_t &p, smem_bm_copy_type_t t, hybm::PreparedBatch &out)
{
    if (!Joined()) return MF_FAIL(ERR_NOT_STARTED, "pool %u: prepared batch before join", id_);
    hybm_data_copy_direction dir = DirectionFor(t, p.sources[0], p.destinations[0], p.dataSizes[0]);
    if (dir == HYBM_DATA_COPY_DIRECTION_BUTT)
        return MF_FAIL(ERR_INVALID_PARAM, "copy type %d does not fit addresses %p -> %p", (int)t, p.sources[0], p.destinations[0]);
    hybm_batch_copy_params hp{p.sources, p.destinations, p.dataSizes, p.batchSize};
    return entity_->PrepareBatch(hp, dir, out);
}

int BmEntry::RegisterUser(uint64_t addr, uint64_t size)
{
    MemSlice *s = nullptr;
    return entity_->RegisterLocal(reinterpret_cast<void *>(addr), size, 0, &s);
}

int BmEntry::UnregisterUser(uint64_t addr) { return entity_->UnregisterLocal(addr); }

}  // namespace smem
}  // namespace mf
