// smem_shm_*: symmetric shared memory for kernels. A static group of `rankSize` ranks; every rank owns
// one slice of equal stride (1 GiB-aligned) in one GVA range mapped by all, so device code addresses a
// peer with a single multiply-add. Creation is a list of steps with rollback:
//   entity -> reserve (windows tried in lockstep, agreed by allgather) -> alloc slice -> exchange slices
//   (allgather + import + barrier) -> exchange entities -> mmap -> barrier
// plus control-plane barrier/allgather (world and sub-group), a unique-number allocator and a global
// exit broadcast, all on the config store.
// Parity: src/smem/csrc/smem_shm/smem_shm.cpp:23-80, smem_shm_entry.cpp:23-38,83-119,151-281,
// src/smem/include/host/smem_shm.h:28-222.
#include <unistd.h>

#include "../include/smem_shm.h"
#include "../include/smem_shm_device.cuh"
#include "../util/mf_trace.h"
#include "mf_smem_common.h"

using namespace mf;
using namespace mf::smem;
using namespace mf::hybm;

namespace {

struct ShmGlobals {
    std::string url;
    uint32_t worldSize = 0, rank = 0;
    uint16_t deviceId = 0;
    smem_shm_config_t config{};
    store::StorePtr store;  // prefixed "SHM_"
    bool inited = false;
};

class ShmEntry {
public:
    ShmEntry(uint32_t id, uint32_t rankSize, uint32_t rank, uint64_t localSize, uint32_t ops, uint32_t flags,
             const ShmGlobals &g)
        : id_(id), rankSize_(rankSize), rank_(rank), localSize_(localSize), ops_(ops), flags_(flags), g_(g)
    {
    }
    ~ShmEntry()
    {
        TeardownMulticast();
        if (group_) group_->StopListen();
        entity_.reset();
    }

    // NVLink multicast ("NVLS") view of the object: ONE multicast object of the slice size to which every
    // rank binds its own slice at offset 0, mapped at mcBase_. A multimem load-reduce at mcBase_ + off sums
    // (in the switch) the values at offset off of ALL ranks' slices; a multimem store writes all of them.
    // Opt-in (MF_SHM_MULTICAST=1): a process that dies while its memory is bound to a multicast object
    // disturbs its peers' NVLink traffic, so jobs that may lose ranks should stay on plain peer mappings.
    // Order: create (rank 0) -> hand out the handle -> every rank adds its device -> barrier -> bind -> barrier
    // -> map. A rank that cannot take part says so in the all-gather and everybody skips the set-up.
    int SetupMulticast()
    {
        mcBase_ = 0;
        auto *dev = CurrentBackend();
        const bool want = EnvInt("MF_SHM_MULTICAST", "ZBAL_NVLS", 0, 0, 1) != 0;
        int32_t can = (want && rankSize_ > 1 && dev != nullptr && dev->Caps().multicast) ? 1 : 0;
        uint64_t gran = 0;
        if (can && dev->McGranularity(localSize_, rankSize_, &gran) != OK) can = 0;
        // the bound range must be backed by this rank's own allocation: sizes that are not a multiple of the
        // multicast granularity (2 MiB on current parts) stay on peer mappings
        if (can && (gran == 0 || localSize_ % gran != 0)) can = 0;
        const uint64_t size = can ? localSize_ : 0;
        struct Blob {
            int32_t can;
            int32_t pid;
            uint64_t token;
            char name[112];
        } mine{}, zero{};
        mine.can = can;
        PhysHandle mc = 0;
        uint64_t token = 0;
        if (can && rank_ == 0) {
            int fd = -1;
            if (dev->McCreate(size, rankSize_, &mc) != OK || dev->ExportFd(mc, &fd) != OK) {
                mine.can = 0;
                if (mc) dev->ReleasePhys(mc);
                mc = 0;
            } else {
                token = FdChannel::Get().Publish(fd);
                mine.token = token;
                mine.pid = (int32_t)getpid();
                snprintf(mine.name, sizeof(mine.name), "%s", FdChannel::Get().Name().c_str());
            }
        }
        std::vector<Blob> all(rankSize_, zero);
        int rc = group_->AllGather(reinterpret_cast<const char *>(&mine), sizeof(mine), reinterpret_cast<char *>(all.data()),
                                   (uint32_t)(all.size() * sizeof(Blob)));
        bool everyone = rc == OK;
        for (auto &b : all) everyone = everyone && b.can == 1;
        int32_t step = everyone ? OK : ERR;
        if (everyone && rank_ != 0) {
            int fd = -1;
            step = FdChannel::Fetch(all[0].name, all[0].token, &fd);
            if (step == OK) step = dev->ImportFd(fd, size, &mc);
        }
        if (step == OK && everyone) step = dev->McAddDevice(mc);
        step = GatherOk(step);  // doubles as the barrier "every device was added"
        if (step == OK && everyone) {
            const uint64_t local = reinterpret_cast<uint64_t>(gva_) + (uint64_t)rank_ * symmetric_;
            step = dev->McBindAddr(mc, 0, local, size);
            if (step == OK) mcBound_ = true;
        }
        step = GatherOk(step);
        if (step == OK && everyone) {
            uint64_t va = 0;
            step = dev->Reserve(0, size, &va);
            if (step == OK) {
                step = dev->Map(va, size, mc);
                if (step != OK) dev->ReleaseVa(va, size);
                else mcBase_ = va;
            }
        }
        step = GatherOk(step);
        if (token) FdChannel::Get().Withdraw(token);
        mcHandle_ = mc;
        mcSize_ = size;
        if (step != OK || !everyone) {
            TeardownMulticast();
            if (want) MF_WARN("shm %u: NVLink multicast not set up (%s); collectives use peer loads and stores", id_,
                              everyone ? "a step failed" : "not supported or refused by a rank");
            return OK;  // optional feature: the object works without it
        }
        MF_INFO("shm %u: NVLink multicast view of %lu MiB per rank at %#lx", id_, (unsigned long)(size >> 20), (unsigned long)mcBase_);
        return OK;
    }

    void TeardownMulticast()
    {
        auto *dev = CurrentBackend();
        if (dev == nullptr || mcHandle_ == 0) return;
        dev->StreamSync(nullptr);
        if (mcBase_) {
            dev->Unmap(mcBase_, mcSize_);
            dev->ReleaseVa(mcBase_, mcSize_);
            mcBase_ = 0;
        }
        if (mcBound_) {
            dev->McUnbind(mcHandle_, 0, mcSize_);
            mcBound_ = false;
        }
        dev->ReleasePhys(mcHandle_);
        mcHandle_ = 0;
    }

    int Initialize()
    {
        MF_TRACE_BEGIN(TP_SHM_CREATE);
        int rc = Steps();
        if (rc != OK) entity_.reset();  // dropping the entity unmaps, frees and unreserves whatever was done
        MF_TRACE_END(TP_SHM_CREATE, rc);
        return rc;
    }

    int Steps()
    {
        store_ = store::StoreFactory::Prefixed(g_.store, "(" + std::to_string(id_) + ")_");
        group::GroupOption go;
        go.rankSize = rankSize_;
        go.rank = rank_;
        go.timeoutMs = 1000ULL * g_.config.controlOperationTimeout;
        go.dynamic = false;
        group_ = group::GroupEngine::Create(store_, go);
        if (!group_) return ERR_INVALID_PARAM;
        symmetric_ = AlignUp(localSize_, kGiB);
        hybm_options ho{};
        ho.bmType = HYBM_TYPE_AI_CORE_INITIATE;
        ho.memType = HYBM_MEM_TYPE_DEVICE;
        ho.bmDataOpType = (hybm_data_op_type)(HYBM_DOP_TYPE_MTE | HYBM_DOP_TYPE_SDMA);
        ho.rankCount = rankSize_;
        ho.rankId = rank_;
        ho.devId = g_.deviceId;
        ho.maxHBMSize = symmetric_;
        ho.scene = HYBM_SCENE_SHM;
        ho.role = HYBM_ROLE_PEER;
        ho.flags = flags_;
        ho.dramShmFd = -1;
        entity_ = Entity::Create((uint16_t)(kShmEntityBase + id_), ho);
        if (!entity_) return LastError::Code() != 0 ? LastError::Code() : (int)ERR;
        // reserve: all ranks walk the same window sequence until every one of them succeeded
        int rc = ERR;
        for (uint32_t attempt = 0; attempt < kReserveAttempts; attempt++) {
            int32_t mine = entity_->ReserveMemSpace(attempt);
            std::vector<int32_t> all(rankSize_, 0);
            rc = group_->AllGather(reinterpret_cast<const char *>(&mine), sizeof(mine), reinterpret_cast<char *>(all.data()),
                                   (uint32_t)(all.size() * sizeof(int32_t)));
            if (rc != OK) return rc;
            bool ok = true;
            for (auto v : all) ok = ok && v == OK;
            if (ok) {
                rc = OK;
                break;
            }
            if (mine == OK) entity_->UnreserveMemSpace();
            rc = ERR_NO_RESOURCES;
        }
        if (rc != OK) return MF_FAIL(rc, "shm %u: no GVA window is free in every rank", id_);
        MemSlice *slice = nullptr;
        rc = entity_->AllocLocal(HYBM_MEM_TYPE_DEVICE, localSize_, 0, &slice);
        int all = GatherOk(rc);
        if (all != OK) return rc != OK ? rc : all;
        // exchange slices, then entities
        hybm_exchange_info mine[2];
        rc = entity_->Export(slice, &mine[0]);
        if (rc == OK) rc = entity_->Export(nullptr, &mine[1]);
        if (rc != OK) return rc;
        std::vector<hybm_exchange_info> everyone((size_t)rankSize_ * 2);
        rc = group_->AllGather(reinterpret_cast<const char *>(mine), sizeof(mine), reinterpret_cast<char *>(everyone.data()),
                               (uint32_t)(everyone.size() * sizeof(hybm_exchange_info)));
        if (rc != OK) return rc;
        rc = entity_->Import(everyone.data(), (uint32_t)everyone.size(), nullptr);
        all = GatherOk(rc);
        if (all != OK) return rc != OK ? rc : all;
        rc = entity_->Mmap();
        all = GatherOk(rc);
        if (all != OK) return rc != OK ? rc : all;
        gva_ = entity_->MemoryPtr(HYBM_MEM_TYPE_DEVICE);
        return SetupMulticast();
    }

    int GatherOk(int32_t mine)
    {
        std::vector<int32_t> all(rankSize_, 0);
        int rc = group_->AllGather(reinterpret_cast<const char *>(&mine), sizeof(mine), reinterpret_cast<char *>(all.data()),
                                   (uint32_t)(all.size() * sizeof(int32_t)));
        if (rc != OK) return rc;
        for (auto v : all)
            if (v != OK) return v;
        return OK;
    }

    uint32_t id_, rankSize_, rank_;
    uint64_t localSize_;
    uint32_t ops_, flags_;
    ShmGlobals g_;
    uint64_t symmetric_ = 0;
    store::StorePtr store_;
    group::GroupPtr group_;
    EntityPtr entity_;
    void *gva_ = nullptr;
    uint64_t mcBase_ = 0, mcSize_ = 0;
    PhysHandle mcHandle_ = 0;
    bool mcBound_ = false;
};

std::mutex g_mu;
ShmGlobals g_shm;
// leaked on purpose: tearing pools down from static destructors would call into a CUDA driver that
// is already shutting down
HandleTable<ShmEntry> &g_handles = *new HandleTable<ShmEntry>();

std::shared_ptr<ShmEntry> H(smem_shm_t h)
{
    if (h == nullptr) {
        MF_FAIL(SMEM_INVALID_PARAM, "handle is NULL");
        return nullptr;
    }
    auto e = g_handles.Find(h);
    if (!e) MF_FAIL(SMEM_INVALID_PARAM, "handle %p is not a live shared-memory object", h);
    return e;
}
}  // namespace

extern "C" {

int32_t smem_shm_config_init(smem_shm_config_t *config)
{
    if (config == nullptr) return MF_FAIL(SMEM_INVALID_PARAM, "config is NULL");
    config->shmInitTimeout = kDefaultTimeoutSec;
    config->shmCreateTimeout = kDefaultTimeoutSec;
    config->controlOperationTimeout = kDefaultTimeoutSec;
    config->startConfigStoreServer = true;
    config->flags = 0;
    return SMEM_OK;
}

int32_t smem_shm_init(const char *configStoreIpPort, uint32_t worldSize, uint32_t rankId, uint16_t deviceId,
                      smem_shm_config_t *config)
{
    if (configStoreIpPort == nullptr || *configStoreIpPort == 0) return MF_FAIL(SMEM_INVALID_PARAM, "store address is empty");
    if (config == nullptr) return MF_FAIL(SMEM_INVALID_PARAM, "config is NULL");
    if (worldSize == 0 || worldSize > SMEM_WORLD_SIZE_MAX || rankId >= worldSize)
        return MF_FAIL(SMEM_INVALID_PARAM, "rank %u / world %u out of range", rankId, worldSize);
    if (config->shmInitTimeout == 0 || config->shmCreateTimeout == 0 || config->controlOperationTimeout == 0)
        return MF_FAIL(SMEM_INVALID_PARAM, "timeouts must be at least 1 second");
    if (!SmemInited()) return MF_FAIL(SMEM_NOT_INIT, "smem_init has not been called");
    std::lock_guard<std::mutex> g(g_mu);
    if (g_shm.inited) return MF_FAIL(SMEM_REPEAT_INVOKE, "smem_shm_init called twice");
    std::string url = configStoreIpPort;
    if (url.find("://") == std::string::npos) url = "tcp://" + url;
    int err = OK;
    auto base = store::StoreFactory::CreateStore(url, config->startConfigStoreServer && rankId == 0, worldSize, rankId,
                                                 1000u * config->shmInitTimeout, 0, &err);
    if (!base) return MF_FAIL(Pub(err), "cannot reach the config store at %s (%d)", url.c_str(), err);
    int rc = HybmInit(deviceId, 0);
    if (rc != OK) {
        store::StoreFactory::DestroyStore(url);
        return Pub(rc);
    }
    g_shm = ShmGlobals();
    g_shm.url = url;
    g_shm.worldSize = worldSize;
    g_shm.rank = rankId;
    g_shm.deviceId = deviceId;
    g_shm.config = *config;
    g_shm.store = store::StoreFactory::Prefixed(base, "SHM_");
    g_shm.inited = true;
    return SMEM_OK;
}

void smem_shm_uninit(uint32_t)
{
    std::lock_guard<std::mutex> g(g_mu);
    if (!g_shm.inited) return;
    for (auto &e : g_handles.TakeAll()) e.reset();
    g_shm.store.reset();
    store::StoreFactory::DestroyStore(g_shm.url);
    HybmUninit();
    g_shm = ShmGlobals();
}

uint32_t smem_shm_query_support_data_operation(void)
{
    auto *dev = CurrentBackend();
    if (dev == nullptr) return 0;
    return SMEMS_DATA_OP_MTE | SMEMS_DATA_OP_SDMA;
}

smem_shm_t smem_shm_create(uint32_t id, uint32_t rankSize, uint32_t rankId, uint64_t localSize,
                           smem_shm_data_op_type dataOpType, uint32_t flags, void **gva)
{
    if (gva == nullptr || localSize == 0 || rankSize == 0 || rankId >= rankSize || id > kIdMax) {
        MF_FAIL(SMEM_INVALID_PARAM, "shm create: bad id %u, rank %u/%u, size %lu or NULL gva", id, rankId, rankSize,
                (unsigned long)localSize);
        return nullptr;
    }
    ShmGlobals snap;
    {
        std::lock_guard<std::mutex> g(g_mu);
        if (!g_shm.inited) {
            MF_FAIL(SMEM_NOT_INIT, "smem_shm_init has not been called");
            return nullptr;
        }
        snap = g_shm;
    }
    if (rankSize > snap.worldSize) {
        MF_FAIL(SMEM_INVALID_PARAM, "shm create: rank size %u above world %u", rankSize, snap.worldSize);
        return nullptr;
    }
    auto e = std::make_shared<ShmEntry>(id, rankSize, rankId, localSize, (uint32_t)dataOpType, flags, snap);
    int rc = e->Initialize();
    if (rc != OK) {
        if (LastError::Code() == 0) LastError::Set(Pub(rc), "shm %u: create failed with %d", id, rc);
        return nullptr;
    }
    // no extra context yet: a kernel that asks for its size must read 0
    {
        const uint64_t at = reinterpret_cast<uint64_t>(e->gva_) + (uint64_t)e->rank_ * e->symmetric_ + SMEM_SHM_EXTRA_CTX_OFFSET;
        hybm::DeviceBackend *dev = hybm::CurrentBackend();
        if (localSize >= SMEM_SHM_USER_OFFSET) {   // a slice smaller than the flag area has no room for it (host-side copy only)
            if (dev != nullptr && dev->Caps().present) {
                dev->BindThread();
                if (dev->MemsetAsync(at, 0, 64, nullptr) == OK) dev->StreamSync(nullptr);
            } else {
                memset(reinterpret_cast<void *>(at), 0, 64);
            }
        }
    }
    *gva = e->gva_;
    return g_handles.Add(e);
}

uint64_t smem_shm_get_symmetric_size(smem_shm_t handle)
{
    auto e = H(handle);
    return e ? e->symmetric_ : 0;
}

int32_t smem_shm_get_device_context(smem_shm_t handle, void *ctx, uint32_t ctxSize)
{
    auto e = H(handle);
    if (!e || ctx == nullptr) return MF_FAIL(SMEM_INVALID_PARAM, "bad handle or NULL context");
    smem_shm_device_ctx_t c{};
    if (ctxSize < sizeof(c)) return MF_FAIL(SMEM_INVALID_PARAM, "context block of %u bytes, %zu needed", ctxSize, sizeof(c));
    c.base = reinterpret_cast<uint64_t>(e->gva_);
    c.symmetric_size = e->symmetric_;
    c.mc_base = e->mcBase_;
    c.rank = e->rank_;
    c.rank_size = e->rankSize_;
    c.spin_limit = (uint32_t)EnvInt("MF_SHM_SPIN_LIMIT", nullptr, 1 << 22, 1024, 1u << 30);
    memcpy(ctx, &c, sizeof(c));
    return SMEM_OK;
}

int32_t smem_shm_destroy(smem_shm_t handle, uint32_t)
{
    auto e = g_handles.Take(handle);
    if (!e) return MF_FAIL(SMEM_INVALID_PARAM, "handle %p is not a live shared-memory object", handle);
    e.reset();
    return SMEM_OK;
}

int32_t smem_shm_set_extra_context(smem_shm_t handle, const void *context, uint32_t size)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    if (context == nullptr || size == 0 || size > 65536) return MF_FAIL(SMEM_INVALID_PARAM, "context must be 1..65536 bytes");
    int rc = e->entity_->SetExtraContext(context, size);
    if (rc != OK) return Pub(rc);
    // kernels read it through smem_shm_get_extra_context_addr / _size (smem_shm_device.cuh): bytes first, then the size
    const uint64_t at = reinterpret_cast<uint64_t>(e->gva_) + (uint64_t)e->rank_ * e->symmetric_ + SMEM_SHM_EXTRA_CTX_OFFSET;
    hybm::DeviceBackend *dev = hybm::CurrentBackend();
    if (e->localSize_ < SMEM_SHM_USER_OFFSET) return SMEM_OK;  // no flag area in such a small slice: kernels cannot read it
    if (dev != nullptr && dev->Caps().present) {
        dev->BindThread();
        alignas(16) uint32_t hdr[4] = {size, 0, 0, 0};
        rc = dev->MemcpyAsync(at + 64, reinterpret_cast<uint64_t>(context), size, hybm::CPY_H2D, nullptr);
        if (rc == OK) rc = dev->MemcpyAsync(at, reinterpret_cast<uint64_t>(hdr), sizeof(hdr), hybm::CPY_H2D, nullptr);
        if (rc == OK) rc = dev->StreamSync(nullptr);
    } else {
        memcpy(reinterpret_cast<void *>(at + 64), context, size);
        *reinterpret_cast<volatile uint32_t *>(at) = size;
    }
    return Pub(rc);
}

uint32_t smem_shm_get_global_rank(smem_shm_t handle)
{
    auto e = H(handle);
    return e ? e->rank_ : UINT32_MAX;
}

uint32_t smem_shm_get_global_rank_size(smem_shm_t handle)
{
    auto e = H(handle);
    return e ? e->rankSize_ : UINT32_MAX;
}

int32_t smem_shm_control_barrier(smem_shm_t handle)
{
    auto e = H(handle);
    return e ? Pub(e->group_->Barrier()) : SMEM_INVALID_PARAM;
}

int32_t smem_shm_control_allgather(smem_shm_t handle, const char *sendBuf, uint32_t sendSize, char *recvBuf,
                                   uint32_t recvSize)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    if (sendBuf == nullptr || recvBuf == nullptr || sendSize == 0 || (uint64_t)sendSize * e->rankSize_ != recvSize)
        return MF_FAIL(SMEM_INVALID_PARAM, "allgather: recvSize must equal sendSize x rank size");
    return Pub(e->group_->AllGather(sendBuf, sendSize, recvBuf, recvSize));
}

int32_t smem_shm_subgroup_barrier(smem_shm_t handle, const char *key, uint32_t rankSize, uint32_t rankId)
{
    auto e = H(handle);
    return e ? Pub(e->group_->Barrier(key, rankSize, rankId)) : SMEM_INVALID_PARAM;
}

int32_t smem_shm_subgroup_allgather(smem_shm_t handle, const char *key, uint32_t rankSize, uint32_t rankId,
                                    const char *sendBuf, uint32_t sendSize, char *recvBuf, uint32_t recvSize)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    if (sendBuf == nullptr || recvBuf == nullptr || sendSize == 0 || (uint64_t)sendSize * rankSize != recvSize)
        return MF_FAIL(SMEM_INVALID_PARAM, "sub-group allgather: recvSize must equal sendSize x rank size");
    return Pub(e->group_->AllGather(key, rankSize, rankId, sendBuf, sendSize, recvBuf, recvSize));
}

int32_t smem_shm_topology_can_reach(smem_shm_t handle, uint32_t remoteRank, uint32_t *reachInfo)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    if (reachInfo == nullptr || remoteRank >= e->rankSize_) return MF_FAIL(SMEM_INVALID_PARAM, "bad remote rank or NULL result");
    uint32_t types = 0;
    int rc = e->entity_->ReachTypes(remoteRank, types);
    if (rc != OK) return Pub(rc);
    uint32_t out = 0;
    if (types & HYBM_DOP_TYPE_MTE) out |= SMEMS_DATA_OP_MTE;
    if (types & HYBM_DOP_TYPE_SDMA) out |= SMEMS_DATA_OP_SDMA;
    *reachInfo = out;
    return SMEM_OK;
}

int32_t smem_shm_atomic_alloc_value(smem_shm_t handle, uint32_t limit, int32_t *value)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    if (value == nullptr || limit == 0 || limit > SMEM_SHM_ATOMIC_NUM_LIMIT) return MF_FAIL(SMEM_INVALID_PARAM, "limit must be 1..1024");
    return Pub(e->group_->AllocNumber(limit, *value));
}

int32_t smem_shm_atomic_release_value(smem_shm_t handle, int32_t value)
{
    auto e = H(handle);
    return e ? Pub(e->group_->ReleaseNumber(value)) : SMEM_INVALID_PARAM;
}

int32_t smem_shm_register_exit(smem_shm_t handle, void (*exitFn)(int))
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    if (exitFn == nullptr) return MF_FAIL(SMEM_INVALID_PARAM, "exit callback is NULL");
    return Pub(e->group_->RegisterExit([exitFn](int st) { exitFn(st); }));
}

void smem_shm_global_exit(smem_shm_t handle, int status)
{
    auto e = H(handle);
    if (e) e->group_->BroadcastExit(status);
}

}  // extern "C"
