#include "mf_entity.h"

#include <chrono>

#include <sys/prctl.h>
#include <unistd.h>

#include <fstream>

#include "../util/mf_trace.h"

namespace mf {
namespace hybm {

namespace {
constexpr uint32_t kUserSliceMark = 0x80000000u;
std::atomic<bool> g_inited{false};
std::atomic<int> g_initRefs{0};
DeviceBackend *g_dev = nullptr;

std::string BootId()
{
    static std::string id = [] {
        std::ifstream f("/proc/sys/kernel/random/boot_id");
        std::string s;
        std::getline(f, s);
        if (s.empty()) {
            char h[128] = {0};
            gethostname(h, sizeof(h) - 1);
            s = h;
        }
        return s;
    }();
    return id;
}

uint8_t SideClass(hybm_data_copy_direction d, bool src)
{
    switch (d) {
        case HYBM_LOCAL_HOST_TO_GLOBAL_HOST: return src ? AC_LH : AC_GH;
        case HYBM_LOCAL_HOST_TO_GLOBAL_DEVICE: return src ? AC_LH : AC_GD;
        case HYBM_LOCAL_DEVICE_TO_GLOBAL_HOST: return src ? AC_LD : AC_GH;
        case HYBM_LOCAL_DEVICE_TO_GLOBAL_DEVICE: return src ? AC_LD : AC_GD;
        case HYBM_GLOBAL_HOST_TO_GLOBAL_HOST: return AC_GH;
        case HYBM_GLOBAL_HOST_TO_GLOBAL_DEVICE: return src ? AC_GH : AC_GD;
        case HYBM_GLOBAL_HOST_TO_LOCAL_HOST: return src ? AC_GH : AC_LH;
        case HYBM_GLOBAL_HOST_TO_LOCAL_DEVICE: return src ? AC_GH : AC_LD;
        case HYBM_GLOBAL_DEVICE_TO_GLOBAL_HOST: return src ? AC_GD : AC_GH;
        case HYBM_GLOBAL_DEVICE_TO_GLOBAL_DEVICE: return AC_GD;
        case HYBM_GLOBAL_DEVICE_TO_LOCAL_HOST: return src ? AC_GD : AC_LH;
        case HYBM_GLOBAL_DEVICE_TO_LOCAL_DEVICE: return src ? AC_GD : AC_LD;
        default: return AC_NONE;
    }
}
}  // namespace

int HybmInit(uint16_t deviceId, uint64_t flags)
{
    (void)flags;
    if (g_initRefs.fetch_add(1) > 0) return OK;
    std::string why;
    g_dev = AcquireBackend(deviceId == 0xFFFF ? 0 : deviceId, &why);
    if (g_dev == nullptr) MF_INFO("no device backend (%s): host-memory pools only", why.c_str());
    else MF_INFO("device backend %s on device %d (%s)", g_dev->Name(), g_dev->DeviceId(), g_dev->Caps().name);
    if (EnvInt("MF_PTRACER_ENABLE", "ENABLE_PTRACER", 0, 0, 1) == 1) PTracer::Start();
    g_inited = true;
    return OK;
}

void HybmUninit()
{
    if (g_initRefs.load() == 0) return;
    if (g_initRefs.fetch_sub(1) > 1) return;
    g_inited = false;
    PTracer::Stop();
    if (g_dev != nullptr) ReleaseBackend();
    g_dev = nullptr;
}

bool HybmInited() { return g_inited.load(); }

std::shared_ptr<Entity> Entity::Create(uint16_t id, const hybm_options &opt)
{
    if (!g_inited) {
        MF_FAIL(ERR_NOT_INIT, "hybm is not initialised");
        return nullptr;
    }
    if (id > kMaxEntityId || opt.rankCount == 0 || opt.rankCount > 1024 || opt.rankId >= opt.rankCount) {
        MF_FAIL(ERR_INVALID_PARAM, "entity %u: bad rank %u of %u", id, opt.rankId, opt.rankCount);
        return nullptr;
    }
    if ((opt.memType & HYBM_MEM_TYPE_DEVICE) != 0 && opt.maxHBMSize != 0 && g_dev == nullptr) {
        MF_FAIL(ERR_NOT_INIT, "entity %u asks for an HBM pool but no device backend is available", id);
        return nullptr;
    }
    return std::make_shared<Entity>(id, opt, g_dev);
}

Entity::Entity(uint16_t id, const hybm_options &opt, DeviceBackend *dev) : id_(id), opt_(opt), dev_(dev)
{
    ops_ = std::make_unique<ComposeDataOp>(dev_, (uint32_t)opt.bmDataOpType);
    transCursor_ = kTransWindowBase;
}

Entity::~Entity()
{
    ops_->Wait();
    for (auto &kv : userSlices_) VaManager::Get().RemoveLocal(kv.first);
    for (auto &rk : remote_)
        for (auto &kv : rk.second)
            if (kv.second.mapped != 0 && dev_ != nullptr) dev_->IpcClose(kv.second.mapped);
    UnreserveMemSpace();
}

int Entity::ReserveMemSpace(uint32_t attempt)
{
    std::lock_guard<std::mutex> g(mu_);
    if (dev_ != nullptr) dev_->BindThread();
    SegmentOptions so;
    so.entityId = id_;
    so.rank = opt_.rankId;
    so.rankCount = opt_.rankCount;
    so.flags = opt_.flags;
    so.shmFd = opt_.dramShmFd;
    so.dev = dev_;
    if ((opt_.memType & HYBM_MEM_TYPE_DEVICE) != 0 && opt_.maxHBMSize != 0 && !hbm_) {
        so.type = HYBM_MEM_TYPE_DEVICE;
        so.slot = AlignUp(opt_.maxHBMSize, kHbmGranule);
        so.publicSlot = 0;
        if (opt_.enable56BitsGva && so.slot > kCompactThreshold / so.rankCount) {  // as for pooled DRAM below
            if (so.slot > kGva56WindowStride / so.rankCount)
                return MF_FAIL(ERR_INVALID_PARAM, "an HBM pool of %u ranks x %lu bytes exceeds the 1 PiB of a 56-bit address window", so.rankCount,
                               (unsigned long)so.slot);
            so.publicSlot = so.slot;
            so.slot = CompactSlot(so.rankCount);
            MF_INFO("HBM pool %u: 56-bit addresses, %lu bytes per rank for callers, %lu mapped per rank in this process", id_,
                    (unsigned long)so.publicSlot, (unsigned long)so.slot);
        }
        auto seg = Segment::Create(so);
        if (!seg) return ERR_NOT_INIT;
        int rc = seg->Reserve(attempt);
        if (rc != OK) return rc;
        hbm_ = seg;
    }
    if ((opt_.memType & HYBM_MEM_TYPE_HOST) != 0 && opt_.maxDRAMSize != 0 && !dram_) {
        so.type = HYBM_MEM_TYPE_HOST;
        so.slot = AlignUp(opt_.maxDRAMSize, 2ULL << 20);
        so.publicSlot = 0;
        if (opt_.enable56BitsGva && so.slot > kCompactThreshold / so.rankCount) {
            // too large to map whole: callers get 56-bit addresses, the process a compact window (mf_hybm_types.h)
            if (so.slot > kGva56WindowStride / so.rankCount)
                return MF_FAIL(ERR_INVALID_PARAM, "a DRAM pool of %u ranks x %lu bytes exceeds the 1 PiB of a 56-bit address window",
                               so.rankCount, (unsigned long)so.slot);
            so.publicSlot = so.slot;
            so.slot = CompactSlot(so.rankCount);
            MF_INFO("DRAM pool %u: 56-bit addresses, %lu bytes per rank for callers, %lu mapped per rank in this process", id_,
                    (unsigned long)so.publicSlot, (unsigned long)so.slot);
        }
        auto seg = Segment::Create(so);
        int rc = seg ? seg->Reserve(attempt) : ERR_NOT_INIT;
        if (rc != OK) {
            if (hbm_) {
                hbm_->Unreserve();
                hbm_.reset();
            }
            return rc;
        }
        dram_ = seg;
    }
    return OK;
}

int Entity::UnreserveMemSpace()
{
    std::lock_guard<std::mutex> g(mu_);
    pooled_.clear();
    if (hbm_) hbm_->Unreserve();
    if (dram_) dram_->Unreserve();
    hbm_.reset();
    dram_.reset();
    return OK;
}

void *Entity::MemoryPtr(hybm_mem_type t)
{
    auto seg = SegmentOf(t);
    return seg ? reinterpret_cast<void *>(seg->PubBase()) : nullptr;
}

uint64_t Entity::LocalBytes(hybm_mem_type t)
{
    auto seg = SegmentOf(t);
    return seg ? seg->LocalBytes() : 0;
}

int Entity::AllocLocal(hybm_mem_type t, uint64_t size, uint32_t, MemSlice **out)
{
    auto seg = SegmentOf(t);
    if (!seg) return MF_FAIL(ERR_NOT_STARTED, "entity %u has no %s pool", id_, t == HYBM_MEM_TYPE_HOST ? "DRAM" : "HBM");
    if (dev_ != nullptr) dev_->BindThread();
    MF_TRACE_BEGIN(TP_HYBM_ALLOC);
    int32_t rc = OK;
    std::shared_ptr<MemSlice> s;
    MF_FIP_START(ALLOC_LOCAL_MEMORY, &rc)
    rc = seg->AllocLocal(size, s);
    MF_FIP_END
    if (rc == OK) {
        std::lock_guard<std::mutex> g(mu_);
        pooled_[s.get()] = s;
        *out = s.get();
    }
    MF_TRACE_END(TP_HYBM_ALLOC, rc);
    return rc;
}

int Entity::FreeLocal(MemSlice *s)
{
    if (s == nullptr || !s->Valid()) return ERR_INVALID_PARAM;
    if (s->origin == SL_USER) return UnregisterLocal(s->gva);
    std::shared_ptr<MemSlice> sp;
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = pooled_.find(s);
        if (it == pooled_.end()) return ERR_NOT_EXIST;
        sp = it->second;
        pooled_.erase(it);
    }
    return SegmentOf(sp->memType)->FreeLocal(sp);
}

int Entity::RegisterLocal(const void *ptr, uint64_t size, uint32_t, MemSlice **out)
{
    uint64_t addr = reinterpret_cast<uint64_t>(ptr);
    if (addr == 0 || size == 0) return ERR_INVALID_PARAM;
    bool device = dev_ != nullptr && dev_->IsDevicePointer(addr);
    auto s = std::make_unique<MemSlice>();
    s->origin = SL_USER;
    s->memType = device ? HYBM_MEM_TYPE_DEVICE : HYBM_MEM_TYPE_HOST;
    s->gva = addr;
    s->size = size;
    if (!device) {
        // Peers reach registered host memory with process_vm_*: allow any process of this user to attach.
        static std::once_flag once;
        std::call_once(once, [] { prctl(PR_SET_PTRACER, PR_SET_PTRACER_ANY, 0, 0, 0); });
    }
    std::lock_guard<std::mutex> g(mu_);
    if (userSlices_.count(addr)) return MF_FAIL(ERR_DUPLICATED, "address %#lx is already registered", (unsigned long)addr);
    s->index = (uint32_t)userSlices_.size();
    VaManager::Get().AddLocal(addr, size, device);
    *out = s.get();
    userSlices_[addr] = std::move(s);
    return OK;
}

int Entity::UnregisterLocal(uint64_t addr)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = userSlices_.find(addr);
    if (it == userSlices_.end()) return MF_FAIL(ERR_NOT_EXIST, "address %#lx was not registered", (unsigned long)addr);
    VaManager::Get().RemoveLocal(addr);
    userSlices_.erase(it);
    return OK;
}

int Entity::Export(const MemSlice *s, hybm_exchange_info *out)
{
    if (out == nullptr) return ERR_INVALID_PARAM;
    MF_TRACE_BEGIN(TP_HYBM_EXPORT);
    int rc = OK;
    if (s == nullptr) {
        ExWriter w(out);
        ExHeader h;
        h.kind = EX_ENTITY;
        h.rank = opt_.rankId;
        h.entityId = id_;
        uint32_t role = opt_.role;
        int32_t pid = getpid();
        int32_t dev = dev_ != nullptr ? dev_->DeviceId() : -1;
        bool ok = w.Put(h) && w.Put(role) && w.Put(pid) && w.Put(dev) && w.PutStr(BootId()) && w.PutStr(opt_.tag);
        rc = ok ? OK : ERR;
    } else if (!s->Valid()) {
        rc = ERR_INVALID_PARAM;
    } else if (s->origin == SL_POOL) {
        rc = SegmentOf(s->memType)->Export(*s, out);
    } else {
        ExWriter w(out);
        ExHeader h;
        h.kind = EX_SLICE;
        h.rank = opt_.rankId;
        h.entityId = id_;
        bool device = s->memType == HYBM_MEM_TYPE_DEVICE;
        uint32_t type = kUserSliceMark | (device ? 1u : 2u);
        int32_t pid = getpid();
        uint8_t ipc[64] = {0};
        uint64_t ipcBase = 0, ipcSize = 0;
        if (device) {
            if (dev_ != nullptr) dev_->BindThread();
            rc = dev_->IpcExport(s->gva, ipc, &ipcBase, &ipcSize);
            if (rc != OK) rc = MF_FAIL(rc, "cannot export device buffer %#lx for inter-process access", (unsigned long)s->gva);
        }
        if (rc == OK) {
            bool ok = w.Put(h) && w.Put(type) && w.Put(s->gva) && w.Put(s->size) && w.Put(pid) && w.Put(ipcBase) &&
                      w.Put(ipcSize) && w.PutBytes(ipc, sizeof(ipc));
            rc = ok ? OK : ERR;
        }
    }
    MF_TRACE_END(TP_HYBM_EXPORT, rc);
    return rc;
}

int Entity::Import(const hybm_exchange_info infos[], uint32_t count, void *addresses[])
{
    MF_TRACE_BEGIN(TP_HYBM_IMPORT);
    int32_t rc = OK;
    MF_FIP_START(IMPORT, &rc)
    for (uint32_t i = 0; i < count && rc == OK; i++) {
        const hybm_exchange_info &in = infos[i];
        if (in.descLen == 0) continue;  // a rank that has nothing to share yet
        ExReader r(&in);
        ExHeader h;
        if (!r.Take(h) || h.magic != kExMagic || h.version != kExVersion) {
            rc = MF_FAIL(ERR_INVALID_PARAM, "exchange blob %u: bad magic or version", i);
            break;
        }
        if (h.kind == EX_ENTITY) {
            PeerEntity p;
            p.rank = h.rank;
            if (!r.Take(p.role) || !r.Take(p.pid) || !r.Take(p.devId) || !r.TakeStr(p.host) || !r.TakeStr(p.tag)) {
                rc = MF_FAIL(ERR_INVALID_PARAM, "exchange blob %u: truncated entity record", i);
                break;
            }
            std::lock_guard<std::mutex> g(mu_);
            peers_[p.rank] = p;
            continue;
        }
        uint32_t type = 0;
        if (!r.Take(type)) {
            rc = ERR_INVALID_PARAM;
            break;
        }
        if ((type & kUserSliceMark) != 0) {
            RemoteRegion reg;
            reg.rank = h.rank;
            reg.device = (type & 1u) != 0;
            uint64_t ipcSize = 0;
            if (!r.Take(reg.remoteAddr) || !r.Take(reg.size) || !r.Take(reg.pid) || !r.Take(reg.mappedBase) ||
                !r.Take(ipcSize) || !r.TakeBytes(reg.ipc, sizeof(reg.ipc))) {
                rc = MF_FAIL(ERR_INVALID_PARAM, "exchange blob %u: truncated user-buffer record", i);
                break;
            }
            if (h.rank == opt_.rankId) continue;
            std::lock_guard<std::mutex> g(mu_);
            auto &m = remote_[h.rank];
            auto it = m.find(reg.remoteAddr);
            if (it != m.end() && it->second.size == reg.size && it->second.pid == reg.pid) continue;
            if (it != m.end() && it->second.mapped != 0 && dev_ != nullptr) dev_->IpcClose(it->second.mapped);
            m[reg.remoteAddr] = reg;
            if (addresses != nullptr) addresses[i] = reinterpret_cast<void *>(reg.remoteAddr);
            continue;
        }
        auto seg = SegmentOf((hybm_mem_type)type);
        if (!seg) {
            rc = MF_FAIL(ERR_INVALID_PARAM, "rank %u shares a %s slice but this entity has no such pool", h.rank,
                         type == HYBM_MEM_TYPE_HOST ? "DRAM" : "HBM");
            break;
        }
        uint64_t addr = 0;
        rc = seg->Import(in, &addr);
        if (rc == OK && addresses != nullptr) addresses[i] = reinterpret_cast<void *>(addr);
    }
    MF_FIP_END
    MF_TRACE_END(TP_HYBM_IMPORT, rc);
    return rc;
}

int Entity::Mmap()
{
    if (dev_ != nullptr) dev_->BindThread();
    int32_t rc = OK;
    MF_FIP_START(MMAP, &rc)
    if (hbm_) rc = hbm_->Mmap();
    if (rc == OK && dram_) rc = dram_->Mmap();
    if (rc == OK) {
        // open IPC mappings of peers' registered device buffers
        std::lock_guard<std::mutex> g(mu_);
        for (auto &rk : remote_)
            for (auto &kv : rk.second) {
                RemoteRegion &reg = kv.second;
                if (!reg.device || reg.mapped != 0) continue;
                if (dev_ == nullptr) {
                    rc = ERR_NOT_INIT;
                    break;
                }
                int r = dev_->IpcOpen(reg.ipc, &reg.mapped);
                if (r != OK) {
                    rc = MF_FAIL(r, "cannot open device buffer %#lx of rank %u", (unsigned long)reg.remoteAddr, reg.rank);
                    break;
                }
            }
    }
    MF_FIP_END
    return rc;
}

void Entity::Unmap()
{
    if (hbm_) hbm_->UnmapAll();
    if (dram_) dram_->UnmapAll();
    std::lock_guard<std::mutex> g(mu_);
    for (auto &rk : remote_)
        for (auto &kv : rk.second)
            if (kv.second.mapped != 0 && dev_ != nullptr) {
                dev_->IpcClose(kv.second.mapped);
                kv.second.mapped = 0;
            }
    remote_.clear();
}

int Entity::RemoveImported(uint32_t rank)
{
    mapGen_.fetch_add(1);
    ops_->Wait();
    if (hbm_) hbm_->RemoveImported(rank);
    if (dram_) dram_->RemoveImported(rank);
    std::lock_guard<std::mutex> g(mu_);
    auto it = remote_.find(rank);
    if (it != remote_.end()) {
        for (auto &kv : it->second)
            if (kv.second.mapped != 0 && dev_ != nullptr) dev_->IpcClose(kv.second.mapped);
        remote_.erase(it);
    }
    peers_.erase(rank);
    return OK;
}

int Entity::SetExtraContext(const void *ctx, uint32_t size)
{
    if (ctx == nullptr || size == 0 || size > 64 * 1024) return ERR_INVALID_PARAM;
    std::lock_guard<std::mutex> g(mu_);
    extraCtx_.assign(static_cast<const char *>(ctx), size);
    return OK;
}

int Entity::ReachTypes(uint32_t rank, uint32_t &types)
{
    types = 0;
    if (rank == opt_.rankId) {
        types = HYBM_DOP_TYPE_MTE | HYBM_DOP_TYPE_SDMA | HYBM_DOP_TYPE_HOST_SHM;
        return OK;
    }
    std::lock_guard<std::mutex> g(mu_);
    auto it = peers_.find(rank);
    if (it == peers_.end()) return MF_FAIL(ERR_NOT_EXIST, "rank %u has not been imported", rank);
    if (it->second.host == BootId()) {
        types |= HYBM_DOP_TYPE_HOST_SHM;
        bool p2p = dev_ != nullptr && it->second.devId >= 0 &&
                   (it->second.devId == dev_->DeviceId() || dev_->CanAccessPeer(it->second.devId) == 1);
        if (p2p) types |= HYBM_DOP_TYPE_MTE | HYBM_DOP_TYPE_SDMA;
    }
    return OK;
}

std::vector<PeerEntity> Entity::Peers()
{
    std::lock_guard<std::mutex> g(mu_);
    std::vector<PeerEntity> v;
    for (auto &kv : peers_) v.push_back(kv.second);
    return v;
}

int Entity::TranslateRemote(uint32_t rank, uint64_t addr, uint64_t len, RemoteRegion &out, uint64_t &local)
{
    std::lock_guard<std::mutex> g(mu_);
    auto rk = remote_.find(rank);
    if (rk == remote_.end()) return ERR_NOT_EXIST;
    auto it = rk->second.upper_bound(addr);
    if (it == rk->second.begin()) return ERR_NOT_EXIST;
    --it;
    const RemoteRegion &reg = it->second;
    if (addr + len > reg.remoteAddr + reg.size) return ERR_NOT_EXIST;
    out = reg;
    local = reg.device ? (reg.mapped != 0 ? reg.mapped + (addr - reg.mappedBase) : 0) : addr;
    if (reg.device && reg.mapped == 0) return ERR_NOT_STARTED;
    return OK;
}

// ------------------------------------------------------------------------------------------------
bool Entity::InPool(const SegmentPtr &seg, uint64_t addr, uint64_t len, int &err, uint64_t *local) const
{
    if (!seg || seg->Base() == 0) return false;
    uint64_t base = seg->PubBase(), slot = seg->PubSlot();
    if (addr < base) return false;
    uint64_t rel = addr - base;
    uint64_t rank64 = rel / slot;
    if (rank64 >= opt_.rankCount) return false;
    uint32_t rank = (uint32_t)rank64;
    uint64_t off = rel - (uint64_t)rank * slot;
    const uint64_t mapped = seg->MappedBytes(rank);
    if (len > mapped || off > mapped - len) {  // written so that a huge len cannot wrap the sum
        err = mapped == 0 ? ERR_NOT_CONNECTED : ERR_INVALID_PARAM;
        return true;
    }
    err = OK;
    if (local != nullptr) *local = seg->Compact() ? seg->LocalOf(rank, off) : addr;  // 56-bit addresses are numbers: where it is mapped here
    return true;
}

// A caller's host buffer that is pinned and device-addressable can be read and written by the copy kernel
// directly: a batch of many small pieces between it and the pool then costs one launch instead of one
// copy-engine submission per piece. The last range that answered yes is remembered (the pieces of a batch
// usually lie in one buffer), so a batch pays for a couple of driver queries, not two per piece.
bool Entity::PinnedHost(uint64_t addr, uint64_t len)
{
    std::lock_guard<std::mutex> g(pinMu_);
    // what is remembered is trusted for 50 ms only: the buffer may have been freed and the addresses reused
    const uint64_t now = (uint64_t)std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now().time_since_epoch()).count();
    if (now - pinStampMs_ > 50) pinLo_ = pinHi_ = 0;
    if (pinHi_ > pinLo_ && addr >= pinLo_ && len <= pinHi_ - pinLo_ && addr - pinLo_ <= (pinHi_ - pinLo_) - len) return true;
    if (len == 0 || addr + len < addr || !dev_->IsPinnedHost(addr, len)) return false;
    // grow the remembered range when this piece touches or extends it, else start a new one
    if (pinHi_ > pinLo_ && addr <= pinHi_ && addr + len >= pinLo_) {
        pinLo_ = std::min(pinLo_, addr);
        pinHi_ = std::max(pinHi_, addr + len);
    } else {
        pinLo_ = addr;
        pinHi_ = addr + len;
        pinStampMs_ = now;
    }
    return true;
}

int Entity::Resolve(uint64_t addr, uint64_t len, bool isSrc, hybm_data_copy_direction dir, Endpoint &ep)
{
    ep.addr = addr;
    ep.pid = 0;
    int err = OK;
    uint8_t want = SideClass(dir, isSrc);
    if (InPool(hbm_, addr, len, err, &ep.addr)) {
        if (err != OK) return err;
        if (want != AC_NONE && want != AC_GD) return ERR_INVALID_PARAM;
        ep.kind = EP_DEVICE;
        return OK;
    }
    if (InPool(dram_, addr, len, err, &ep.addr)) {
        if (err != OK) return err;
        if (want != AC_NONE && want != AC_GH) return ERR_INVALID_PARAM;
        ep.kind = EP_HOST_PINNED;
        return OK;
    }
    if (want == AC_GD || want == AC_GH) return ERR_INVALID_PARAM;  // named a pooled side but the address is outside
    if (want == AC_LD) ep.kind = EP_DEVICE;
    else if (want == AC_LH) ep.kind = (dev_ != nullptr && PinnedHost(addr, len)) ? EP_HOST_PINNED : EP_HOST;
    else ep.kind = (dev_ != nullptr && dev_->IsDevicePointer(addr)) ? EP_DEVICE : EP_HOST;
    return OK;
}

int Entity::CopyData(const hybm_copy_params &p, hybm_data_copy_direction dir, void *stream, uint32_t flags)
{
    if (p.src == nullptr || p.dest == nullptr || p.dataSize == 0 || dir >= HYBM_DATA_COPY_DIRECTION_BUTT)
        return MF_FAIL(ERR_INVALID_PARAM, "copy: null address, zero size or bad direction %d", (int)dir);
    PublishCopyWindow();
    // (the one-element vector is thread-local: a copy call is often a few microseconds of work in total)
    static thread_local std::vector<ResolvedCopy> one(1);
    one.resize(1);
    one[0] = ResolvedCopy();
    one[0].len = p.dataSize;
    int rc = Resolve(reinterpret_cast<uint64_t>(p.src), p.dataSize, true, dir, one[0].src);
    if (rc == OK) rc = Resolve(reinterpret_cast<uint64_t>(p.dest), p.dataSize, false, dir, one[0].dst);
    if (rc != OK)
        return MF_FAIL(rc, "copy %p -> %p (%lu bytes, direction %d): address outside the mapped pool", p.src, p.dest,
                       (unsigned long)p.dataSize, (int)dir);
    // A short host-to-host copy (pooled DRAM on either side, no device involved) is a memcpy: skip the operator's queue.
    if (ops_->HostFast(one[0])) return OK;
    return ops_->Submit(one, stream, flags, nullptr);
}

void Entity::PublishCopyWindow()
{
    static const bool debug = EnvInt("MF_XCOPY_DEBUG", nullptr, 0, 0, 1) != 0;
    if (!debug || dev_ == nullptr || !hbm_ || hbm_->Base() == 0 || opt_.rankCount > 64) return;
    uint64_t mapped[64];
    for (uint32_t r = 0; r < opt_.rankCount; r++) mapped[r] = hbm_->MappedBytes(r);
    dev_->SetCopyWindow(hbm_->Base(), hbm_->Slot(), opt_.rankCount, mapped);
}

int Entity::BatchCopyData(const hybm_batch_copy_params &p, hybm_data_copy_direction dir, void *stream, uint32_t flags,
                          int32_t *perItem)
{
    if (p.sources == nullptr || p.destinations == nullptr || p.dataSizes == nullptr || p.batchSize == 0 ||
        dir >= HYBM_DATA_COPY_DIRECTION_BUTT)
        return MF_FAIL(ERR_INVALID_PARAM, "batch copy: null array, empty batch or bad direction %d", (int)dir);
    PublishCopyWindow();
    // Hot path: every item is device<->device with at least one side in the HBM pool (KV-block put/get).
    // Pass 1 validates with arithmetic only; pass 2 streams the items into the descriptor ring.
    if (perItem == nullptr && dev_ != nullptr && hbm_ && hbm_->Base() != 0 && !hbm_->Compact() &&  // (56-bit addresses need translating: general path)
        (dir == HYBM_LOCAL_DEVICE_TO_GLOBAL_DEVICE || dir == HYBM_GLOBAL_DEVICE_TO_GLOBAL_DEVICE ||
         dir == HYBM_GLOBAL_DEVICE_TO_LOCAL_DEVICE)) {
        const uint64_t base = hbm_->Base(), slot = hbm_->Slot();
        const uint64_t end = base + slot * opt_.rankCount;
        const bool srcPool = dir != HYBM_LOCAL_DEVICE_TO_GLOBAL_DEVICE, dstPool = dir != HYBM_GLOBAL_DEVICE_TO_LOCAL_DEVICE;
        Segment *seg = hbm_.get();
        auto poolOk = [&](uint64_t a, uint64_t len) {
            if (a < base || a >= end) return false;
            uint64_t rel = a - base;
            uint32_t r = (uint32_t)(rel / slot);
            const uint64_t mapped = seg->MappedBytes(r);
            return len <= mapped && rel - (uint64_t)r * slot <= mapped - len;  // no sum that a huge len could wrap
        };
        uint64_t total = 0;
        for (uint32_t i = 0; i < p.batchSize; i++) {
            uint64_t s = reinterpret_cast<uint64_t>(p.sources[i]), d = reinterpret_cast<uint64_t>(p.destinations[i]);
            uint64_t len = p.dataSizes[i];
            if (s == 0 || d == 0 || len == 0 || (srcPool && !poolOk(s, len)) || (dstPool && !poolOk(d, len)))
                return MF_FAIL(ERR_INVALID_PARAM, "batch copy item %u (%p -> %p, %lu bytes): null, empty or outside the mapped pool",
                               i, p.sources[i], p.destinations[i], (unsigned long)len);
            total += len;
        }
        KernelBatch kb(*ops_, stream, flags, total);
        if (kb.Ready()) {
            for (uint32_t i = 0; i < p.batchSize; i++)
                kb.Add(reinterpret_cast<uint64_t>(p.sources[i]), reinterpret_cast<uint64_t>(p.destinations[i]), p.dataSizes[i]);
            return kb.Finish();
        }
    }
    // General path: validate + resolve each item with arithmetic only (no map lookups, no locks).
    std::vector<ResolvedCopy> items;
    items.reserve(p.batchSize);
    int firstErr = OK;
    for (uint32_t i = 0; i < p.batchSize; i++) {
        ResolvedCopy c;
        c.index = i;
        c.len = p.dataSizes[i];
        int rc = (p.sources[i] == nullptr || p.destinations[i] == nullptr || c.len == 0) ? (int)ERR_INVALID_PARAM : (int)OK;
        if (rc == OK) rc = Resolve(reinterpret_cast<uint64_t>(p.sources[i]), c.len, true, dir, c.src);
        if (rc == OK) rc = Resolve(reinterpret_cast<uint64_t>(p.destinations[i]), c.len, false, dir, c.dst);
        if (perItem != nullptr) perItem[i] = rc;
        if (rc != OK) {
            if (firstErr == OK) firstErr = rc;
            if (perItem == nullptr)
                return MF_FAIL(rc, "batch copy item %u (%p -> %p, %lu bytes): address outside the mapped pool", i,
                               p.sources[i], p.destinations[i], (unsigned long)c.len);
            continue;
        }
        items.push_back(c);
    }
    int rc = ops_->Submit(items, stream, flags, perItem);
    return rc != OK ? rc : firstErr;
}

int Entity::PrepareBatch(const hybm_batch_copy_params &p, hybm_data_copy_direction dir, PreparedBatch &out)
{
    if (p.sources == nullptr || p.destinations == nullptr || p.dataSizes == nullptr || p.batchSize == 0)
        return MF_FAIL(ERR_INVALID_PARAM, "prepared batch: null array or empty batch");
    if (dir != HYBM_LOCAL_DEVICE_TO_GLOBAL_DEVICE && dir != HYBM_GLOBAL_DEVICE_TO_GLOBAL_DEVICE && dir != HYBM_GLOBAL_DEVICE_TO_LOCAL_DEVICE)
        return MF_FAIL(ERR_INVALID_PARAM, "prepared batch: device-to-device directions only (L2G, G2G, G2L)");
    if (dev_ == nullptr || !dev_->Caps().present) return MF_FAIL(ERR_NOT_INIT, "prepared batch: no device");
    const uint64_t gen = mapGen_.load();
    std::vector<ResolvedCopy> items(p.batchSize);
    for (uint32_t i = 0; i < p.batchSize; i++) {
        ResolvedCopy &c = items[i];
        c.index = i;
        c.len = p.dataSizes[i];
        int rc = (p.sources[i] == nullptr || p.destinations[i] == nullptr || c.len == 0) ? (int)ERR_INVALID_PARAM : (int)OK;
        if (rc == OK) rc = Resolve(reinterpret_cast<uint64_t>(p.sources[i]), c.len, true, dir, c.src);
        if (rc == OK) rc = Resolve(reinterpret_cast<uint64_t>(p.destinations[i]), c.len, false, dir, c.dst);
        if (rc != OK)
            return MF_FAIL(rc, "prepared batch item %u (%p -> %p, %lu bytes): null, empty or outside the mapped pool", i, p.sources[i],
                           p.destinations[i], (unsigned long)c.len);
    }
    int rc = ops_->Prepare(items, out);
    if (rc == OK) out.mapGen = gen;
    return rc;
}

int Entity::LaunchPrepared(const PreparedBatch &b, void *stream)
{
    // a member left (its slice is unmapped) since the batch was validated: the descriptors may name memory that is gone
    if (b.mapGen != mapGen_.load()) return MF_FAIL(ERR_NOT_CONNECTED, "prepared batch is stale: the pool's membership changed since it was built");
    return ops_->LaunchPrepared(b, stream);
}

int Entity::QuantCopy(const hybm_quant_copy_params &p, int mode)
{
    if (p.sources == nullptr || p.destinations == nullptr || p.dataSizes == nullptr || p.scale == nullptr || p.batchSize == 0 ||
        p.unitNum == 0 || p.unitNum > 32768)
        return MF_FAIL(ERR_INVALID_PARAM, "quant copy: null array, empty batch or unit %u out of (0, 32768]", p.unitNum);
    std::vector<QuantItem> items(p.batchSize);
    // An address inside a pool window must lie in a mapped slice for the whole range the kernel touches:
    // elems * 2 bytes read, elems bytes written, one float per unit written. Addresses outside every
    // window (the caller's own device buffers) are taken as given, as in the copy paths.
    auto pooled = [&](uint64_t addr, uint64_t len, const char *what, uint32_t i) -> int {
        int err = OK;
        if ((dram_ && dram_->Compact() && InPool(dram_, addr, len, err)) || (hbm_ && hbm_->Compact() && InPool(hbm_, addr, len, err)))
            return MF_FAIL(ERR_INVALID_PARAM, "quant copy item %u: %s %#lx is a 56-bit pool address, which the quantising copy does not translate", i, what,
                           (unsigned long)addr);
        if ((InPool(hbm_, addr, len, err) || InPool(dram_, addr, len, err)) && err != OK)
            return MF_FAIL(err, "quant copy item %u: %s %#lx (+%lu bytes) %s", i, what, (unsigned long)addr, (unsigned long)len,
                           err == ERR_NOT_CONNECTED ? "lies in the slice of a rank that is not mapped here" : "runs past the mapped part of the pool");
        return OK;
    };
    for (uint32_t i = 0; i < p.batchSize; i++) {
        if (p.sources[i] == nullptr || p.destinations[i] == nullptr || p.scale[i] == nullptr || (p.dataSizes[i] & 1))
            return MF_FAIL(ERR_INVALID_PARAM, "quant copy item %u: null address or odd byte count", i);
        const uint64_t elems = p.dataSizes[i] / 2;
        const uint64_t units = (elems + p.unitNum - 1) / p.unitNum;
        int rc = pooled(reinterpret_cast<uint64_t>(p.sources[i]), p.dataSizes[i], "source", i);
        if (rc == OK) rc = pooled(reinterpret_cast<uint64_t>(p.destinations[i]), elems, "destination", i);
        if (rc == OK) rc = pooled(reinterpret_cast<uint64_t>(p.scale[i]), units * sizeof(float), "factor array", i);
        if (rc != OK) return rc;
        items[i] = QuantItem{reinterpret_cast<uint64_t>(p.sources[i]), reinterpret_cast<uint64_t>(p.destinations[i]),
                             reinterpret_cast<uint64_t>(p.scale[i]), p.dataSizes[i] / 2};
    }
    return ops_->Quant(items, p.unitNum, p.inputType == 1, mode, p.stream);
}

int Entity::Wait() { return ops_->Wait(); }

}  // namespace hybm
}  // namespace mf
