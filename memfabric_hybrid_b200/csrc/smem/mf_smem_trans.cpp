// smem_trans_*: point-to-point transfers between processes named by "ip:port[_pid]" strings (KV-cache
// hand-off between prefill and decode instances). Each process joins one dynamic group through the
// store (auto-ranked), publishes its identity and its registered buffers; peers import those buffers
// (CUDA IPC mapping for device memory, process_vm for host memory) and address them by the OWNER's
// local addresses, which this layer translates.
//   store keys under "TRANS_": ID_<uniqueId> -> {rank, role}, RK_<rank> -> uniqueId,
//                              MR_<rank> -> packed exchange blobs of every registered buffer
// Parity: src/smem/csrc/smem_trans/smem_trans_entry_manager.cpp:31-77,
// smem_trans_entry.cpp:75-122,230-449,515-692,773-858, src/smem/include/host/smem_trans.h:30-252.
#include <unistd.h>

#include "../include/smem_trans.h"
#include "../util/mf_trace.h"
#include "mf_smem_common.h"

using namespace mf;
using namespace mf::smem;
using namespace mf::hybm;

namespace {

#pragma pack(push, 1)
struct IdRecord {
    uint32_t rank;
    uint32_t role;
    int32_t pid;
};
#pragma pack(pop)

struct TransGlobals {
    smem_trans_config_t config{};
    bool inited = false;
};
std::mutex g_mu;
TransGlobals g_trans;

class TransEntry : public std::enable_shared_from_this<TransEntry> {
public:
    TransEntry(std::string url, std::string uid, const smem_trans_config_t &cfg) : url_(std::move(url)), uid_(std::move(uid)), cfg_(cfg) {}
    ~TransEntry() { Close(); }

    int Initialize()
    {
        int err = OK;
        base_ = store::StoreFactory::CreateStore(url_, false, SMEM_TRANS_RANK_COUNT_MAX, store::kAutoRank,
                                                 1000u * cfg_.initTimeout, 0, &err);
        if (!base_) return MF_FAIL(err, "trans %s: cannot reach the config store at %s", uid_.c_str(), url_.c_str());
        int rc = base_->AutoRank(rank_);
        if (rc != OK) return rc;
        store_ = store::StoreFactory::Prefixed(base_, "TRANS_");
        hybm_options ho{};
        ho.bmType = HYBM_TYPE_HOST_INITIATE;
        ho.memType = (hybm_mem_type)0;
        ho.bmDataOpType = (hybm_data_op_type)(HYBM_DOP_TYPE_SDMA | HYBM_DOP_TYPE_MTE);
        ho.rankCount = SMEM_TRANS_RANK_COUNT_MAX;
        ho.rankId = rank_;
        ho.devId = (uint16_t)cfg_.deviceId;
        ho.scene = HYBM_SCENE_TRANS;
        ho.role = cfg_.role == SMEM_TRANS_SENDER ? HYBM_ROLE_SENDER : (cfg_.role == SMEM_TRANS_RECEIVER ? HYBM_ROLE_RECEIVER : HYBM_ROLE_PEER);
        ho.dramShmFd = -1;
        entity_ = Entity::Create(0, ho);
        if (!entity_) return LastError::Code() != 0 ? LastError::Code() : (int)ERR;
        IdRecord me{rank_, (uint32_t)cfg_.role, (int32_t)getpid()};
        rc = store_->Set("ID_" + uid_, std::string(reinterpret_cast<const char *>(&me), sizeof(me)));
        if (rc == OK) rc = store_->Set("RK_" + std::to_string(rank_), uid_);
        if (rc != OK) return rc;
        group::GroupOption go;
        go.rankSize = SMEM_TRANS_RANK_COUNT_MAX;
        go.rank = rank_;
        go.timeoutMs = 1000ULL * cfg_.initTimeout;
        go.dynamic = true;
        std::weak_ptr<TransEntry> weak = weak_from_this();
        go.joinCb = [](uint32_t) { return OK; };  // buffers are imported on demand
        go.updateCb = [weak](uint32_t r) {
            auto s = weak.lock();
            if (s && r != s->rank_) s->RefreshPeer(r, false);
            return OK;
        };
        go.leaveCb = [weak](uint32_t r) {
            auto s = weak.lock();
            if (s && r != s->rank_) s->DropPeer(r, false);
            return OK;
        };
        go.linkDownCb = [weak](uint32_t r) {
            auto s = weak.lock();
            if (s) s->DropPeer(r, true);
            return OK;
        };
        group_ = group::GroupEngine::Create(store_, go);
        if (!group_) return ERR_INVALID_PARAM;
        // A store that restarted (a new leader after the old one died) has lost this endpoint's identity and the records
        // of its registered buffers: peers that look it up from then on need them again.
        store_->RegisterReconnectHandler([weak]() -> int {
            auto s = weak.lock();
            if (!s || s->closed_.load()) return OK;
            IdRecord me{s->rank_, (uint32_t)s->cfg_.role, (int32_t)getpid()};
            int rc = s->store_->Set("ID_" + s->uid_, std::string(reinterpret_cast<const char *>(&me), sizeof(me)));
            if (rc == OK) rc = s->store_->Set("RK_" + std::to_string(s->rank_), s->uid_);
            std::lock_guard<std::mutex> g(s->mu_);
            return rc == OK ? s->PublishLocked() : rc;
        });
        rc = group_->Join();
        return rc;
    }

    void Close()
    {
        if (closed_.exchange(true)) return;
        if (group_ && group_->Joined()) group_->Leave();
        if (group_) group_->StopListen();
        if (store_) {
            store_->Remove("ID_" + uid_, true);
            store_->Remove("RK_" + std::to_string(rank_), true);
            store_->Remove("MR_" + std::to_string(rank_), true);
        }
        entity_.reset();
        group_.reset();
        store_.reset();
        if (base_) store::StoreFactory::DestroyStore(url_);
        base_.reset();
    }

    int Register(void *const *addrs, const size_t *caps, uint32_t count)
    {
        MF_TRACE_BEGIN(TP_TRANS_REGISTER);
        int rc = OK;
        {
            std::lock_guard<std::mutex> g(mu_);
            for (uint32_t i = 0; i < count && rc == OK; i++) {
                uint64_t a = reinterpret_cast<uint64_t>(addrs[i]);
                if (a == 0 || caps[i] == 0) {
                    rc = MF_FAIL(ERR_INVALID_PARAM, "register: null address or zero capacity at %u", i);
                    break;
                }
                if (regs_.count(a)) continue;
                MemSlice *s = nullptr;
                rc = entity_->RegisterLocal(addrs[i], caps[i], 0, &s);
                if (rc == OK) regs_[a] = s;
            }
            if (rc == OK) rc = PublishLocked();
        }
        if (rc == OK) rc = group_->Update();
        MF_TRACE_END(TP_TRANS_REGISTER, rc);
        return rc;
    }

    int Deregister(void *addr)
    {
        uint64_t a = reinterpret_cast<uint64_t>(addr);
        int rc;
        {
            std::lock_guard<std::mutex> g(mu_);
            auto it = regs_.find(a);
            if (it == regs_.end()) return MF_FAIL(ERR_NOT_EXIST, "address %p was not registered", addr);
            entity_->UnregisterLocal(a);
            regs_.erase(it);
            rc = PublishLocked();
        }
        if (rc == OK) rc = group_->Update();
        return rc;
    }

    // dir: true = write local -> remote, false = read remote -> local
    int Transfer(bool write, void *const *locals, const char *remoteUid, void *const *remotes, const size_t *sizes,
                 uint32_t count, void *stream, bool submitOnly)
    {
        if (remoteUid == nullptr || locals == nullptr || remotes == nullptr || sizes == nullptr || count == 0)
            return MF_FAIL(ERR_INVALID_PARAM, "transfer: null argument or empty batch");
        IdRecord peer{};
        int rc = LookupPeer(remoteUid, peer);
        if (rc != OK) return rc;
        if (cfg_.role == SMEM_TRANS_RECEIVER && write) return MF_FAIL(ERR_INVALID_PARAM, "a RECEIVER cannot write");
        std::vector<ResolvedCopy> items(count);
        auto *dev = entity_->Device();
        for (uint32_t i = 0; i < count; i++) {
            uint64_t l = reinterpret_cast<uint64_t>(locals[i]), r = reinterpret_cast<uint64_t>(remotes[i]);
            if (l == 0 || r == 0 || sizes[i] == 0) return MF_FAIL(ERR_INVALID_PARAM, "transfer item %u: null address or zero size", i);
            RemoteRegion reg;
            uint64_t mapped = 0;
            rc = entity_->TranslateRemote(peer.rank, r, sizes[i], reg, mapped);
            if (rc != OK) {  // unknown or not yet mapped: fetch the peer's current registrations once
                RefreshPeer(peer.rank, true);
                rc = entity_->TranslateRemote(peer.rank, r, sizes[i], reg, mapped);
            }
            if (rc != OK)
                return MF_FAIL(ERR_INVALID_PARAM, "transfer item %u: %p (+%zu) is not inside a buffer registered by %s", i,
                               remotes[i], sizes[i], remoteUid);
            Endpoint le, re;
            le.addr = l;
            uint8_t cls = VaManager::Get().Classify(l, sizes[i]);
            le.kind = cls == AC_LD ? EP_DEVICE : (cls == AC_LH ? EP_HOST : ((dev != nullptr && dev->IsDevicePointer(l)) ? EP_DEVICE : EP_HOST));
            if (reg.device) {
                re.addr = mapped;
                re.kind = EP_DEVICE;
            } else {
                re.addr = r;
                re.kind = EP_REMOTE_VM;
                re.pid = reg.pid;
            }
            items[i].index = i;
            items[i].len = sizes[i];
            items[i].src = write ? le : re;
            items[i].dst = write ? re : le;
        }
        uint32_t flags = submitOnly ? (ASYNC_COPY_FLAG | SMEM_BM_FLAG_USE_EXTERNAL_STREAM) : 0;
        return entity_->SubmitResolved(items, stream, flags);
    }

    int QuantWrite(const smem_trans_quant_copy_param_t &p)
    {
        if (p.remoteUniqueId == nullptr || p.localAddrs == nullptr || p.remoteAddrs == nullptr || p.dataSizes == nullptr ||
            p.scale == nullptr || p.batchSize == 0 || p.unitNum == 0 || p.unitNum > 32768)
            return MF_FAIL(ERR_INVALID_PARAM, "quant write: null argument, empty batch or unit out of (0, 32768]");
        IdRecord peer{};
        int rc = LookupPeer(p.remoteUniqueId, peer);
        if (rc != OK) return rc;
        std::vector<QuantItem> items(p.batchSize);
        for (uint32_t i = 0; i < p.batchSize; i++) {
            uint64_t elems = p.dataSizes[i] / 2;
            uint64_t units = (elems + p.unitNum - 1) / p.unitNum;
            RemoteRegion reg;
            uint64_t dst = 0, sc = 0;
            for (int pass = 0; pass < 2; pass++) {
                rc = entity_->TranslateRemote(peer.rank, reinterpret_cast<uint64_t>(p.remoteAddrs[i]), elems, reg, dst);
                if (rc == OK && !reg.device) rc = ERR_INVALID_PARAM;
                if (rc == OK) rc = entity_->TranslateRemote(peer.rank, reinterpret_cast<uint64_t>(p.scale[i]), units * 4, reg, sc);
                if (rc == OK && !reg.device) rc = ERR_INVALID_PARAM;
                if (rc == OK || pass == 1) break;
                RefreshPeer(peer.rank, true);
            }
            if (rc != OK) return MF_FAIL(ERR_INVALID_PARAM, "quant write item %u: destination or scale is not a registered device buffer of %s", i, p.remoteUniqueId);
            items[i] = QuantItem{reinterpret_cast<uint64_t>(p.localAddrs[i]), dst, sc, elems};
        }
        return entity_->SubmitQuant(items, p.unitNum, p.inputType == 1, (p.flags & SMEM_TRANS_QUANT_FP8_E4M3) ? 1 : 0, p.stream);
    }

    void SetPeerDown(smem_trans_peer_down_callback_t cb, void *ud)
    {
        std::lock_guard<std::mutex> g(mu_);
        downCb_ = cb;
        downCtx_ = ud;
    }

    uint32_t Rank() const { return rank_; }

private:
    int PublishLocked()
    {
        std::vector<hybm_exchange_info> v(1 + regs_.size());
        int rc = entity_->Export(nullptr, &v[0]);
        size_t i = 1;
        for (auto &kv : regs_) {
            if (rc != OK) break;
            rc = entity_->Export(kv.second, &v[i++]);
        }
        if (rc != OK) return rc;
        return store_->Set("MR_" + std::to_string(rank_), PackInfos(v));
    }

    int LookupPeer(const std::string &uid, IdRecord &out)
    {
        {
            std::lock_guard<std::mutex> g(mu_);
            auto it = peers_.find(uid);
            if (it != peers_.end()) {
                out = it->second;
                return OK;
            }
        }
        std::string v;
        int rc = store_->Get("ID_" + uid, v, 0);
        if (rc != OK || v.size() != sizeof(IdRecord)) return MF_FAIL(ERR_NOT_EXIST, "no transfer endpoint named %s is registered", uid.c_str());
        memcpy(&out, v.data(), sizeof(out));
        std::lock_guard<std::mutex> g(mu_);
        peers_[uid] = out;
        rankNames_[out.rank] = uid;
        return OK;
    }

    bool Opposite(uint32_t otherRole) const
    {
        if (cfg_.role == SMEM_TRANS_BOTH || otherRole == SMEM_TRANS_BOTH) return true;
        return (cfg_.role == SMEM_TRANS_SENDER && otherRole == SMEM_TRANS_RECEIVER) ||
               (cfg_.role == SMEM_TRANS_RECEIVER && otherRole == SMEM_TRANS_SENDER);
    }

    void RefreshPeer(uint32_t rank, bool force)
    {
        if (!force) {
            // eager import only for peers of the opposite role that we already talk to
            std::lock_guard<std::mutex> g(mu_);
            auto it = rankNames_.find(rank);
            if (it == rankNames_.end()) return;
            if (!Opposite(peers_[it->second].role)) return;
        }
        std::string blob;
        if (store_->Get("MR_" + std::to_string(rank), blob, 0) != OK) return;
        std::vector<hybm_exchange_info> infos;
        if (!UnpackInfos(blob, infos)) return;
        if (entity_->Import(infos.data(), (uint32_t)infos.size(), nullptr) == OK) entity_->Mmap();
    }

    void DropPeer(uint32_t rank, bool linkDown)
    {
        std::string name;
        smem_trans_peer_down_callback_t cb;
        void *ctx;
        {
            std::lock_guard<std::mutex> g(mu_);
            auto it = rankNames_.find(rank);
            if (it != rankNames_.end()) {
                name = it->second;
                peers_.erase(name);
                rankNames_.erase(it);
            }
            cb = downCb_;
            ctx = downCtx_;
        }
        entity_->RemoveImported(rank);
        if (linkDown) {
            // the dead process cannot clean its own records
            store_->Remove("MR_" + std::to_string(rank), true);
            std::string uid;
            if (name.empty() && store_->Get("RK_" + std::to_string(rank), uid, 0) == OK) name = uid;
            if (!name.empty()) store_->Remove("ID_" + name, true);
            store_->Remove("RK_" + std::to_string(rank), true);
        }
        if (cb != nullptr && !name.empty()) cb(name.c_str(), ctx);
    }

    std::string url_, uid_;
    smem_trans_config_t cfg_;
    store::StorePtr base_, store_;
    uint32_t rank_ = 0;
    EntityPtr entity_;
    group::GroupPtr group_;
    std::mutex mu_;
    std::map<uint64_t, MemSlice *> regs_;
    std::map<std::string, IdRecord> peers_;
    std::map<uint32_t, std::string> rankNames_;
    smem_trans_peer_down_callback_t downCb_ = nullptr;
    void *downCtx_ = nullptr;
    std::atomic<bool> closed_{false};
};

// leaked on purpose: tearing pools down from static destructors would call into a CUDA driver that
// is already shutting down
HandleTable<TransEntry> &g_handles = *new HandleTable<TransEntry>();

std::shared_ptr<TransEntry> H(smem_trans_t h)
{
    if (h == nullptr) {
        MF_FAIL(SMEM_INVALID_PARAM, "handle is NULL");
        return nullptr;
    }
    auto e = g_handles.Find(h);
    if (!e) MF_FAIL(SMEM_INVALID_PARAM, "handle %p is not a live transfer object", h);
    return e;
}
}  // namespace

extern "C" {

int32_t smem_trans_config_init(smem_trans_config_t *config)
{
    if (config == nullptr) return MF_FAIL(SMEM_INVALID_PARAM, "config is NULL");
    config->role = SMEM_TRANS_BOTH;
    config->initTimeout = kDefaultTimeoutSec;
    config->deviceId = 0;
    config->flags = 0;
    config->dataOpType = SMEMB_DATA_OP_SDMA;
    return SMEM_OK;
}

int32_t smem_trans_init(const smem_trans_config_t *config)
{
    if (config == nullptr) return MF_FAIL(SMEM_INVALID_PARAM, "config is NULL");
    if (!SmemInited()) return MF_FAIL(SMEM_NOT_INIT, "smem_init has not been called");
    std::lock_guard<std::mutex> g(g_mu);
    if (g_trans.inited) return SMEM_OK;
    int rc = HybmInit((uint16_t)config->deviceId, 0);
    if (rc != OK) return Pub(rc);
    g_trans.config = *config;
    g_trans.inited = true;
    return SMEM_OK;
}

void smem_trans_uninit(uint32_t)
{
    std::lock_guard<std::mutex> g(g_mu);
    if (!g_trans.inited) return;
    for (auto &e : g_handles.TakeAll()) e->Close();
    HybmUninit();
    g_trans = TransGlobals();
}

smem_trans_t smem_trans_create(const char *storeUrl, const char *uniqueId, const smem_trans_config_t *config)
{
    if (storeUrl == nullptr || uniqueId == nullptr || *uniqueId == 0 || config == nullptr) {
        MF_FAIL(SMEM_INVALID_PARAM, "trans create: null argument");
        return nullptr;
    }
    if (config->role <= SMEM_TRANS_NONE || config->role >= SMEM_TRANS_BUTT || config->initTimeout == 0) {
        MF_FAIL(SMEM_INVALID_PARAM, "trans create: bad role %d or zero timeout", (int)config->role);
        return nullptr;
    }
    {
        std::lock_guard<std::mutex> g(g_mu);
        if (!g_trans.inited) {
            MF_FAIL(SMEM_NOT_INIT, "smem_trans_init has not been called");
            return nullptr;
        }
    }
    auto e = std::make_shared<TransEntry>(storeUrl, uniqueId, *config);
    int rc = e->Initialize();
    if (rc != OK) {
        if (LastError::Code() == 0) LastError::Set(Pub(rc), "trans %s: create failed with %d", uniqueId, rc);
        e->Close();
        return nullptr;
    }
    return g_handles.Add(e);
}

void smem_trans_destroy(smem_trans_t handle, uint32_t)
{
    auto e = g_handles.Take(handle);
    if (e) e->Close();
}

int32_t smem_trans_register_mem(smem_trans_t handle, void *address, size_t capacity, uint32_t)
{
    auto e = H(handle);
    return e ? Pub(e->Register(&address, &capacity, 1)) : SMEM_INVALID_PARAM;
}

int32_t smem_trans_batch_register_mem(smem_trans_t handle, void *addresses[], size_t capacities[], uint32_t count, uint32_t)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    if (addresses == nullptr || capacities == nullptr || count == 0) return MF_FAIL(SMEM_INVALID_PARAM, "batch register: null array or empty");
    return Pub(e->Register(addresses, capacities, count));
}

int32_t smem_trans_deregister_mem(smem_trans_t handle, void *address)
{
    auto e = H(handle);
    return e ? Pub(e->Deregister(address)) : SMEM_INVALID_PARAM;
}

int32_t smem_trans_write(smem_trans_t handle, const void *localAddr, const char *remoteUniqueId, void *remoteAddr,
                         size_t dataSize, uint32_t)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    void *l = const_cast<void *>(localAddr);
    MF_TRACE_BEGIN(TP_TRANS_BATCH_WRITE);
    int rc = e->Transfer(true, &l, remoteUniqueId, &remoteAddr, &dataSize, 1, nullptr, false);
    MF_TRACE_END(TP_TRANS_BATCH_WRITE, rc);
    return Pub(rc);
}

int32_t smem_trans_batch_write(smem_trans_t handle, const void *localAddrs[], const char *remoteUniqueId,
                               void *remoteAddrs[], size_t dataSizes[], uint32_t batchSize, uint32_t)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    MF_TRACE_BEGIN(TP_TRANS_BATCH_WRITE);
    int rc = e->Transfer(true, const_cast<void *const *>(localAddrs), remoteUniqueId, remoteAddrs, dataSizes, batchSize, nullptr, false);
    MF_TRACE_END(TP_TRANS_BATCH_WRITE, rc);
    return Pub(rc);
}

int32_t smem_trans_read(smem_trans_t handle, void *localAddr, const char *remoteUniqueId, const void *remoteAddr,
                        size_t dataSize, uint32_t)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    void *r = const_cast<void *>(remoteAddr);
    MF_TRACE_BEGIN(TP_TRANS_BATCH_READ);
    int rc = e->Transfer(false, &localAddr, remoteUniqueId, &r, &dataSize, 1, nullptr, false);
    MF_TRACE_END(TP_TRANS_BATCH_READ, rc);
    return Pub(rc);
}

int32_t smem_trans_batch_read(smem_trans_t handle, void *localAddrs[], const char *remoteUniqueId,
                              const void *remoteAddrs[], size_t dataSizes[], uint32_t batchSize, uint32_t)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    MF_TRACE_BEGIN(TP_TRANS_BATCH_READ);
    int rc = e->Transfer(false, localAddrs, remoteUniqueId, const_cast<void *const *>(remoteAddrs), dataSizes, batchSize, nullptr, false);
    MF_TRACE_END(TP_TRANS_BATCH_READ, rc);
    return Pub(rc);
}

int32_t smem_trans_read_submit(smem_trans_t handle, void *localAddr, const char *remoteUniqueId, const void *remoteAddr,
                               size_t dataSize, void *stream, uint32_t)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    void *r = const_cast<void *>(remoteAddr);
    return Pub(e->Transfer(false, &localAddr, remoteUniqueId, &r, &dataSize, 1, stream, stream != nullptr));
}

int32_t smem_trans_write_submit(smem_trans_t handle, const void *localAddr, const char *remoteUniqueId,
                                void *remoteAddr, size_t dataSize, void *stream, uint32_t)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    void *l = const_cast<void *>(localAddr);
    return Pub(e->Transfer(true, &l, remoteUniqueId, &remoteAddr, &dataSize, 1, stream, stream != nullptr));
}

int32_t smem_trans_batch_read_submit(smem_trans_t handle, void *localAddrs[], const char *remoteUniqueId,
                                     const void *remoteAddrs[], size_t dataSizes[], uint32_t batchSize, void *stream, uint32_t)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    return Pub(e->Transfer(false, localAddrs, remoteUniqueId, const_cast<void *const *>(remoteAddrs), dataSizes, batchSize, stream, stream != nullptr));
}

int32_t smem_trans_batch_write_submit(smem_trans_t handle, const void *localAddrs[], const char *remoteUniqueId,
                                      void *remoteAddrs[], size_t dataSizes[], uint32_t batchSize, void *stream, uint32_t)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    return Pub(e->Transfer(true, const_cast<void *const *>(localAddrs), remoteUniqueId, remoteAddrs, dataSizes, batchSize, stream, stream != nullptr));
}

int32_t smem_trans_batch_quant_write(smem_trans_t handle, smem_trans_quant_copy_param_t *params)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    if (params == nullptr) return MF_FAIL(SMEM_INVALID_PARAM, "params is NULL");
    return Pub(e->QuantWrite(*params));
}

int32_t smem_trans_set_peer_down_callback(smem_trans_t handle, smem_trans_peer_down_callback_t callback, void *userData)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    e->SetPeerDown(callback, userData);
    return SMEM_OK;
}

}  // extern "C"
