// C entry points over the internal C++ classes (config store client/server, HA store, group engine,
// trace table, fault points), so that their behaviour can be driven from scripts and tests without
// going through a whole memory-pool bring-up. Handles are opaque pointers owned by the caller and
// released with the matching *_free call. Every function is prefixed mf_t_.
#include <cstring>
#include <memory>
#include <thread>

#include "../net/mf_tls.h"
#include "../group/mf_group.h"
#include "../hybm/mf_entity.h"
#include "../store/mf_store.h"
#include "../store/mf_store_backend.h"
#include "../store/mf_store_etcd.h"
#include "../store/mf_store_ha.h"
#include "../util/mf_trace.h"
#include "../util/mf_util.h"

using namespace mf;
using namespace mf::store;

namespace {

struct StoreBox {
    StorePtr s;
    std::shared_ptr<TcpStoreClient> tcp;
    std::shared_ptr<HaConfigStore> ha;
};
struct ServerBox {
    std::shared_ptr<StoreServer> srv;
};
struct GroupBox {
    std::shared_ptr<group::GroupEngine> g;
};

int CopyOut(const std::string &v, char *buf, int cap)
{
    if (buf != nullptr && cap > 0) {
        const size_t n = std::min<size_t>(v.size(), (size_t)cap);
        memcpy(buf, v.data(), n);
    }
    return (int)v.size();
}

}  // namespace

extern "C" {

// ---- server ---------------------------------------------------------------------------------------
void *mf_t_server_start(const char *ip, uint16_t port, uint32_t world, uint64_t flags, int *rc)
{
    auto b = new ServerBox{std::make_shared<StoreServer>(ip, port, world, flags)};
    int r = b->srv->Startup();
    if (rc != nullptr) *rc = r;
    if (r != OK) {
        delete b;
        return nullptr;
    }
    return b;
}
void mf_t_server_stop(void *h)
{
    auto b = static_cast<ServerBox *>(h);
    if (b == nullptr) return;
    b->srv->Shutdown();
    delete b;
}
uint64_t mf_t_server_keys(void *h) { return static_cast<ServerBox *>(h)->srv->KeyCount(); }
int mf_t_server_state(void *h) { return (int)static_cast<ServerBox *>(h)->srv->GetState(); }
uint16_t mf_t_server_port(void *h) { return static_cast<ServerBox *>(h)->srv->Port(); }
// persistence of world size / alive ranks in a named in-memory backend (shared by name inside the process)
void mf_t_server_set_backend(void *h, const char *backendName, int firstLeader)
{
    static_cast<ServerBox *>(h)->srv->SetBackend(std::make_shared<LocalMemoryBackend>(backendName, true), firstLeader != 0);
}

// ---- client ---------------------------------------------------------------------------------------
void *mf_t_client_new(const char *ip, uint16_t port, uint32_t world, uint32_t rank, uint32_t timeoutMs, int *rc)
{
    auto c = std::make_shared<TcpStoreClient>(ip, port, world, rank);
    int r = c->Startup(timeoutMs);
    if (rc != nullptr) *rc = r;
    if (r != OK) return nullptr;
    return new StoreBox{c, c, nullptr};
}
void *mf_t_store_prefixed(void *h, const char *prefix)
{
    auto b = static_cast<StoreBox *>(h);
    return new StoreBox{StoreFactory::Prefixed(b->s, prefix), nullptr, nullptr};
}
void mf_t_store_free(void *h)
{
    auto b = static_cast<StoreBox *>(h);
    if (b == nullptr) return;
    if (b->tcp) b->tcp->Shutdown();
    if (b->ha) b->ha->Shutdown();
    delete b;
}
void mf_t_client_crash(void *h)
{
    auto b = static_cast<StoreBox *>(h);
    if (b->tcp) b->tcp->SimulateCrash();
}
void mf_t_client_set_reconnect(void *h, uint32_t tries, uint32_t intervalMs)
{
    auto b = static_cast<StoreBox *>(h);
    if (b->tcp) b->tcp->SetReconnectPolicy(tries, intervalMs);
}
int mf_t_store_connected(void *h) { return static_cast<StoreBox *>(h)->s->Connected() ? 1 : 0; }
uint32_t mf_t_store_rank(void *h) { return static_cast<StoreBox *>(h)->s->Rank(); }

int mf_t_store_set(void *h, const char *key, const void *val, int len)
{
    return static_cast<StoreBox *>(h)->s->Set(key, std::string(static_cast<const char *>(val), (size_t)len));
}
// returns the value's size (>= 0) or a negative error code
int mf_t_store_get(void *h, const char *key, char *buf, int cap, int64_t timeoutMs)
{
    std::string v;
    int rc = static_cast<StoreBox *>(h)->s->Get(key, v, timeoutMs);
    if (rc != OK) return rc < 0 ? rc : -1;
    return CopyOut(v, buf, cap);
}
int mf_t_store_add(void *h, const char *key, int64_t inc, int64_t *result) { return static_cast<StoreBox *>(h)->s->Add(key, inc, *result); }
int mf_t_store_remove(void *h, const char *key, int quiet) { return static_cast<StoreBox *>(h)->s->Remove(key, quiet != 0); }
int mf_t_store_append(void *h, const char *key, const void *val, int len, uint64_t *newSize)
{
    return static_cast<StoreBox *>(h)->s->Append(key, std::string(static_cast<const char *>(val), (size_t)len), *newSize);
}
// existing (when the swap lost) is copied to buf; *existingLen receives its size
int mf_t_store_cas(void *h, const char *key, const void *expect, int elen, const void *desired, int dlen, char *buf, int cap, int *existingLen)
{
    std::string ex;
    int rc = static_cast<StoreBox *>(h)->s->Cas(key, std::string(static_cast<const char *>(expect), (size_t)elen),
                                                  std::string(static_cast<const char *>(desired), (size_t)dlen), ex);
    if (existingLen != nullptr) *existingLen = CopyOut(ex, buf, cap);
    return rc;
}
int mf_t_store_write(void *h, const char *key, uint32_t off, const void *val, int len)
{
    return static_cast<StoreBox *>(h)->s->Write(key, off, std::string(static_cast<const char *>(val), (size_t)len));
}
// keys come back '\n'-joined in buf; returns the number of keys or a negative error code
int mf_t_store_prefix_get(void *h, const char *prefix, char *buf, int cap)
{
    std::vector<std::string> ks, vs;
    int rc = static_cast<StoreBox *>(h)->s->PrefixGet(prefix, ks, vs);
    if (rc != OK) return rc < 0 ? rc : -1;
    std::string joined;
    for (auto &k : ks) joined += k + "\n";
    if (buf != nullptr && cap > 0) {
        const size_t n = std::min<size_t>(joined.size(), (size_t)cap - 1);
        memcpy(buf, joined.data(), n);
        buf[n] = 0;
    }
    return (int)ks.size();
}
typedef void (*mf_t_watch_cb)(int result, const char *key, const char *value, int valueLen);
int mf_t_store_watch(void *h, const char *key, mf_t_watch_cb cb, uint32_t *id)
{
    return static_cast<StoreBox *>(h)->s->Watch(
        key, [cb](int rc, const std::string &k, const std::string &v) { cb(rc, k.c_str(), v.data(), (int)v.size()); }, *id);
}
int mf_t_store_unwatch(void *h, uint32_t id) { return static_cast<StoreBox *>(h)->s->Unwatch(id); }
typedef void (*mf_t_rank_cb)(uint32_t rank);
int mf_t_store_watch_rank(void *h, mf_t_rank_cb cb, uint32_t *id)
{
    return static_cast<StoreBox *>(h)->s->WatchRankState([cb](uint32_t r) { cb(r); }, *id);
}
int mf_t_store_query_alive(void *h, uint32_t rank, int *alive)
{
    bool a = false;
    int rc = static_cast<StoreBox *>(h)->s->QueryAlive(rank, a);
    *alive = a ? 1 : 0;
    return rc;
}
int mf_t_store_auto_rank(void *h, uint32_t *rank) { return static_cast<StoreBox *>(h)->s->AutoRank(*rank); }

// ---- highly available store -------------------------------------------------------------------------
void *mf_t_ha_new(const char *ip, uint16_t basePort, uint32_t world, uint32_t rank, const char *backendName, int candidate)
{
    auto be = std::make_shared<LocalMemoryBackend>(backendName, true);
    auto ha = std::make_shared<HaConfigStore>(ip, basePort, world, rank, be, candidate != 0);
    return new StoreBox{ha, nullptr, ha};
}
void mf_t_ha_set_timings(void *h, uint32_t leaseMs, uint32_t healthMs, uint32_t lo, uint32_t hi)
{
    static_cast<StoreBox *>(h)->ha->SetTimings(leaseMs, healthMs, lo, hi);
}
int mf_t_ha_start(void *h, uint32_t timeoutMs) { return static_cast<StoreBox *>(h)->ha->Startup(timeoutMs); }
int mf_t_ha_is_leader(void *h) { return static_cast<StoreBox *>(h)->ha->IsLeader() ? 1 : 0; }
int mf_t_ha_leader_addr(void *h, char *buf, int cap)
{
    std::string a = static_cast<StoreBox *>(h)->ha->LeaderAddress();
    int n = CopyOut(a, buf, cap - 1);
    if (buf != nullptr && cap > 0) buf[std::min(n, cap - 1)] = 0;
    return n;
}
void mf_t_ha_kill_leader(void *h) { static_cast<StoreBox *>(h)->ha->KillLeaderServer(); }
// the same store on an etcd backend (native v3 client)
void *mf_t_ha_new_etcd(const char *ip, uint16_t basePort, uint32_t world, uint32_t rank, const char *etcdIp, uint16_t etcdPort,
                       const char *instance, int candidate)
{
    auto be = std::make_shared<EtcdBackend>(etcdIp, etcdPort, instance ? instance : "");
    auto ha = std::make_shared<HaConfigStore>(ip, basePort, world, rank, be, candidate != 0);
    return new StoreBox{ha, nullptr, ha};
}
// ---- etcd backend on its own ----------------------------------------------------------------------------
void *mf_t_etcd_new(const char *ip, uint16_t port, const char *instance, const char *user, const char *password, uint32_t timeoutMs)
{
    auto *b = new EtcdBackend(ip, port, instance ? instance : "", user ? user : "", password ? password : "");
    if (timeoutMs != 0) b->SetTimeoutMs(timeoutMs);
    return b;
}
void mf_t_etcd_free(void *h) { delete static_cast<EtcdBackend *>(h); }
int mf_t_etcd_connect(void *h) { return static_cast<EtcdBackend *>(h)->Connect(); }
int mf_t_etcd_put(void *h, const char *key, const void *val, int len, uint32_t ttlMs)
{
    return static_cast<EtcdBackend *>(h)->Put(key, std::string((const char *)val, (size_t)len), ttlMs);
}
int mf_t_etcd_get(void *h, const char *key, char *buf, int cap)  // -> length (>= 0) or a negative error code
{
    std::string v;
    int rc = static_cast<EtcdBackend *>(h)->Get(key, v);
    if (rc != OK) return rc < 0 ? rc : -1;
    return CopyOut(v, buf, cap);
}
int mf_t_etcd_prefix_get(void *h, const char *prefix, char *buf, int cap)  // "key=value\n" lines -> length or a negative code
{
    std::vector<std::pair<std::string, std::string>> kvs;
    int rc = static_cast<EtcdBackend *>(h)->PrefixGet(prefix, kvs);
    if (rc != OK) return rc < 0 ? rc : -1;
    std::string all;
    for (auto &kv : kvs) all += kv.first + "=" + kv.second + "\n";
    return CopyOut(all, buf, cap);
}
int mf_t_etcd_delete(void *h, const char *key) { return static_cast<EtcdBackend *>(h)->Delete(key); }
int mf_t_etcd_clear(void *h, const char *prefix) { return static_cast<EtcdBackend *>(h)->Clear(prefix); }
int mf_t_etcd_exist(void *h, const char *key) { return static_cast<EtcdBackend *>(h)->Exist(key) ? 1 : 0; }
int mf_t_etcd_lock(void *h, const char *name) { return static_cast<EtcdBackend *>(h)->Lock(name); }
int mf_t_etcd_try_lock(void *h, const char *name) { return static_cast<EtcdBackend *>(h)->TryLock(name); }
int mf_t_etcd_unlock(void *h, const char *name) { return static_cast<EtcdBackend *>(h)->Unlock(name); }
int mf_t_etcd_last_error(void *h, char *buf, int cap)
{
    int n = CopyOut(static_cast<EtcdBackend *>(h)->LastError(), buf, cap - 1);
    if (buf != nullptr && cap > 0) buf[std::min(n, cap - 1)] = 0;
    return n;
}

void mf_t_backend_set_reachable(const char *name, int reachable) { LocalMemoryBackend::SetReachable(name, reachable != 0); }
void mf_t_backend_reset(const char *name) { LocalMemoryBackend::Reset(name); }

// ---- group engine -------------------------------------------------------------------------------------
typedef int (*mf_t_change_cb)(int event, uint32_t rank);  // event: 0 join, 1 leave, 3 link down, 4 update
void *mf_t_group_new(void *store, uint32_t rankSize, uint32_t rank, uint64_t timeoutMs, int dynamic, mf_t_change_cb cb)
{
    group::GroupOption o;
    o.rankSize = rankSize;
    o.rank = rank;
    o.timeoutMs = timeoutMs;
    o.dynamic = dynamic != 0;
    if (cb != nullptr) {
        o.joinCb = [cb](uint32_t r) { return cb(group::EV_JOIN, r); };
        o.leaveCb = [cb](uint32_t r) { return cb(group::EV_LEAVE, r); };
        o.linkDownCb = [cb](uint32_t r) { return cb(group::EV_LINK_DOWN, r); };
        o.updateCb = [cb](uint32_t r) { return cb(group::EV_UPDATE, r); };
    }
    auto g = group::GroupEngine::Create(static_cast<StoreBox *>(store)->s, o);
    if (!g) return nullptr;
    return new GroupBox{g};
}
void mf_t_group_free(void *h)
{
    auto b = static_cast<GroupBox *>(h);
    if (b == nullptr) return;
    b->g->StopListen();
    delete b;
}
int mf_t_group_barrier(void *h) { return static_cast<GroupBox *>(h)->g->Barrier(); }
int mf_t_group_allgather(void *h, const char *send, uint32_t sendSize, char *recv, uint32_t recvSize)
{
    return static_cast<GroupBox *>(h)->g->AllGather(send, sendSize, recv, recvSize);
}
int mf_t_group_sub_barrier(void *h, const char *key, uint32_t size, uint32_t rank) { return static_cast<GroupBox *>(h)->g->Barrier(key, size, rank); }
int mf_t_group_sub_allgather(void *h, const char *key, uint32_t size, uint32_t rank, const char *send, uint32_t sendSize, char *recv,
                             uint32_t recvSize)
{
    return static_cast<GroupBox *>(h)->g->AllGather(key, size, rank, send, sendSize, recv, recvSize);
}
int mf_t_group_start_listen(void *h) { return static_cast<GroupBox *>(h)->g->StartListen(); }
int mf_t_group_join(void *h) { return static_cast<GroupBox *>(h)->g->Join(); }
int mf_t_group_update(void *h) { return static_cast<GroupBox *>(h)->g->Update(); }
int mf_t_group_leave(void *h) { return static_cast<GroupBox *>(h)->g->Leave(); }
int mf_t_group_joined(void *h) { return static_cast<GroupBox *>(h)->g->Joined() ? 1 : 0; }
uint32_t mf_t_group_size(void *h) { return static_cast<GroupBox *>(h)->g->RankSize(); }
// version, groupSize, curEvent and the first bitmap word of the membership record this rank knows
void mf_t_group_info(void *h, uint32_t *version, uint32_t *size, uint32_t *event, uint64_t *bitmap0)
{
    auto i = static_cast<GroupBox *>(h)->g->Info();
    *version = i.version;
    *size = i.groupSize;
    *event = i.curEvent;
    *bitmap0 = i.bitmap[0];
}
int mf_t_group_alloc_number(void *h, uint32_t limit, int32_t *value) { return static_cast<GroupBox *>(h)->g->AllocNumber(limit, *value); }
int mf_t_group_release_number(void *h, int32_t value) { return static_cast<GroupBox *>(h)->g->ReleaseNumber(value); }

// ---- trace table --------------------------------------------------------------------------------------
int mf_t_trace_start(const char *dir, uint32_t periodMs) { return PTracer::Start(dir ? dir : "", periodMs); }
void mf_t_trace_stop(void) { PTracer::Stop(); }
// runs one bracketed operation of `sleepUs` on trace point `id` ending with `ret`
void mf_t_trace_hit(uint32_t id, int32_t ret, uint32_t sleepUs)
{
    const auto &t = PTracer::Current();
    uint64_t t0 = 0;
    if (t.enabled) {
        t0 = NowNs();
        if (t.begin) t.begin(id, t0);
    }
    if (sleepUs) std::this_thread::sleep_for(std::chrono::microseconds(sleepUs));
    if (t.enabled && t.end) t.end(id, t0, NowNs(), ret);
}
int mf_t_trace_dump(char *buf, int cap, int reset)
{
    std::string s = PTracer::DumpTable(reset != 0);
    int n = CopyOut(s, buf, cap - 1);
    if (buf != nullptr && cap > 0) buf[std::min(n, cap - 1)] = 0;
    return n;
}
int mf_t_trace_file(char *buf, int cap)
{
    std::string s = PTracer::FilePath();
    int n = CopyOut(s, buf, cap - 1);
    if (buf != nullptr && cap > 0) buf[std::min(n, cap - 1)] = 0;
    return n;
}
void mf_t_trace_row(uint32_t id, uint64_t out[6])
{
    auto r = PTracer::Snapshot(id);
    out[0] = r.begin, out[1] = r.goodEnd, out[2] = r.badEnd, out[3] = r.minNs, out[4] = r.maxNs, out[5] = r.totalNs;
}
// out[0 .. buckets) per-bucket counts (bucket i: at most 1 us * 2^i), out[buckets] the slower ones, out[buckets + 1] the
// sum of the durations in ns; -> number of buckets (call with out == NULL to size the array: buckets + 2 entries).
uint32_t mf_t_trace_hist(uint32_t id, uint64_t *out)
{
    if (out != nullptr) PTracer::Histogram(id, out, out + PTracer::kHistBuckets + 1);
    return PTracer::kHistBuckets;
}
const char *mf_t_trace_name(uint32_t id) { return TracePointName(id); }
uint32_t mf_t_trace_count(void) { return TP_COUNT; }

// ---- exchange records of the memory layer ------------------------------------------------------------------
// A host-memory entity that stands for rank `rank` of `ranks`; its own exchange records can be read out and records
// from elsewhere (a peer's, or damaged ones) imported and mapped.
struct ExBox {
    hybm::EntityPtr e;
    hybm::MemSlice *slice = nullptr;
};
void *mf_t_ex_new(uint16_t id, uint32_t rank, uint32_t ranks, uint64_t slot, uint64_t local)
{
    if (hybm::HybmInit(0xFFFF, 0) != OK) return nullptr;
    hybm_options ho{};
    ho.bmType = HYBM_TYPE_HOST_INITIATE;
    ho.memType = HYBM_MEM_TYPE_HOST;
    ho.bmDataOpType = HYBM_DOP_TYPE_HOST_SHM;
    ho.rankCount = ranks;
    ho.rankId = rank;
    ho.maxDRAMSize = slot;
    ho.scene = HYBM_SCENE_DEFAULT;
    ho.role = HYBM_ROLE_PEER;
    ho.dramShmFd = -1;
    auto e = hybm::Entity::Create(id, ho);
    if (!e || e->ReserveMemSpace(0) != OK) {
        hybm::HybmUninit();
        return nullptr;
    }
    auto *b = new ExBox{e, nullptr};
    if (local != 0 && e->AllocLocal(HYBM_MEM_TYPE_HOST, local, 0, &b->slice) != OK) {
        e->UnreserveMemSpace();
        delete b;
        hybm::HybmUninit();
        return nullptr;
    }
    return b;
}
void mf_t_ex_free(void *h)
{
    auto *b = static_cast<ExBox *>(h);
    b->e->Unmap();
    b->e->UnreserveMemSpace();
    delete b;
    hybm::HybmUninit();
}
uint32_t mf_t_ex_record_size(void) { return (uint32_t)sizeof(hybm_exchange_info); }
// out: room for two records (the entity's and its slice's); -> number of records written or a negative code
int mf_t_ex_export(void *h, uint8_t *out)
{
    auto *b = static_cast<ExBox *>(h);
    auto *recs = reinterpret_cast<hybm_exchange_info *>(out);
    int rc = b->e->Export(nullptr, &recs[0]);
    if (rc != OK) return rc;
    if (b->slice == nullptr) return 1;
    rc = b->e->Export(b->slice, &recs[1]);
    return rc != OK ? rc : 2;
}
// records: count * mf_t_ex_record_size() bytes. map != 0: maps what was imported as well. -> the first error code
int mf_t_ex_import(void *h, const uint8_t *records, uint32_t count, int map)
{
    auto *b = static_cast<ExBox *>(h);
    std::vector<hybm_exchange_info> v(count);
    memcpy(v.data(), records, (size_t)count * sizeof(hybm_exchange_info));
    int rc = b->e->Import(v.data(), count, nullptr);
    if (rc == OK && map != 0) rc = b->e->Mmap();
    return rc;
}
uint64_t mf_t_ex_mapped_bytes(void *h, uint32_t rank)
{
    auto seg = static_cast<ExBox *>(h)->e->SegmentOf(HYBM_MEM_TYPE_HOST);
    return seg ? seg->MappedBytes(rank) : 0;
}

// ---- fault points -------------------------------------------------------------------------------------
// Runs the periodic TLS certificate check now; -> the smallest number of days left over the live contexts.
int mf_t_tls_check_now(void) { return mf::net::TlsCheckAllNow(); }

void mf_t_fip_init(const char *confPath)
{
    FaultPoints::Init(confPath ? confPath : "");
    FaultPoints::RegisterBuiltins();
}
void mf_t_fip_exit(void)
{
    FaultPoints::UnregisterBuiltins();
    FaultPoints::Exit();
}
int mf_t_fip_activate(const char *name, int type, int32_t hits, int64_t param) { return FaultPoints::Activate(name, (FipType)type, hits, param); }
int mf_t_fip_deactivate(const char *name) { return FaultPoints::Deactivate(name); }
int mf_t_fip_is_active(const char *name) { return FaultPoints::IsActive(name) ? 1 : 0; }
void mf_t_fip_reload(void) { FaultPoints::Reload(); }
// Runs a guarded block: returns 1 when the block ran, 0 when the active point skipped it; *ret is what the
// point set (0 when it did not touch it).
int mf_t_fip_run(const char *name, int32_t *ret)
{
    *ret = 0;
    if (FaultPoints::Begin(name, ret)) return 0;
    return 1;
}

}  // extern "C"
