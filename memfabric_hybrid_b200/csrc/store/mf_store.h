// Config store: the control-plane key/value service every other layer bootstraps through.
//   * StoreMessage  — the packed request/reply body
//   * ConfigStore   — abstract client interface (Set/Get/Add/Append/Cas/Watch/...)
//   * TcpStoreClient / StoreServer — TCP implementation, wire compatible with the reference
//   * PrefixStore   — key namespacing decorator
//   * StoreFactory  — URL parsing (tcp:// etc:// reg://, "#instance"), per-URL singletons
// Body layout (host-endian):
//   [u64 totalSize][i64 userDef][i16 mt][u64 keyCount]{[u64 len][bytes]}*[u64 valueCount]{[u64 len][bytes]}*
// Parity: src/smem/csrc/config_store/tcp_store/smem_message_packer.{h,cpp},
// src/smem/csrc/config_store/smem_config_store.h:50-293, smem_store_factory.h:25-91,
// src/smem/csrc/config_store/tcp_store/smem_prefix_config_store.h:21-90.
#pragma once
#include <list>
#include <set>

#include "../net/mf_rpc.h"

namespace mf {
namespace store {

enum MsgType : int16_t {
    MT_SET = 0,
    MT_GET = 1,
    MT_PREFIX = 2,
    MT_WATCH = 3,
    MT_ADD = 4,
    MT_REMOVE = 5,
    MT_APPEND = 6,
    MT_CAS = 7,
    MT_WRITE = 8,
    MT_QUERY_ALIVE = 9,
    MT_WATCH_RANK_STATE = 10,
    MT_HEARTBEAT = 11,
    MT_UNWATCH = 12,
    MT_COUNT
};

constexpr uint64_t kMaxKeys = 1024, kMaxKeyLen = 2048, kMaxValues = 1024, kMaxValueLen = 64ULL << 20;
constexpr const char *kAutoRankKey = "AutoRanking#";
constexpr const char *kRankDownKey = "WATCH_RANK_DOWN_KEY";
constexpr uint32_t kAutoRank = 0xFFFFFFFFu;

struct StoreMessage {
    MsgType mt = MT_SET;
    int64_t userDef = -1;
    std::vector<std::string> keys;
    std::vector<std::string> values;
    StoreMessage() = default;
    explicit StoreMessage(MsgType t) : mt(t) {}
    StoreMessage(MsgType t, std::string k) : mt(t) { keys.emplace_back(std::move(k)); }
    StoreMessage(MsgType t, std::string k, std::string v) : mt(t)
    {
        keys.emplace_back(std::move(k));
        values.emplace_back(std::move(v));
    }
    std::string Pack() const;
    // Returns false on a malformed or over-limit body.
    static bool Unpack(const std::string &buf, StoreMessage &out);
    static bool Unpack(const void *buf, size_t len, StoreMessage &out);
};

// Heartbeat period: 2 s in production; MF_STORE_HEARTBEAT_MS shortens it for tests.
uint32_t HeartbeatMs();

class ConfigStore {
public:
    virtual ~ConfigStore() = default;
    using WatchFn = std::function<void(int result, const std::string &key, const std::string &value)>;
    using RankDownFn = std::function<void(uint32_t rank)>;
    using ReconnectFn = std::function<int()>;
    using BrokenFn = std::function<void()>;

    virtual int Set(const std::string &key, const std::string &value) = 0;
    // timeoutMs: 0 => fail immediately with ERR_NOT_EXIST when absent; <0 => wait forever.
    virtual int Get(const std::string &key, std::string &value, int64_t timeoutMs) = 0;
    virtual int PrefixGet(const std::string &prefix, std::vector<std::string> &keys,
                          std::vector<std::string> &values) = 0;
    virtual int Add(const std::string &key, int64_t inc, int64_t &result) = 0;
    virtual int Remove(const std::string &key, bool quiet = false) = 0;
    virtual int Append(const std::string &key, const std::string &value, uint64_t &newSize) = 0;
    // Returns OK when `desired` was stored; ST_RESTORE-style loss returns ERR_IN_USE with `existing` filled.
    virtual int Cas(const std::string &key, const std::string &expect, const std::string &desired,
                    std::string &existing) = 0;
    virtual int Write(const std::string &key, uint32_t offset, const std::string &bytes) = 0;
    virtual int Watch(const std::string &key, WatchFn fn, uint32_t &watchId) = 0;
    virtual int Unwatch(uint32_t watchId) = 0;
    virtual int WatchRankState(RankDownFn fn, uint32_t &watchId) = 0;
    virtual int QueryAlive(uint32_t rank, bool &alive) = 0;
    virtual int AutoRank(uint32_t &rank) = 0;
    virtual void RegisterReconnectHandler(ReconnectFn fn) = 0;
    virtual void RegisterBrokenHandler(BrokenFn fn) = 0;
    virtual std::string Prefix() const { return ""; }
    virtual bool Connected() const = 0;
    virtual uint32_t Rank() const = 0;  // rank bound to this client's link (after AutoRank when asked for)
};
using StorePtr = std::shared_ptr<ConfigStore>;

// -------------------------------------------------------------------------------------------------
class TcpStoreClient : public ConfigStore, public std::enable_shared_from_this<TcpStoreClient> {
public:
    TcpStoreClient(std::string ip, uint16_t port, uint32_t worldSize, uint32_t rank);
    ~TcpStoreClient() override;
    // Dials until connected or `timeoutMs` elapses (the server may be in its recovery window).
    int Startup(uint32_t timeoutMs, uint32_t maxRetry = 0);
    void Shutdown();
    // Test hook: close the socket abruptly, as a crashed process would.
    void SimulateCrash();

    int Set(const std::string &key, const std::string &value) override;
    int Get(const std::string &key, std::string &value, int64_t timeoutMs) override;
    int PrefixGet(const std::string &prefix, std::vector<std::string> &keys, std::vector<std::string> &values) override;
    int Add(const std::string &key, int64_t inc, int64_t &result) override;
    int Remove(const std::string &key, bool quiet) override;
    int Append(const std::string &key, const std::string &value, uint64_t &newSize) override;
    int Cas(const std::string &key, const std::string &expect, const std::string &desired,
            std::string &existing) override;
    int Write(const std::string &key, uint32_t offset, const std::string &bytes) override;
    int Watch(const std::string &key, WatchFn fn, uint32_t &watchId) override;
    int Unwatch(uint32_t watchId) override;
    int WatchRankState(RankDownFn fn, uint32_t &watchId) override;
    int QueryAlive(uint32_t rank, bool &alive) override;
    int AutoRank(uint32_t &rank) override;
    void RegisterReconnectHandler(ReconnectFn fn) override;
    void RegisterBrokenHandler(BrokenFn fn) override;
    bool Connected() const override
    {
        std::lock_guard<std::mutex> g(linkMu_);  // the reconnector replaces link_ under this lock
        return link_ && link_->Alive();
    }
    uint32_t Rank() const override { return rank_; }
    void SetReconnectPolicy(uint32_t tries, uint32_t intervalMs)
    {
        reconnectTries_ = tries;
        reconnectIntervalMs_ = intervalMs;
    }
    // The first dial of Startup announces itself as a reconnect: for a process that was a member before
    // and now reaches a NEW server (HA fail-over), which admits only returning ranks while it recovers.
    void SetDialAsReconnect(bool on) { dialAsReconnect_ = on; }

private:
    struct Pending {
        std::mutex mu;
        std::condition_variable cv;
        bool done = false;
        int16_t result = 0;
        std::string body;
    };
    struct WatchCtx {
        uint32_t seq;
        std::string key;
        WatchFn fn;
        RankDownFn rankFn;
    };
    int Request(const StoreMessage &msg, int16_t &status, std::string &reply, int64_t waitMs);
    int SendNoReply(const StoreMessage &msg);
    void OnMessage(const net::MsgHeader &h, std::string &body);
    void OnBroken();
    void HeartbeatLoop();
    int Dial(bool reconnect, uint32_t timeoutMs);

    std::string ip_;
    uint16_t port_;
    uint32_t worldSize_;
    uint32_t rank_;
    std::unique_ptr<net::Endpoint> ep_;
    net::LinkPtr link_;
    mutable std::mutex linkMu_;
    std::atomic<uint32_t> seq_{1};
    std::mutex pendMu_;
    std::unordered_map<uint32_t, std::shared_ptr<Pending>> pending_;
    std::mutex watchMu_;
    std::unordered_map<uint32_t, std::shared_ptr<WatchCtx>> watches_;
    std::mutex cbMu_;
    std::vector<ReconnectFn> reconnectFns_;
    std::vector<BrokenFn> brokenFns_;
    std::thread hb_;
    std::thread reconnector_;
    std::mutex reMu_;  // reconnector_: started by a link's worker thread when the link breaks, joined by Shutdown
    std::mutex hbMu_;
    std::condition_variable hbCv_;
    std::atomic<bool> running_{false};
    std::atomic<bool> reconnecting_{false};
    uint32_t reconnectTries_ = 60;
    uint32_t reconnectIntervalMs_ = 1000;
    bool dialAsReconnect_ = false;
};

// -------------------------------------------------------------------------------------------------
class StoreBackend;
class StoreServer {
public:
    StoreServer(std::string ip, uint16_t port, uint32_t worldSize, uint64_t flags = 0);
    ~StoreServer();
    int Startup();
    void Shutdown();
    uint16_t Port() const { return port_; }
    // Persistence hook: world size and the alive-rank list go to the backend; restored at start-up.
    void SetBackend(std::shared_ptr<StoreBackend> b, bool firstLeader);
    size_t KeyCount();
    enum State { INITED, RECOVER, NORMAL };
    State GetState() const { return state_.load(); }

private:
    struct Waiter {
        net::LinkPtr link;
        uint32_t seq;
        uint64_t deadlineMs;  // 0 = forever
        int64_t timeoutMs;
    };
    struct Watcher {
        net::LinkPtr link;
        uint32_t seq;
    };
    using Handler = void (StoreServer::*)(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    int OnNewLink(const net::ConnReq &req, const net::LinkPtr &l);
    void OnBroken(const net::LinkPtr &l);
    void OnMessage(const net::LinkPtr &l, const net::MsgHeader &h, std::string &body);
    void Reply(const net::LinkPtr &l, uint32_t seq, int16_t code, const std::string &body);
    void ReplyMsg(const net::LinkPtr &l, uint32_t seq, int16_t code, const StoreMessage &m);
    void Wake(const std::string &key, const std::string &value);  // kvMu_ held
    void HSet(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void HGet(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void HPrefix(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void HWatch(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void HAdd(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void HRemove(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void HAppend(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void HCas(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void HWrite(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void HQueryAlive(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void HWatchRank(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void HHeartbeat(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void HUnwatch(const net::LinkPtr &, const net::MsgHeader &, StoreMessage &);
    void AutoRank(const net::LinkPtr &l, uint32_t seq);
    void TimerLoop();
    void PersistAlive();  // rankMu_ held

    std::string ip_;
    uint16_t port_;
    uint32_t worldSize_;
    uint64_t flags_;
    std::unique_ptr<net::Endpoint> ep_;
    Handler handlers_[MT_COUNT];
    std::mutex kvMu_;
    std::map<std::string, std::string> kv_;
    std::unordered_map<std::string, std::list<Waiter>> waiters_;
    std::unordered_map<std::string, std::list<Watcher>> watchers_;
    std::mutex rankMu_;
    std::map<uint32_t, net::LinkPtr> rankLinks_;          // rank -> link
    std::unordered_map<uint64_t, uint32_t> linkRanks_;    // link id -> rank
    std::unordered_map<uint64_t, net::LinkPtr> allLinks_; // link id -> link (rank may be unassigned)
    std::unordered_map<uint64_t, Watcher> rankWatchers_;  // link id -> subscription
    std::set<uint32_t> expectedBack_;                     // ranks alive before a restart
    uint32_t rankCursor_ = 0;
    std::atomic<State> state_{INITED};
    uint64_t recoverDeadlineMs_ = 0;
    std::thread timer_;
    std::atomic<bool> running_{false};
    std::shared_ptr<StoreBackend> backend_;
};

// -------------------------------------------------------------------------------------------------
class PrefixStore : public ConfigStore {
public:
    PrefixStore(StorePtr base, std::string prefix) : base_(std::move(base)), prefix_(std::move(prefix)) {}
    int Set(const std::string &k, const std::string &v) override { return base_->Set(prefix_ + k, v); }
    int Get(const std::string &k, std::string &v, int64_t t) override { return base_->Get(prefix_ + k, v, t); }
    int PrefixGet(const std::string &p, std::vector<std::string> &keys, std::vector<std::string> &values) override
    {
        int rc = base_->PrefixGet(prefix_ + p, keys, values);
        if (rc == OK)
            for (auto &k : keys)
                if (k.compare(0, prefix_.size(), prefix_) == 0) k.erase(0, prefix_.size());
        return rc;
    }
    int Add(const std::string &k, int64_t inc, int64_t &r) override { return base_->Add(prefix_ + k, inc, r); }
    int Remove(const std::string &k, bool quiet) override { return base_->Remove(prefix_ + k, quiet); }
    int Append(const std::string &k, const std::string &v, uint64_t &n) override
    {
        return base_->Append(prefix_ + k, v, n);
    }
    int Cas(const std::string &k, const std::string &e, const std::string &d, std::string &x) override
    {
        return base_->Cas(prefix_ + k, e, d, x);
    }
    int Write(const std::string &k, uint32_t off, const std::string &b) override
    {
        return base_->Write(prefix_ + k, off, b);
    }
    int Watch(const std::string &k, WatchFn fn, uint32_t &id) override
    {
        size_t n = prefix_.size();
        return base_->Watch(prefix_ + k,
                            [fn, n](int rc, const std::string &key, const std::string &v) {
                                fn(rc, key.size() >= n ? key.substr(n) : key, v);
                            },
                            id);
    }
    int Unwatch(uint32_t id) override { return base_->Unwatch(id); }
    int WatchRankState(RankDownFn fn, uint32_t &id) override { return base_->WatchRankState(std::move(fn), id); }
    int QueryAlive(uint32_t rank, bool &alive) override { return base_->QueryAlive(rank, alive); }
    int AutoRank(uint32_t &rank) override { return base_->AutoRank(rank); }
    void RegisterReconnectHandler(ReconnectFn fn) override { base_->RegisterReconnectHandler(std::move(fn)); }
    void RegisterBrokenHandler(BrokenFn fn) override { base_->RegisterBrokenHandler(std::move(fn)); }
    std::string Prefix() const override { return base_->Prefix() + prefix_; }
    bool Connected() const override { return base_->Connected(); }
    uint32_t Rank() const override { return base_->Rank(); }
    StorePtr Base() const { return base_; }

private:
    StorePtr base_;
    std::string prefix_;
};

// -------------------------------------------------------------------------------------------------
struct StoreUrl {
    enum Scheme { TCP, ETCD, REG } scheme = TCP;
    std::string ip;
    uint16_t port = 0;
    std::string instance;  // text after '#'
    std::string raw;
    static bool Parse(const std::string &url, StoreUrl &out);
};

struct TlsOptions {
    bool enable = false;
    std::string info;
    net::TlsSettings settings;
};

class StoreFactory {
public:
    // One shared client (and optionally one server) per URL.
    static StorePtr CreateStore(const std::string &url, bool isServer, uint32_t worldSize, uint32_t rank,
                                uint32_t timeoutMs, uint64_t serverFlags = 0, int *err = nullptr);
    static int CreateServerOnly(const std::string &url, uint32_t worldSize, uint64_t flags);
    static void DestroyStore(const std::string &url);
    static void DestroyServer(const std::string &url);  // counterpart of CreateServerOnly
    static void DestroyAll();
    static StorePtr Prefixed(const StorePtr &base, const std::string &prefix);
    // TLS for every store link of this process: SetTls takes the "key: value; ..." info string, SetTlsConfig the path
    // fields of a smem_tls_config, SetTlsKey the private key (a PEM text or a file path) with its pass phrase.
    static int SetTls(bool enable, const std::string &info);
    static int SetTlsConfig(const net::TlsSettings &s);
    static int SetTlsKey(const std::string &pk, const std::string &pass, net::TlsDecryptFn decrypt);
    static const TlsOptions &Tls();
    // The shared TLS context (built on first use), nullptr with rc == OK when TLS is off.
    static std::shared_ptr<net::TlsContext> TlsContextFor(int &rc);
    static std::shared_ptr<StoreServer> ServerOf(const std::string &url);
};

}  // namespace store
}  // namespace mf
