#include "mf_store_ha.h"

#include <random>

namespace mf {
namespace store {

HaConfigStore::HaConfigStore(std::string ip, uint16_t basePort, uint32_t worldSize, uint32_t rank, BackendPtr backend,
                             bool candidate)
    : ip_(std::move(ip)), basePort_(basePort), worldSize_(worldSize), rank_(rank), backend_(std::move(backend)),
      candidate_(candidate)
{
}

HaConfigStore::~HaConfigStore() { Shutdown(); }

void HaConfigStore::SetTimings(uint32_t leaseMs, uint32_t healthMs, uint32_t backoffLoMs, uint32_t backoffHiMs)
{
    leaseMs_ = leaseMs;
    healthMs_ = healthMs;
    backoffLo_ = backoffLoMs;
    backoffHi_ = std::max(backoffHiMs, backoffLoMs + 1);
}

std::shared_ptr<TcpStoreClient> HaConfigStore::Client()
{
    std::lock_guard<std::mutex> g(mu_);
    return client_;
}

std::string HaConfigStore::LeaderAddress()
{
    std::lock_guard<std::mutex> g(mu_);
    return leaderAddr_;
}

int HaConfigStore::Startup(uint32_t timeoutMs)
{
    if (running_.exchange(true)) return OK;
    int rc = Elect(timeoutMs);
    if (rc != OK) {
        running_ = false;
        return rc;
    }
    health_ = std::thread([this] {
        pthread_setname_np(pthread_self(), "mf-ha-health");
        HealthLoop();
    });
    return OK;
}

void HaConfigStore::Shutdown()
{
    if (!running_.exchange(false)) return;
    {
        std::lock_guard<std::mutex> g(cvMu_);
        cv_.notify_all();
    }
    JoinOrDetach(health_);
    std::shared_ptr<TcpStoreClient> c;
    std::shared_ptr<StoreServer> s;
    {
        std::lock_guard<std::mutex> g(mu_);
        c.swap(client_);
        s.swap(server_);
    }
    if (c) c->Shutdown();
    if (s) {
        s->Shutdown();
        if (leader_) backend_->Delete(kBackendKeyLeader);
    }
    leader_ = false;
}

void HaConfigStore::KillLeaderServer()
{
    std::shared_ptr<StoreServer> s;
    {
        std::lock_guard<std::mutex> g(mu_);
        s.swap(server_);
    }
    if (s) s->Shutdown();
    leader_ = false;
    candidate_ = false;  // a dead process does not stand again
}

int HaConfigStore::FollowLeader(const std::string &addr)
{
    std::string ip;
    uint16_t port = 0;
    if (!net::ParseIpPort(addr, ip, port)) return ERR_INVALID_PARAM;
    auto c = std::make_shared<TcpStoreClient>(ip, port, worldSize_, rank_);
    c->SetReconnectPolicy(0, 0);  // the HA layer re-elects instead of re-dialling a dead leader
    c->SetDialAsReconnect(everFollowed_.load());  // a returning member: admitted while the new leader recovers
    int rc = c->Startup(2000);
    if (rc != OK) return rc;
    std::weak_ptr<HaConfigStore> weak = weak_from_this();
    c->RegisterBrokenHandler([weak] {
        if (auto self = weak.lock()) self->ScheduleReelect();
    });
    std::map<uint32_t, SavedWatch> ws;
    {
        std::lock_guard<std::mutex> g(mu_);
        client_ = c;
        leaderAddr_ = addr;
        ws = watches_;
    }
    everFollowed_ = true;
    for (auto &kv : ws) {  // re-arm watches on the new leader
        uint32_t inner = 0;
        if (kv.second.rankFn) c->WatchRankState(kv.second.rankFn, inner);
        else c->Watch(kv.second.key, kv.second.fn, inner);
        std::lock_guard<std::mutex> g(mu_);
        auto it = watches_.find(kv.first);
        if (it != watches_.end()) it->second.innerId = inner;
    }
    return OK;
}

int HaConfigStore::BecomeLeader(bool first)
{
    uint16_t port = net::FindFreePort(ip_, basePort_);
    if (port == 0) return MF_FAIL(ERR_NO_RESOURCES, "no free port at or above %u for the store leader", basePort_);
    auto s = std::make_shared<StoreServer>(ip_, port, worldSize_, 0);
    s->SetBackend(backend_, first);
    int rc = s->Startup();
    if (rc != OK) return rc;
    std::string addr = ip_ + ":" + std::to_string(s->Port());
    rc = backend_->Put(kBackendKeyLeader, addr, leaseMs_);
    if (rc != OK) {
        s->Shutdown();
        return rc;
    }
    backend_->Put(kBackendKeyLeaderStatus, "serving", 0);
    {
        std::lock_guard<std::mutex> g(mu_);
        server_ = s;
    }
    leader_ = true;
    MF_INFO("became config-store leader at %s", addr.c_str());
    return FollowLeader(addr);
}

int HaConfigStore::Elect(uint32_t timeoutMs)
{
    std::mt19937 rng((uint32_t)(NowNs() ^ (uint64_t)(uintptr_t)this));
    uint64_t deadline = NowMs() + timeoutMs;
    while (running_) {
        uint32_t backoff = backoffLo_ + rng() % (backoffHi_ - backoffLo_);
        std::this_thread::sleep_for(std::chrono::milliseconds(backoff));
        if (backend_->Connect() == OK) {
            std::string addr, ip;
            uint16_t port = 0;
            bool haveLeader = backend_->Get(kBackendKeyLeader, addr) == OK && net::ParseIpPort(addr, ip, port) &&
                              net::ProbeReachable(ip, port, 500);
            if (haveLeader) {
                if (FollowLeader(addr) == OK) return OK;
            } else if (candidate_) {
                DistributedLockGuard lock(backend_, "backend");
                if (lock.Held()) {
                    // somebody may have won while we waited for the lock
                    if (backend_->Get(kBackendKeyLeader, addr) == OK && net::ParseIpPort(addr, ip, port) &&
                        net::ProbeReachable(ip, port, 500)) {
                        if (FollowLeader(addr) == OK) return OK;
                    } else {
                        bool first = !backend_->Exist(kBackendKeyLeaderStatus);
                        if (BecomeLeader(first) == OK) return OK;
                    }
                }
            }
        }
        if (NowMs() >= deadline) return MF_FAIL(ERR_TIMEOUT, "config-store leader election timed out");
    }
    return ERR_NOT_STARTED;
}

void HaConfigStore::Demote()
{
    std::shared_ptr<StoreServer> s;
    {
        std::lock_guard<std::mutex> g(mu_);
        s.swap(server_);
    }
    leader_ = false;
    if (s) {
        MF_WARN("store leader lost its backend: stepping down");
        s->Shutdown();
    }
}

void HaConfigStore::ScheduleReelect()
{
    reelect_ = true;
    std::lock_guard<std::mutex> g(cvMu_);
    cv_.notify_all();
}

void HaConfigStore::HealthLoop()
{
    while (running_) {
        {
            std::unique_lock<std::mutex> lk(cvMu_);
            cv_.wait_for(lk, std::chrono::milliseconds(healthMs_), [this] { return !running_ || reelect_.load(); });
        }
        if (!running_) break;
        if (leader_) {
            std::string addr = LeaderAddress(), cur, ip;
            uint16_t port = 0;
            if (backend_->Connect() == OK && backend_->Get(kBackendKeyLeader, cur) == OK && cur != addr && net::ParseIpPort(cur, ip, port) &&
                net::ProbeReachable(ip, port, 500)) {
                // Somebody else was elected while this node could not be reached (it looked dead from there) and serves:
                // two leaders would split the members between them. The key decides: follow it.
                MF_WARN("config-store leader key names %s, which answers: stepping down at %s", cur.c_str(), addr.c_str());
                Demote();
                reelect_ = true;
            } else if (backend_->Connect() != OK || backend_->Put(kBackendKeyLeader, addr, leaseMs_) != OK) {
                Demote();
                reelect_ = true;
            }
        }
        if (reelect_.exchange(false)) {
            std::shared_ptr<TcpStoreClient> old;
            {
                std::lock_guard<std::mutex> g(mu_);
                old.swap(client_);
            }
            if (old) old->Shutdown();
            if (Elect(30000) == OK) {
                std::vector<ReconnectFn> fns;
                {
                    std::lock_guard<std::mutex> g(mu_);
                    fns = reconnectFns_;
                }
                for (auto &f : fns) f();
            } else if (running_) {
                reelect_ = true;  // keep trying
            }
        }
    }
}

#define HA_FORWARD(expr)                       \
    auto c = Client();                         \
    if (!c) return ERR_NOT_CONNECTED;          \
    return c->expr

int HaConfigStore::Set(const std::string &k, const std::string &v) { HA_FORWARD(Set(k, v)); }
int HaConfigStore::Get(const std::string &k, std::string &v, int64_t t) { HA_FORWARD(Get(k, v, t)); }
int HaConfigStore::PrefixGet(const std::string &p, std::vector<std::string> &ks, std::vector<std::string> &vs)
{
    HA_FORWARD(PrefixGet(p, ks, vs));
}
int HaConfigStore::Add(const std::string &k, int64_t inc, int64_t &r) { HA_FORWARD(Add(k, inc, r)); }
int HaConfigStore::Remove(const std::string &k, bool q) { HA_FORWARD(Remove(k, q)); }
int HaConfigStore::Append(const std::string &k, const std::string &v, uint64_t &n) { HA_FORWARD(Append(k, v, n)); }
int HaConfigStore::Cas(const std::string &k, const std::string &e, const std::string &d, std::string &x)
{
    HA_FORWARD(Cas(k, e, d, x));
}
int HaConfigStore::Write(const std::string &k, uint32_t off, const std::string &b) { HA_FORWARD(Write(k, off, b)); }
int HaConfigStore::QueryAlive(uint32_t rank, bool &alive) { HA_FORWARD(QueryAlive(rank, alive)); }
int HaConfigStore::AutoRank(uint32_t &rank)
{
    auto c = Client();
    if (!c) return ERR_NOT_CONNECTED;
    int rc = c->AutoRank(rank);
    if (rc == OK) rank_ = rank;
    return rc;
}

int HaConfigStore::Watch(const std::string &key, WatchFn fn, uint32_t &watchId)
{
    auto c = Client();
    if (!c) return ERR_NOT_CONNECTED;
    uint32_t inner = 0;
    int rc = c->Watch(key, fn, inner);
    if (rc != OK) return rc;
    std::lock_guard<std::mutex> g(mu_);
    watchId = nextWatch_++;
    watches_[watchId] = SavedWatch{key, fn, nullptr, inner};
    return OK;
}

int HaConfigStore::WatchRankState(RankDownFn fn, uint32_t &watchId)
{
    auto c = Client();
    if (!c) return ERR_NOT_CONNECTED;
    uint32_t inner = 0;
    int rc = c->WatchRankState(fn, inner);
    if (rc != OK) return rc;
    std::lock_guard<std::mutex> g(mu_);
    watchId = nextWatch_++;
    watches_[watchId] = SavedWatch{kRankDownKey, nullptr, fn, inner};
    return OK;
}

int HaConfigStore::Unwatch(uint32_t watchId)
{
    uint32_t inner;
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = watches_.find(watchId);
        if (it == watches_.end()) return ERR_NOT_EXIST;
        inner = it->second.innerId;
        watches_.erase(it);
    }
    auto c = Client();
    return c ? c->Unwatch(inner) : OK;
}

void HaConfigStore::RegisterReconnectHandler(ReconnectFn fn)
{
    std::lock_guard<std::mutex> g(mu_);
    reconnectFns_.push_back(std::move(fn));
}

void HaConfigStore::RegisterBrokenHandler(BrokenFn fn)
{
    std::lock_guard<std::mutex> g(mu_);
    brokenFns_.push_back(std::move(fn));
}

bool HaConfigStore::Connected() const
{
    auto c = const_cast<HaConfigStore *>(this)->Client();
    return c && c->Connected();
}

}  // namespace store
}  // namespace mf
