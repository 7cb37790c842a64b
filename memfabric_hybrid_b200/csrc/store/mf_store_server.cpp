// Config store server: 13 request types over the framed RPC, blocking GET with a timer thread,
// persistent key watchers, rank-down subscriptions, heartbeat checker, automatic rank assignment,
// a recovery window after a restart, and "clear everything when the last client leaves".
// Parity: src/smem/csrc/config_store/tcp_store/smem_tcp_config_store_server.cpp
// (handlers :348-975, admission :236-273, link loss :275-319, auto-rank :385-461, timer :1048-1142).
#include "mf_store.h"
#include "mf_store_backend.h"

namespace mf {
namespace store {

namespace {
constexpr uint64_t kWriteLimit = 1ULL << 30;
constexpr uint32_t kMissedHeartbeats = 3;
const std::string kOkText = "success";
}  // namespace

StoreServer::StoreServer(std::string ip, uint16_t port, uint32_t worldSize, uint64_t flags)
    : ip_(std::move(ip)), port_(port), worldSize_(worldSize), flags_(flags)
{
    handlers_[MT_SET] = &StoreServer::HSet;
    handlers_[MT_GET] = &StoreServer::HGet;
    handlers_[MT_PREFIX] = &StoreServer::HPrefix;
    handlers_[MT_WATCH] = &StoreServer::HWatch;
    handlers_[MT_ADD] = &StoreServer::HAdd;
    handlers_[MT_REMOVE] = &StoreServer::HRemove;
    handlers_[MT_APPEND] = &StoreServer::HAppend;
    handlers_[MT_CAS] = &StoreServer::HCas;
    handlers_[MT_WRITE] = &StoreServer::HWrite;
    handlers_[MT_QUERY_ALIVE] = &StoreServer::HQueryAlive;
    handlers_[MT_WATCH_RANK_STATE] = &StoreServer::HWatchRank;
    handlers_[MT_HEARTBEAT] = &StoreServer::HHeartbeat;
    handlers_[MT_UNWATCH] = &StoreServer::HUnwatch;
}

StoreServer::~StoreServer() { Shutdown(); }

void StoreServer::SetBackend(std::shared_ptr<StoreBackend> b, bool firstLeader)
{
    std::lock_guard<std::mutex> g(rankMu_);  // a server that is already accepting links reads all of this under the same lock
    backend_ = std::move(b);
    if (!backend_ || firstLeader) return;
    std::string v;
    if (backend_->Get(kBackendKeyWorldSize, v) == OK) {
        uint64_t ws = 0;
        if (ParseU64(v, ws) && ws > 0 && ws <= 1024 && worldSize_ == 0) worldSize_ = (uint32_t)ws;
    }
    if (backend_->Get(kBackendKeyAliveRanks, v) == OK) {
        for (auto &s : Split(v, ',')) {
            uint64_t r = 0;
            if (ParseU64(s, r)) expectedBack_.insert((uint32_t)r);
        }
    }
}

int StoreServer::Startup()
{
    if (running_.exchange(true)) return OK;
    net::EndpointOptions opt;
    opt.workers = 2;
    int tlsRc = OK;
    opt.tls = StoreFactory::TlsContextFor(tlsRc);
    if (tlsRc != OK) {
        running_ = false;
        return tlsRc;
    }
    ep_ = std::make_unique<net::Endpoint>(opt);
    ep_->OnNewLink([this](const net::ConnReq &r, const net::LinkPtr &l) { return OnNewLink(r, l); });
    ep_->OnMessage([this](const net::LinkPtr &l, const net::MsgHeader &h, std::string &b) { OnMessage(l, h, b); });
    ep_->OnBroken([this](const net::LinkPtr &l) { OnBroken(l); });
    int rc = ep_->Start();
    if (rc == OK) rc = ep_->Listen(ip_, port_);
    if (rc != OK) {
        running_ = false;
        ep_->Stop();
        ep_.reset();
        return rc;
    }
    port_ = ep_->ListenPort();
    if (!expectedBack_.empty() && (flags_ & 1ULL) == 0) {  // bit 0: skip the recovery window
        state_ = RECOVER;
        recoverDeadlineMs_ = NowMs() + ((backend_ && backend_->Distributed()) ? 60000 : 10000);
        uint64_t ovr = (uint64_t)EnvInt("MF_STORE_RECOVER_MS", nullptr, 0, 0, 600000);
        if (ovr > 0) recoverDeadlineMs_ = NowMs() + ovr;
    } else {
        expectedBack_.clear();
        state_ = NORMAL;
    }
    timer_ = std::thread([this] {
        pthread_setname_np(pthread_self(), "mf-store-timer");
        TimerLoop();
    });
    MF_INFO("config store server listening on %s:%u (world %u)", ip_.c_str(), port_, worldSize_);
    return OK;
}

void StoreServer::Shutdown()
{
    if (!running_.exchange(false)) return;
    if (timer_.joinable()) timer_.join();
    if (ep_) ep_->Stop();
    ep_.reset();
    std::lock_guard<std::mutex> g(kvMu_);
    kv_.clear();
    waiters_.clear();
    watchers_.clear();
}

size_t StoreServer::KeyCount()
{
    std::lock_guard<std::mutex> g(kvMu_);
    return kv_.size();
}

void StoreServer::PersistAlive()
{
    if (!backend_) return;
    std::string s;
    for (auto &kv : rankLinks_) {
        if (!s.empty()) s += ',';
        s += std::to_string(kv.first);
    }
    backend_->Put(kBackendKeyAliveRanks, s, 0);
    backend_->Put(kBackendKeyWorldSize, std::to_string(worldSize_), 0);
}

int StoreServer::OnNewLink(const net::ConnReq &req, const net::LinkPtr &l)
{
    uint32_t world = (uint32_t)(req.rankId >> 32);
    uint32_t rank = (uint32_t)(req.rankId & 0xFFFFFFFFu);
    std::lock_guard<std::mutex> g(rankMu_);
    if (state_ == RECOVER && req.reconnect == 0) {
        MF_INFO("store in recovery window: refusing new link (rank %u)", rank);
        return ERR_RECONNECT;
    }
    if (world != 0) {
        if (worldSize_ == 0) worldSize_ = world;
        else if (world != worldSize_) {
            MF_WARN("link claims world size %u but store serves %u: refused", world, worldSize_);
            return ERR_INVALID_PARAM;
        }
    }
    if (rank != kAutoRank) {
        if (worldSize_ != 0 && rank >= worldSize_ && rank < 0xFFFF0000u) {
            MF_WARN("link rank %u outside world %u: refused", rank, worldSize_);
            return ERR_INVALID_PARAM;
        }
        auto it = rankLinks_.find(rank);
        if (it != rankLinks_.end() && it->second->Alive() && rank < 0xFFFF0000u) {
            MF_WARN("rank %u already connected: refused", rank);
            return ERR_DUPLICATED;
        }
        if (rank < 0xFFFF0000u) {  // ranks at and above 0xFFFF0000 are anonymous observers (tools)
            rankLinks_[rank] = l;
            linkRanks_[l->Id()] = rank;
            expectedBack_.erase(rank);
            PersistAlive();
        }
    }
    allLinks_[l->Id()] = l;
    if (state_ == RECOVER && expectedBack_.empty()) state_ = NORMAL;
    return 0;
}

void StoreServer::OnBroken(const net::LinkPtr &l)
{
    uint32_t rank = kAutoRank;
    std::vector<Watcher> subs;
    bool lastGone = false;
    {
        std::lock_guard<std::mutex> g(rankMu_);
        allLinks_.erase(l->Id());
        rankWatchers_.erase(l->Id());
        auto it = linkRanks_.find(l->Id());
        if (it != linkRanks_.end()) {
            rank = it->second;
            linkRanks_.erase(it);
            auto rl = rankLinks_.find(rank);
            if (rl != rankLinks_.end() && rl->second->Id() == l->Id()) rankLinks_.erase(rl);
            PersistAlive();
            for (auto &kv : rankWatchers_) subs.push_back(kv.second);
        }
        lastGone = allLinks_.empty();
    }
    {
        std::lock_guard<std::mutex> g(kvMu_);
        for (auto it = waiters_.begin(); it != waiters_.end();) {
            it->second.remove_if([&](const Waiter &w) { return w.link->Id() == l->Id(); });
            it = it->second.empty() ? waiters_.erase(it) : std::next(it);
        }
        for (auto it = watchers_.begin(); it != watchers_.end();) {
            it->second.remove_if([&](const Watcher &w) { return w.link->Id() == l->Id(); });
            it = it->second.empty() ? watchers_.erase(it) : std::next(it);
        }
        if (lastGone) {
            kv_.clear();
            MF_INFO("last client left: store content cleared");
        }
    }
    if (rank != kAutoRank) {
        MF_INFO("rank %u link down, notifying %zu subscribers", rank, subs.size());
        StoreMessage m(MT_WATCH_RANK_STATE);
        m.values.emplace_back(reinterpret_cast<const char *>(&rank), sizeof(rank));
        for (auto &w : subs) ReplyMsg(w.link, w.seq, ST_OK, m);
    }
}

void StoreServer::Reply(const net::LinkPtr &l, uint32_t seq, int16_t code, const std::string &body)
{
    l->Send(0, code, seq, body.data(), (uint32_t)body.size());
}

void StoreServer::ReplyMsg(const net::LinkPtr &l, uint32_t seq, int16_t code, const StoreMessage &m)
{
    Reply(l, seq, code, m.Pack());
}

void StoreServer::OnMessage(const net::LinkPtr &l, const net::MsgHeader &h, std::string &body)
{
    StoreMessage m;
    if (!StoreMessage::Unpack(body, m)) {
        if (h.seqNo != 0) Reply(l, h.seqNo, ST_INVALID_MESSAGE, "invalid message");
        return;
    }
    (this->*handlers_[m.mt])(l, h, m);
}

void StoreServer::Wake(const std::string &key, const std::string &value)
{
    auto wi = waiters_.find(key);
    auto wa = watchers_.find(key);
    if (wi == waiters_.end() && wa == watchers_.end()) return;
    StoreMessage m(MT_GET);
    m.values.push_back(value);
    if (wi != waiters_.end()) {
        std::string packed = m.Pack();
        for (auto &w : wi->second)
            if (w.link->Alive()) Reply(w.link, w.seq, ST_OK, packed);
        waiters_.erase(wi);
    }
    if (wa != watchers_.end()) {
        m.mt = MT_WATCH;
        std::string packed = m.Pack();
        for (auto &w : wa->second)
            if (w.link->Alive()) Reply(w.link, w.seq, ST_OK, packed);
    }
}

void StoreServer::HSet(const net::LinkPtr &l, const net::MsgHeader &h, StoreMessage &m)
{
    if (m.keys.size() != 1 || m.values.size() != 1) return Reply(l, h.seqNo, ST_INVALID_MESSAGE, "SET wants 1 key 1 value");
    {
        std::lock_guard<std::mutex> g(kvMu_);
        auto it = kv_.find(m.keys[0]);
        bool changed = it == kv_.end() || it->second != m.values[0];
        if (it == kv_.end()) kv_.emplace(m.keys[0], m.values[0]);
        else it->second = m.values[0];
        if (changed) Wake(m.keys[0], m.values[0]);
    }
    Reply(l, h.seqNo, ST_OK, kOkText);
}

void StoreServer::AutoRank(const net::LinkPtr &l, uint32_t seq)
{
    std::unique_lock<std::mutex> g(rankMu_);
    uint32_t rank = kAutoRank;
    auto it = linkRanks_.find(l->Id());
    if (it != linkRanks_.end()) {
        rank = it->second;
    } else {
        if (worldSize_ == 0 || rankLinks_.size() >= worldSize_) {
            g.unlock();
            return Reply(l, seq, ST_ERROR, "error: no rank left in this world");
        }
        for (uint32_t scan = 0; scan <= worldSize_; scan++) {
            rankCursor_ %= worldSize_;
            if (rankLinks_.find(rankCursor_) == rankLinks_.end()) {
                rank = rankCursor_;
                break;
            }
            rankCursor_++;
        }
        if (rank == kAutoRank) {
            g.unlock();
            return Reply(l, seq, ST_ERROR, "no available rank");
        }
        rankLinks_[rank] = l;
        linkRanks_[l->Id()] = rank;
        expectedBack_.erase(rank);
        PersistAlive();
    }
    g.unlock();
    StoreMessage r(MT_GET);
    r.values.emplace_back(reinterpret_cast<const char *>(&rank), sizeof(rank));
    ReplyMsg(l, seq, ST_OK, r);
}

void StoreServer::HGet(const net::LinkPtr &l, const net::MsgHeader &h, StoreMessage &m)
{
    if (m.keys.size() != 1) return Reply(l, h.seqNo, ST_INVALID_MESSAGE, "GET wants 1 key");
    const std::string &key = m.keys[0];
    if (key.find(kAutoRankKey) != std::string::npos && key.size() >= strlen(kAutoRankKey) &&
        key.compare(key.size() - strlen(kAutoRankKey), strlen(kAutoRankKey), kAutoRankKey) == 0) {
        return AutoRank(l, h.seqNo);
    }
    std::unique_lock<std::mutex> g(kvMu_);
    auto it = kv_.find(key);
    if (it != kv_.end()) {
        StoreMessage r(MT_GET);
        r.values.push_back(it->second);
        g.unlock();
        return ReplyMsg(l, h.seqNo, ST_OK, r);
    }
    if (m.userDef == 0) {
        g.unlock();
        return Reply(l, h.seqNo, ST_NOT_EXIST, "not exist");
    }
    Waiter w{l, h.seqNo, m.userDef > 0 ? NowMs() + (uint64_t)m.userDef : 0, m.userDef};
    waiters_[key].push_back(std::move(w));
}

void StoreServer::HPrefix(const net::LinkPtr &l, const net::MsgHeader &h, StoreMessage &m)
{
    if (m.keys.size() != 1) return ReplyMsg(l, h.seqNo, ST_ERROR, StoreMessage(MT_PREFIX));
    StoreMessage r(MT_PREFIX);
    {
        std::lock_guard<std::mutex> g(kvMu_);
        const std::string &p = m.keys[0];
        for (auto it = kv_.lower_bound(p); it != kv_.end() && it->first.compare(0, p.size(), p) == 0; ++it) {
            if (r.keys.size() >= kMaxKeys) break;
            r.keys.push_back(it->first);
            r.values.push_back(it->second);
        }
    }
    ReplyMsg(l, h.seqNo, ST_OK, r);
}

void StoreServer::HWatch(const net::LinkPtr &l, const net::MsgHeader &h, StoreMessage &m)
{
    if (m.keys.size() != 1) return Reply(l, h.seqNo, ST_INVALID_MESSAGE, "WATCH wants 1 key");
    std::unique_lock<std::mutex> g(kvMu_);
    auto &lst = watchers_[m.keys[0]];
    lst.remove_if([&](const Watcher &w) { return w.link->Id() == l->Id(); });
    lst.push_back(Watcher{l, h.seqNo});
    auto it = kv_.find(m.keys[0]);
    if (it != kv_.end()) {
        StoreMessage r(MT_WATCH);
        r.values.push_back(it->second);
        g.unlock();
        ReplyMsg(l, h.seqNo, ST_OK, r);
    }
}

void StoreServer::HAdd(const net::LinkPtr &l, const net::MsgHeader &h, StoreMessage &m)
{
    if (m.keys.size() != 1 || m.values.size() != 1) return Reply(l, h.seqNo, ST_INVALID_MESSAGE, "ADD wants 1 key 1 value");
    int64_t inc = 0;
    if (!ParseI64(m.values[0], inc)) return Reply(l, h.seqNo, ST_INVALID_MESSAGE, "ADD value is not a decimal integer");
    std::string text;
    {
        std::lock_guard<std::mutex> g(kvMu_);
        int64_t cur = 0;
        auto it = kv_.find(m.keys[0]);
        if (it != kv_.end() && !ParseI64(it->second, cur)) return Reply(l, h.seqNo, ST_ERROR, "stored value is not a counter");
        int64_t next;
        if (__builtin_add_overflow(cur, inc, &next)) return Reply(l, h.seqNo, ST_ERROR, "counter overflow");
        text = std::to_string(next);
        kv_[m.keys[0]] = text;
        Wake(m.keys[0], text);
    }
    Reply(l, h.seqNo, ST_OK, text);
}

void StoreServer::HRemove(const net::LinkPtr &l, const net::MsgHeader &h, StoreMessage &m)
{
    if (m.keys.size() != 1) return Reply(l, h.seqNo, ST_INVALID_MESSAGE, "REMOVE wants 1 key");
    bool found;
    {
        std::lock_guard<std::mutex> g(kvMu_);
        found = kv_.erase(m.keys[0]) > 0;
    }
    if (found) Reply(l, h.seqNo, ST_OK, kOkText);
    else Reply(l, h.seqNo, ST_NOT_EXIST, "not exist");
}

void StoreServer::HAppend(const net::LinkPtr &l, const net::MsgHeader &h, StoreMessage &m)
{
    if (m.keys.size() != 1 || m.values.size() != 1) return Reply(l, h.seqNo, ST_INVALID_MESSAGE, "APPEND wants 1 key 1 value");
    uint64_t total;
    {
        std::lock_guard<std::mutex> g(kvMu_);
        std::string &v = kv_[m.keys[0]];
        if (v.size() + m.values[0].size() > kMaxValueLen) return Reply(l, h.seqNo, ST_ERROR, "value too large");
        v += m.values[0];
        total = v.size();
        Wake(m.keys[0], m.values[0]);  // blocked readers receive the appended piece
    }
    Reply(l, h.seqNo, ST_OK, std::to_string(total));
}

void StoreServer::HCas(const net::LinkPtr &l, const net::MsgHeader &h, StoreMessage &m)
{
    if (m.keys.size() != 1 || m.values.size() != 2) return Reply(l, h.seqNo, ST_INVALID_MESSAGE, "CAS wants 1 key 2 values");
    StoreMessage r(MT_CAS);
    {
        std::lock_guard<std::mutex> g(kvMu_);
        auto it = kv_.find(m.keys[0]);
        // An empty `expect` also means "only if the key does not exist".
        if (it == kv_.end() || it->second == m.values[0]) {
            bool changed = it == kv_.end() || it->second != m.values[1];
            kv_[m.keys[0]] = m.values[1];
            r.values.push_back(m.values[1]);
            if (changed) Wake(m.keys[0], m.values[1]);
        } else {
            r.values.push_back(it->second);
            r.values.push_back(it->second);
        }
    }
    ReplyMsg(l, h.seqNo, ST_OK, r);
}

void StoreServer::HWrite(const net::LinkPtr &l, const net::MsgHeader &h, StoreMessage &m)
{
    if (m.keys.size() != 1 || m.values.size() != 1 || m.values[0].size() < sizeof(uint32_t))
        return Reply(l, h.seqNo, ST_INVALID_MESSAGE, "WRITE wants 1 key and offset+bytes");
    uint32_t off = 0;
    memcpy(&off, m.values[0].data(), sizeof(off));
    size_t n = m.values[0].size() - sizeof(off);
    if ((uint64_t)off + n > kWriteLimit) return Reply(l, h.seqNo, ST_ERROR, "write beyond 1 GiB");
    {
        std::lock_guard<std::mutex> g(kvMu_);
        std::string &v = kv_[m.keys[0]];
        if (v.size() < off + n) v.resize(off + n, '\0');
        memcpy(&v[off], m.values[0].data() + sizeof(off), n);
        Wake(m.keys[0], v);
    }
    Reply(l, h.seqNo, ST_OK, kOkText);
}

void StoreServer::HQueryAlive(const net::LinkPtr &l, const net::MsgHeader &h, StoreMessage &m)
{
    uint64_t rank = 0;
    if (m.keys.size() != 1 || !ParseU64(m.keys[0], rank)) return Reply(l, h.seqNo, ST_INVALID_MESSAGE, "QUERY_ALIVE wants a rank");
    StoreMessage r(MT_QUERY_ALIVE);
    {
        std::lock_guard<std::mutex> g(rankMu_);
        auto it = rankLinks_.find((uint32_t)rank);
        if (it != rankLinks_.end() && it->second->Alive()) r.values.emplace_back("1");
    }
    ReplyMsg(l, h.seqNo, ST_OK, r);
}

void StoreServer::HWatchRank(const net::LinkPtr &l, const net::MsgHeader &h, StoreMessage &)
{
    std::lock_guard<std::mutex> g(rankMu_);
    rankWatchers_[l->Id()] = Watcher{l, h.seqNo};
}

void StoreServer::HHeartbeat(const net::LinkPtr &l, const net::MsgHeader &, StoreMessage &)
{
    l->userData.store(reinterpret_cast<void *>(1), std::memory_order_relaxed);  // this peer heartbeats: the checker may judge it
}

void StoreServer::HUnwatch(const net::LinkPtr &l, const net::MsgHeader &, StoreMessage &m)
{
    if (m.keys.size() != 1) return;
    if (m.keys[0] == kRankDownKey) {
        std::lock_guard<std::mutex> g(rankMu_);
        rankWatchers_.erase(l->Id());
        return;
    }
    std::lock_guard<std::mutex> g(kvMu_);
    auto it = watchers_.find(m.keys[0]);
    if (it == watchers_.end()) return;
    it->second.remove_if([&](const Watcher &w) { return w.link->Id() == l->Id(); });
    if (it->second.empty()) watchers_.erase(it);
}

void StoreServer::TimerLoop()
{
    uint64_t lastCheck = NowMs();
    while (running_) {
        bool timed = false;
        std::vector<Waiter> expired;
        uint64_t now = NowMs();
        {
            std::lock_guard<std::mutex> g(kvMu_);
            for (auto it = waiters_.begin(); it != waiters_.end();) {
                for (auto w = it->second.begin(); w != it->second.end();) {
                    if (w->deadlineMs != 0 && now >= w->deadlineMs) {
                        expired.push_back(*w);
                        w = it->second.erase(w);
                    } else {
                        timed = timed || w->deadlineMs != 0;
                        ++w;
                    }
                }
                it = it->second.empty() ? waiters_.erase(it) : std::next(it);
            }
        }
        for (auto &w : expired)
            if (w.link->Alive()) Reply(w.link, w.seq, ST_TIMEOUT, std::to_string(w.timeoutMs));
        uint32_t hb = HeartbeatMs();
        if (now - lastCheck >= hb) {
            lastCheck = now;
            std::vector<net::LinkPtr> dead;
            std::vector<uint32_t> missing;   // members of the previous leader's store that did not come back in time
            std::vector<Watcher> subs;
            {
                std::lock_guard<std::mutex> g(rankMu_);
                if (state_ == RECOVER && (expectedBack_.empty() || now >= recoverDeadlineMs_)) {
                    missing.assign(expectedBack_.begin(), expectedBack_.end());
                    expectedBack_.clear();
                    state_ = NORMAL;
                    MF_INFO("store recovery window closed, %zu member(s) did not return", missing.size());
                    if (!missing.empty()) {
                        PersistAlive();
                        for (auto &kv : rankWatchers_) subs.push_back(kv.second);
                    }
                }
                for (auto &kv : allLinks_) {
                    if (kv.second->userData.load(std::memory_order_relaxed) == nullptr) continue;
                    if (now - kv.second->lastSeenMs.load() > (uint64_t)kMissedHeartbeats * hb) dead.push_back(kv.second);
                }
            }
            // whoever did not return is down for good (it may have died with the old leader: nobody else saw its link
            // break): tell the subscribers, exactly as when a link breaks here
            for (uint32_t r : missing) {
                MF_INFO("rank %u did not return after the change of leader, notifying %zu subscribers", r, subs.size());
                StoreMessage m(MT_WATCH_RANK_STATE);
                m.values.emplace_back(reinterpret_cast<const char *>(&r), sizeof(r));
                for (auto &w : subs)
                    if (w.link->Alive()) ReplyMsg(w.link, w.seq, ST_OK, m);
            }
            for (auto &l : dead) {
                MF_WARN("link %lu missed %u heartbeats: closing", (unsigned long)l->Id(), kMissedHeartbeats);
                l->Shutdown();
            }
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(timed ? 1 : 20));
    }
}

}  // namespace store
}  // namespace mf
