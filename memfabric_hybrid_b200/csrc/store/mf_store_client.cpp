// TCP config-store client: one blocked caller per sequence number, persistent watch contexts that
// survive a reconnect, a heartbeat thread, and a reconnect loop (60 x 1 s by default) that re-dials
// with the reconnect bit set, re-arms the watches and runs the registered reconnect handlers.
// Parity: src/smem/csrc/config_store/tcp_store/smem_tcp_config_store.cpp:172-236,560-700,676-848.
#include "../util/mf_trace.h"
#include "mf_store.h"

namespace mf {
namespace store {

TcpStoreClient::TcpStoreClient(std::string ip, uint16_t port, uint32_t worldSize, uint32_t rank)
    : ip_(std::move(ip)), port_(port), worldSize_(worldSize), rank_(rank)
{
}

TcpStoreClient::~TcpStoreClient() { Shutdown(); }

int TcpStoreClient::Dial(bool reconnect, uint32_t timeoutMs)
{
    int32_t fip = OK;
    MF_FIP_START(STORE_CONNECT, &fip)
    MF_FIP_END
    if (fip != OK) return fip;
    net::ConnReq req;
    req.reconnect = reconnect ? 1 : 0;
    req.rankId = ((uint64_t)worldSize_ << 32) | rank_;
    net::LinkPtr l;
    int16_t refused = 0;
    int rc = ep_->Connect(ip_, port_, req, timeoutMs, l, &refused);
    if (rc != OK) return rc;
    std::lock_guard<std::mutex> g(linkMu_);
    link_ = l;
    return OK;
}

int TcpStoreClient::Startup(uint32_t timeoutMs, uint32_t maxRetry)
{
    if (running_.exchange(true)) return OK;
    net::EndpointOptions opt;
    opt.workers = 1;
    int tlsRc = OK;
    opt.tls = StoreFactory::TlsContextFor(tlsRc);
    if (tlsRc != OK) {
        running_ = false;
        return tlsRc;
    }
    ep_ = std::make_unique<net::Endpoint>(opt);
    std::weak_ptr<TcpStoreClient> weak = weak_from_this();
    ep_->OnMessage([this](const net::LinkPtr &, const net::MsgHeader &h, std::string &b) { OnMessage(h, b); });
    ep_->OnBroken([this](const net::LinkPtr &l) {
        bool mine;
        {
            std::lock_guard<std::mutex> g(linkMu_);
            mine = link_ && link_->Id() == l->Id();
        }
        if (mine) OnBroken();
    });
    int rc = ep_->Start();
    if (rc != OK) {
        running_ = false;
        return rc;
    }
    uint64_t deadline = NowMs() + timeoutMs;
    uint32_t tries = 0;
    for (;;) {
        rc = Dial(dialAsReconnect_, std::min<uint32_t>(timeoutMs == 0 ? 1000 : timeoutMs, 3000));
        if (rc == OK) break;
        tries++;
        if (NowMs() >= deadline || (maxRetry != 0 && tries >= maxRetry)) {
            running_ = false;
            ep_->Stop();
            ep_.reset();
            return MF_FAIL(rc == ERR_RECONNECT ? ERR_RECONNECT : ERR_NOT_CONNECTED,
                           "cannot reach config store %s:%u within %u ms", ip_.c_str(), port_, timeoutMs);
        }
        std::this_thread::sleep_for(std::chrono::milliseconds(rc == ERR_RECONNECT ? 500 : 100));
    }
    hb_ = std::thread([this] {
        pthread_setname_np(pthread_self(), "mf-store-hb");
        HeartbeatLoop();
    });
    return OK;
}

void TcpStoreClient::Shutdown()
{
    if (!running_.exchange(false)) return;
    {
        std::lock_guard<std::mutex> g(hbMu_);
        hbCv_.notify_all();
    }
    JoinOrDetach(hb_);
    {
        // A link that breaks right now may be about to start the reconnector on its worker thread: take the thread out
        // under the lock (whoever gets the lock after us sees running_ == false and starts nothing).
        std::thread re;
        {
            std::lock_guard<std::mutex> g(reMu_);
            re.swap(reconnector_);
        }
        JoinOrDetach(re);
    }
    {
        std::lock_guard<std::mutex> g(linkMu_);
        if (link_) link_->Shutdown();
    }
    if (ep_) ep_->Stop();
    ep_.reset();
    // release callers still blocked
    std::lock_guard<std::mutex> g(pendMu_);
    for (auto &kv : pending_) {
        std::lock_guard<std::mutex> pg(kv.second->mu);
        kv.second->done = true;
        kv.second->result = ST_IO_ERROR;
        kv.second->cv.notify_all();
    }
    pending_.clear();
}

void TcpStoreClient::SimulateCrash()
{
    // Stop heartbeats and reconnection, then drop the socket without any goodbye.
    reconnectTries_ = 0;
    std::lock_guard<std::mutex> g(linkMu_);
    if (link_) link_->Shutdown();
}

void TcpStoreClient::HeartbeatLoop()
{
    StoreMessage hb(MT_HEARTBEAT);
    std::string packed = hb.Pack();
    while (running_) {
        {
            std::unique_lock<std::mutex> lk(hbMu_);
            hbCv_.wait_for(lk, std::chrono::milliseconds(HeartbeatMs()));
        }
        if (!running_) break;
        net::LinkPtr l;
        {
            std::lock_guard<std::mutex> g(linkMu_);
            l = link_;
        }
        if (l && l->Alive()) l->Send(0, 0, 0, packed.data(), (uint32_t)packed.size());
    }
}

void TcpStoreClient::OnMessage(const net::MsgHeader &h, std::string &body)
{
    std::shared_ptr<Pending> p;
    {
        std::lock_guard<std::mutex> g(pendMu_);
        auto it = pending_.find(h.seqNo);
        if (it != pending_.end()) {
            p = it->second;
            pending_.erase(it);
        }
    }
    if (p) {
        std::lock_guard<std::mutex> g(p->mu);
        p->result = h.result;
        p->body.swap(body);
        p->done = true;
        p->cv.notify_all();
        return;
    }
    std::shared_ptr<WatchCtx> w;
    {
        std::lock_guard<std::mutex> g(watchMu_);
        auto it = watches_.find(h.seqNo);
        if (it != watches_.end()) w = it->second;
    }
    if (!w) return;
    StoreMessage m;
    if (!StoreMessage::Unpack(body, m) || m.values.empty()) return;
    if (w->rankFn) {
        if (m.values[0].size() >= sizeof(uint32_t)) {
            uint32_t r;
            memcpy(&r, m.values[0].data(), sizeof(r));
            w->rankFn(r);
        }
    } else if (w->fn) {
        w->fn(h.result == ST_OK ? OK : ERR, w->key, m.values[0]);
    }
}

void TcpStoreClient::OnBroken()
{
    {
        std::lock_guard<std::mutex> g(pendMu_);
        for (auto &kv : pending_) {
            std::lock_guard<std::mutex> pg(kv.second->mu);
            kv.second->done = true;
            kv.second->result = ST_IO_ERROR;
            kv.second->cv.notify_all();
        }
        pending_.clear();
    }
    std::vector<BrokenFn> fns;
    {
        std::lock_guard<std::mutex> g(cbMu_);
        fns = brokenFns_;
    }
    for (auto &f : fns) f();
    std::lock_guard<std::mutex> rg(reMu_);
    if (!running_ || reconnectTries_ == 0 || reconnecting_.exchange(true)) return;
    JoinOrDetach(reconnector_);
    reconnector_ = std::thread([this] {
        pthread_setname_np(pthread_self(), "mf-store-redial");
        bool ok = false;
        for (uint32_t i = 0; i < reconnectTries_ && running_; i++) {
            std::this_thread::sleep_for(std::chrono::milliseconds(reconnectIntervalMs_));
            if (!running_) break;
            if (Dial(true, 1000) == OK) {
                ok = true;
                break;
            }
        }
        reconnecting_ = false;
        if (!ok || !running_) {
            if (running_) MF_ERROR("config store %s:%u unreachable after %u attempts", ip_.c_str(), port_, reconnectTries_);
            return;
        }
        MF_INFO("reconnected to config store %s:%u", ip_.c_str(), port_);
        // re-arm watches under their original sequence numbers
        std::vector<std::shared_ptr<WatchCtx>> ws;
        {
            std::lock_guard<std::mutex> g(watchMu_);
            for (auto &kv : watches_) ws.push_back(kv.second);
        }
        net::LinkPtr l;
        {
            std::lock_guard<std::mutex> g(linkMu_);
            l = link_;
        }
        for (auto &w : ws) {
            StoreMessage m(w->rankFn ? MT_WATCH_RANK_STATE : MT_WATCH, w->key);
            std::string packed = m.Pack();
            if (l) l->Send(0, 0, w->seq, packed.data(), (uint32_t)packed.size());
        }
        std::vector<ReconnectFn> fns;
        {
            std::lock_guard<std::mutex> g(cbMu_);
            fns = reconnectFns_;
        }
        for (auto &f : fns) f();
    });
}

int TcpStoreClient::Request(const StoreMessage &msg, int16_t &status, std::string &reply, int64_t waitMs)
{
    net::LinkPtr l;
    {
        std::lock_guard<std::mutex> g(linkMu_);
        l = link_;
    }
    if (!l || !l->Alive()) return ERR_NOT_CONNECTED;
    uint32_t seq = seq_.fetch_add(1);
    if (seq == 0) seq = seq_.fetch_add(1);
    auto p = std::make_shared<Pending>();
    {
        std::lock_guard<std::mutex> g(pendMu_);
        pending_[seq] = p;
    }
    std::string packed = msg.Pack();
    if (l->Send(0, 0, seq, packed.data(), (uint32_t)packed.size()) != OK) {
        std::lock_guard<std::mutex> g(pendMu_);
        pending_.erase(seq);
        return ERR_NOT_CONNECTED;
    }
    std::unique_lock<std::mutex> lk(p->mu);
    if (waitMs < 0) {
        p->cv.wait(lk, [&] { return p->done; });
    } else if (!p->cv.wait_for(lk, std::chrono::milliseconds(waitMs), [&] { return p->done; })) {
        lk.unlock();
        std::lock_guard<std::mutex> g(pendMu_);
        pending_.erase(seq);
        return ERR_TIMEOUT;
    }
    status = p->result;
    reply.swap(p->body);
    return status == ST_IO_ERROR ? ERR_NOT_CONNECTED : OK;
}

int TcpStoreClient::SendNoReply(const StoreMessage &msg)
{
    net::LinkPtr l;
    {
        std::lock_guard<std::mutex> g(linkMu_);
        l = link_;
    }
    if (!l || !l->Alive()) return ERR_NOT_CONNECTED;
    std::string packed = msg.Pack();
    return l->Send(0, 0, 0, packed.data(), (uint32_t)packed.size());
}

static constexpr int64_t kRpcWaitMs = 30000;

static int MapStatus(int16_t st)
{
    switch (st) {
        case ST_OK: return OK;
        case ST_NOT_EXIST: return ERR_NOT_EXIST;
        case ST_TIMEOUT: return ERR_TIMEOUT;
        case ST_IO_ERROR: return ERR_NOT_CONNECTED;
        case ST_INVALID_MESSAGE:
        case ST_INVALID_KEY: return ERR_INVALID_PARAM;
        default: return ERR;
    }
}

int TcpStoreClient::Set(const std::string &key, const std::string &value)
{
    if (key.empty() || key.size() > kMaxKeyLen || value.size() > kMaxValueLen) return ERR_INVALID_PARAM;
    MF_TRACE_BEGIN(TP_STORE_SET);
    int16_t st = 0;
    std::string rep;
    int rc = Request(StoreMessage(MT_SET, key, value), st, rep, kRpcWaitMs);
    if (rc == OK) rc = MapStatus(st);
    MF_TRACE_END(TP_STORE_SET, rc);
    return rc;
}

int TcpStoreClient::Get(const std::string &key, std::string &value, int64_t timeoutMs)
{
    if (key.empty() || key.size() > kMaxKeyLen) return ERR_INVALID_PARAM;
    MF_TRACE_BEGIN(TP_STORE_GET);
    StoreMessage m(MT_GET, key);
    m.userDef = timeoutMs;
    int16_t st = 0;
    std::string rep;
    int rc = Request(m, st, rep, timeoutMs < 0 ? -1 : timeoutMs + 5000);
    if (rc == OK) rc = MapStatus(st);
    if (rc == OK) {
        StoreMessage r;
        if (!StoreMessage::Unpack(rep, r) || r.values.size() != 1) rc = ERR;
        else value.swap(r.values[0]);
    }
    MF_TRACE_END(TP_STORE_GET, rc == ERR_NOT_EXIST ? 0 : rc);
    return rc;
}

int TcpStoreClient::PrefixGet(const std::string &prefix, std::vector<std::string> &keys, std::vector<std::string> &values)
{
    int16_t st = 0;
    std::string rep;
    int rc = Request(StoreMessage(MT_PREFIX, prefix), st, rep, kRpcWaitMs);
    if (rc != OK) return rc;
    if (st != ST_OK) return MapStatus(st);
    StoreMessage r;
    if (!StoreMessage::Unpack(rep, r) || r.keys.size() != r.values.size()) return ERR;
    keys.swap(r.keys);
    values.swap(r.values);
    return OK;
}

int TcpStoreClient::Add(const std::string &key, int64_t inc, int64_t &result)
{
    int16_t st = 0;
    std::string rep;
    int rc = Request(StoreMessage(MT_ADD, key, std::to_string(inc)), st, rep, kRpcWaitMs);
    if (rc != OK) return rc;
    if (st != ST_OK) return MapStatus(st);
    return ParseI64(rep, result) ? OK : ERR;
}

int TcpStoreClient::Remove(const std::string &key, bool quiet)
{
    int16_t st = 0;
    std::string rep;
    int rc = Request(StoreMessage(MT_REMOVE, key), st, rep, kRpcWaitMs);
    if (rc != OK) return rc;
    if (st == ST_NOT_EXIST && quiet) return OK;
    return MapStatus(st);
}

int TcpStoreClient::Append(const std::string &key, const std::string &value, uint64_t &newSize)
{
    int16_t st = 0;
    std::string rep;
    int rc = Request(StoreMessage(MT_APPEND, key, value), st, rep, kRpcWaitMs);
    if (rc != OK) return rc;
    if (st != ST_OK) return MapStatus(st);
    return ParseU64(rep, newSize) ? OK : ERR;
}

int TcpStoreClient::Cas(const std::string &key, const std::string &expect, const std::string &desired,
                        std::string &existing)
{
    MF_TRACE_BEGIN(TP_STORE_CAS);
    StoreMessage m(MT_CAS, key);
    m.values.push_back(expect);
    m.values.push_back(desired);
    int16_t st = 0;
    std::string rep;
    int rc = Request(m, st, rep, kRpcWaitMs);
    if (rc == OK) rc = MapStatus(st);
    if (rc == OK) {
        StoreMessage r;
        if (!StoreMessage::Unpack(rep, r) || r.values.empty()) {
            rc = ERR;
        } else {
            existing = r.values[0];
            if (r.values.size() > 1) rc = ERR_IN_USE;  // two values: somebody else's record won
        }
    }
    MF_TRACE_END(TP_STORE_CAS, rc == ERR_IN_USE ? 0 : rc);
    return rc;
}

int TcpStoreClient::Write(const std::string &key, uint32_t offset, const std::string &bytes)
{
    std::string v(reinterpret_cast<const char *>(&offset), sizeof(offset));
    v += bytes;
    int16_t st = 0;
    std::string rep;
    int rc = Request(StoreMessage(MT_WRITE, key, v), st, rep, kRpcWaitMs);
    if (rc != OK) return rc;
    return MapStatus(st);
}

int TcpStoreClient::Watch(const std::string &key, WatchFn fn, uint32_t &watchId)
{
    net::LinkPtr l;
    {
        std::lock_guard<std::mutex> g(linkMu_);
        l = link_;
    }
    if (!l || !l->Alive()) return ERR_NOT_CONNECTED;
    auto w = std::make_shared<WatchCtx>();
    w->seq = seq_.fetch_add(1);
    w->key = key;
    w->fn = std::move(fn);
    {
        std::lock_guard<std::mutex> g(watchMu_);
        watches_[w->seq] = w;
    }
    watchId = w->seq;
    std::string packed = StoreMessage(MT_WATCH, key).Pack();
    return l->Send(0, 0, w->seq, packed.data(), (uint32_t)packed.size());
}

int TcpStoreClient::WatchRankState(RankDownFn fn, uint32_t &watchId)
{
    net::LinkPtr l;
    {
        std::lock_guard<std::mutex> g(linkMu_);
        l = link_;
    }
    if (!l || !l->Alive()) return ERR_NOT_CONNECTED;
    auto w = std::make_shared<WatchCtx>();
    w->seq = seq_.fetch_add(1);
    w->key = kRankDownKey;
    w->rankFn = std::move(fn);
    {
        std::lock_guard<std::mutex> g(watchMu_);
        watches_[w->seq] = w;
    }
    watchId = w->seq;
    std::string packed = StoreMessage(MT_WATCH_RANK_STATE, kRankDownKey).Pack();
    return l->Send(0, 0, w->seq, packed.data(), (uint32_t)packed.size());
}

int TcpStoreClient::Unwatch(uint32_t watchId)
{
    std::shared_ptr<WatchCtx> w;
    {
        std::lock_guard<std::mutex> g(watchMu_);
        auto it = watches_.find(watchId);
        if (it == watches_.end()) return ERR_NOT_EXIST;
        w = it->second;
        watches_.erase(it);
    }
    SendNoReply(StoreMessage(MT_UNWATCH, w->key));
    return OK;
}

int TcpStoreClient::QueryAlive(uint32_t rank, bool &alive)
{
    int16_t st = 0;
    std::string rep;
    int rc = Request(StoreMessage(MT_QUERY_ALIVE, std::to_string(rank)), st, rep, kRpcWaitMs);
    if (rc != OK) return rc;
    if (st != ST_OK) return MapStatus(st);
    StoreMessage r;
    if (!StoreMessage::Unpack(rep, r)) return ERR;
    alive = !r.values.empty();
    return OK;
}

int TcpStoreClient::AutoRank(uint32_t &rank)
{
    StoreMessage m(MT_GET, kAutoRankKey);
    m.userDef = 0;
    int16_t st = 0;
    std::string rep;
    int rc = Request(m, st, rep, kRpcWaitMs);
    if (rc != OK) return rc;
    if (st != ST_OK) return MF_FAIL(ERR_NO_RESOURCES, "store refused to assign a rank: %s", rep.c_str());
    StoreMessage r;
    if (!StoreMessage::Unpack(rep, r) || r.values.size() != 1 || r.values[0].size() != sizeof(uint32_t)) return ERR;
    memcpy(&rank, r.values[0].data(), sizeof(rank));
    rank_ = rank;
    return OK;
}

void TcpStoreClient::RegisterReconnectHandler(ReconnectFn fn)
{
    std::lock_guard<std::mutex> g(cbMu_);
    reconnectFns_.push_back(std::move(fn));
}

void TcpStoreClient::RegisterBrokenHandler(BrokenFn fn)
{
    std::lock_guard<std::mutex> g(cbMu_);
    brokenFns_.push_back(std::move(fn));
}

}  // namespace store
}  // namespace mf
