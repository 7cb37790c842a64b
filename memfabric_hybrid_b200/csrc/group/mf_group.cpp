#include "mf_group.h"

#include <algorithm>

#include "../util/mf_trace.h"

namespace mf {
namespace group {

namespace {
const char *kEventKey = "EVENT";
const char *kExitKey = "EXIT";
const char *kNumKey = "AT_NUM";
constexpr uint32_t kStaleEventMs = 3000;

std::string Ser(const GroupInfo &g) { return std::string(reinterpret_cast<const char *>(&g), sizeof(g)); }
bool De(const std::string &s, GroupInfo &g)
{
    if (s.size() != sizeof(GroupInfo)) return false;
    memcpy(&g, s.data(), sizeof(g));
    return true;
}
uint64_t RetryMs() { return (uint64_t)EnvInt("MF_GROUP_RETRY_TIME", "SMEM_GROUP_RETRY_TIME", 100, 1, 60000); }
uint64_t JoinMaxMs()
{
    return 1000ULL * (uint64_t)EnvInt("MF_GROUP_JOIN_MAX_TIMEOUT", "SMEM_GROUP_JOIN_MAX_TIMEOUT", 600, 1, 86400);
}
}  // namespace

std::shared_ptr<GroupEngine> GroupEngine::Create(const store::StorePtr &st, const GroupOption &opt)
{
    if (!st || opt.rankSize == 0 || opt.rankSize > kMaxRanks || (!opt.dynamic && opt.rank >= opt.rankSize)) {
        MF_FAIL(ERR_INVALID_PARAM, "group engine: bad option (size %u rank %u)", opt.rankSize, opt.rank);
        return nullptr;
    }
    auto g = std::make_shared<GroupEngine>(st, opt);
    auto alive = g->alive_;
    GroupEngine *raw = g.get();
    st->RegisterReconnectHandler([raw, alive]() -> int {
        if (!alive->load()) return OK;
        // A restarted store lost every key: put our membership record back if nobody has yet.
        if (raw->opt_.dynamic && raw->joined_) {
            GroupInfo mine = raw->Info();
            std::string existing;
            raw->store_->Cas(kEventKey, "", Ser(mine), existing);
        }
        raw->changeEpoch_.fetch_add(1);
        return OK;
    });
    return g;
}

GroupEngine::GroupEngine(store::StorePtr st, const GroupOption &opt) : store_(std::move(st)), opt_(opt)
{
    joined_ = !opt.dynamic;
    info_.groupSize = opt.dynamic ? 0 : opt.rankSize;
    if (!opt.dynamic)
        for (uint32_t r = 0; r < opt.rankSize; r++) info_.Put(r);
}

GroupEngine::~GroupEngine()
{
    alive_->store(false);
    StopListen();
}

GroupInfo GroupEngine::Info()
{
    std::lock_guard<std::mutex> g(mu_);
    return info_;
}

uint32_t GroupEngine::RankSize()
{
    std::lock_guard<std::mutex> g(mu_);
    return info_.groupSize;
}

int GroupEngine::WaitKey(const std::string &key, uint64_t timeoutMs, std::string &out)
{
    // Blocks on the server side in slices so that a membership change can interrupt the wait.
    uint64_t deadline = NowMs() + timeoutMs;
    uint32_t epoch = changeEpoch_.load();
    for (;;) {
        uint64_t now = NowMs();
        if (now >= deadline) return ERR_TIMEOUT;
        int64_t slice = (int64_t)std::min<uint64_t>(deadline - now, 1000);
        int rc = store_->Get(key, out, slice);
        if (rc == OK) return OK;
        if (rc != ERR_TIMEOUT) return rc;
        if (opt_.dynamic && changeEpoch_.load() != epoch && eventOpVersion_ == 0) return ERR_BUSY;
    }
}

void GroupEngine::GcKey(const std::string &base, uint32_t sn)
{
    if (sn < kKeyGcLag) return;
    std::string old = base + std::to_string(sn - kKeyGcLag);
    store_->Remove(old + "_BA", true);
    store_->Remove(old + "_BW", true);
    store_->Remove(old + "_GA", true);
    store_->Remove(old + "_GW", true);
}

int GroupEngine::BarrierImpl(const std::string &base, uint32_t size)
{
    uint64_t t0 = NowNs();
    int64_t n = 0;
    int rc = store_->Add(base + "_BA", 1, n);
    if (rc != OK) return rc;
    if ((uint32_t)n == size) {
        rc = store_->Set(base + "_BW", "ok");
        if (rc != OK) return rc;
    }
    std::string v;
    rc = WaitKey(base + "_BW", opt_.timeoutMs, v);
    MF_DEBUG("barrier %s size %u done rc %d in %.1f us", base.c_str(), size, rc, (NowNs() - t0) / 1000.0);
    return rc;
}

int GroupEngine::GatherImpl(const std::string &base, uint32_t size, uint32_t rank, const char *send, uint32_t sendSize,
                            char *recv, uint32_t recvSize)
{
    if (send == nullptr || recv == nullptr || sendSize == 0 || (uint64_t)sendSize * size > recvSize)
        return MF_FAIL(ERR_INVALID_PARAM, "allgather: buffers do not fit (%u x %u into %u)", sendSize, size, recvSize);
    std::string blob(reinterpret_cast<const char *>(&rank), sizeof(rank));
    blob.append(send, sendSize);
    uint64_t total = 0;
    int rc = store_->Append(base + "_GA", blob, total);
    if (rc != OK) return rc;
    uint64_t piece = sizeof(uint32_t) + sendSize;
    if (total == piece * size) {
        rc = store_->Set(base + "_GW", "ok");
        if (rc != OK) return rc;
    }
    std::string v;
    rc = WaitKey(base + "_GW", opt_.timeoutMs, v);
    if (rc != OK) return rc;
    rc = store_->Get(base + "_GA", v, 0);
    if (rc != OK) return rc;
    if (v.size() != piece * size) return MF_FAIL(ERR, "allgather %s: %zu bytes gathered, want %lu", base.c_str(), v.size(), (unsigned long)(piece * size));
    std::vector<bool> seen(kMaxRanks, false);
    std::vector<std::pair<uint32_t, const char *>> parts;
    for (uint32_t i = 0; i < size; i++) {
        uint32_t r;
        memcpy(&r, v.data() + i * piece, sizeof(r));
        if (r >= kMaxRanks || seen[r]) return MF_FAIL(ERR, "allgather %s: bad or duplicate rank tag %u", base.c_str(), r);
        seen[r] = true;
        parts.emplace_back(r, v.data() + i * piece + sizeof(r));
    }
    std::sort(parts.begin(), parts.end(), [](auto &a, auto &b) { return a.first < b.first; });
    for (uint32_t i = 0; i < size; i++) memcpy(recv + (uint64_t)i * sendSize, parts[i].second, sendSize);
    return OK;
}

int GroupEngine::Barrier()
{
    MF_TRACE_BEGIN(TP_GROUP_BARRIER);
    uint32_t sn, size, ver;
    {
        std::lock_guard<std::mutex> g(mu_);
        sn = barrierSn_++;
        size = info_.groupSize;
        ver = opt_.dynamic ? info_.version : 0;
    }
    std::string base = std::to_string(ver) + "_";
    int rc = size == 0 ? ERR_NOT_STARTED : BarrierImpl(base + std::to_string(sn), size);
    if (rc == OK && opt_.rank == 0) GcKey(base, sn);
    MF_TRACE_END(TP_GROUP_BARRIER, rc);
    return rc;
}

int GroupEngine::AllGather(const char *send, uint32_t sendSize, char *recv, uint32_t recvSize)
{
    MF_TRACE_BEGIN(TP_GROUP_ALLGATHER);
    uint32_t sn, size, ver;
    {
        std::lock_guard<std::mutex> g(mu_);
        sn = gatherSn_++;
        size = info_.groupSize;
        ver = opt_.dynamic ? info_.version : 0;
    }
    std::string base = std::to_string(ver) + "_g";
    int rc = size == 0 ? ERR_NOT_STARTED : GatherImpl(base + std::to_string(sn), size, opt_.rank, send, sendSize, recv, recvSize);
    if (rc == OK && opt_.rank == 0) GcKey(base, sn);
    MF_TRACE_END(TP_GROUP_ALLGATHER, rc);
    return rc;
}

int GroupEngine::Barrier(const char *key, uint32_t rankSize, uint32_t rankId)
{
    if (key == nullptr || *key == 0 || rankSize == 0 || rankId >= rankSize) return ERR_INVALID_PARAM;
    uint32_t sn;
    {
        std::lock_guard<std::mutex> g(mu_);
        sn = subSn_[std::string("b:") + key]++;
    }
    std::string base = std::string(key) + "_";
    int rc = BarrierImpl(base + std::to_string(sn), rankSize);
    if (rc == OK && rankId == 0) GcKey(base, sn);
    return rc;
}

int GroupEngine::AllGather(const char *key, uint32_t rankSize, uint32_t rankId, const char *send, uint32_t sendSize,
                           char *recv, uint32_t recvSize)
{
    if (key == nullptr || *key == 0 || rankSize == 0 || rankId >= rankSize) return ERR_INVALID_PARAM;
    uint32_t sn;
    {
        std::lock_guard<std::mutex> g(mu_);
        sn = subSn_[std::string("g:") + key]++;
    }
    std::string base = std::string(key) + "_g";
    int rc = GatherImpl(base + std::to_string(sn), rankSize, rankId, send, sendSize, recv, recvSize);
    if (rc == OK && rankId == 0) GcKey(base, sn);
    return rc;
}

int GroupEngine::EventBarrier()
{
    uint32_t sn, size, ver;
    {
        std::lock_guard<std::mutex> g(mu_);
        if (eventOpVersion_ == 0) return ERR_NOT_STARTED;
        sn = eventOpSn_++;
        size = info_.groupSize;
        ver = eventOpVersion_;
    }
    return BarrierImpl("EV" + std::to_string(ver) + "_" + std::to_string(sn), size);
}

int GroupEngine::EventGatherResult(int32_t mine)
{
    uint32_t sn, size, ver;
    {
        std::lock_guard<std::mutex> g(mu_);
        if (eventOpVersion_ == 0) return ERR_NOT_STARTED;
        sn = eventOpSn_++;
        size = info_.groupSize;
        ver = eventOpVersion_;
    }
    std::vector<int32_t> all(size, 0);
    int rc = GatherImpl("EV" + std::to_string(ver) + "_" + std::to_string(sn), size, opt_.rank,
                        reinterpret_cast<const char *>(&mine), sizeof(mine), reinterpret_cast<char *>(all.data()),
                        (uint32_t)(all.size() * sizeof(int32_t)));
    if (rc != OK) return rc;
    for (auto v : all)
        if (v != 0) return v;
    return OK;
}

int GroupEngine::BroadcastExit(int status) { return store_->Set(kExitKey, std::to_string(status)); }

int GroupEngine::RegisterExit(std::function<void(int)> cb)
{
    exitCb_ = std::move(cb);
    auto alive = alive_;
    return store_->Watch(
        kExitKey,
        [this, alive](int rc, const std::string &, const std::string &v) {
            if (!alive->load() || rc != OK || !exitCb_) return;
            int64_t st = 0;
            ParseI64(v, st);
            exitCb_((int)st);
        },
        exitWatch_);
}

int GroupEngine::AllocNumber(uint32_t limit, int32_t &value)
{
    if (limit == 0 || limit > kMaxRanks) return ERR_INVALID_PARAM;
    for (int attempt = 0; attempt < 4096; attempt++) {
        std::string cur;
        int rc = store_->Get(kNumKey, cur, 0);
        if (rc != OK && rc != ERR_NOT_EXIST) return rc;
        std::string next = cur;
        if (next.size() != kMaxRanks / 8) next.assign(kMaxRanks / 8, '\0');
        int32_t found = -1;
        for (uint32_t i = 0; i < limit; i++) {
            if (((uint8_t)next[i / 8] >> (i % 8) & 1) == 0) {
                found = (int32_t)i;
                next[i / 8] = (char)((uint8_t)next[i / 8] | (1u << (i % 8)));
                break;
            }
        }
        if (found < 0) return MF_FAIL(ERR_NO_RESOURCES, "no free number below %u", limit);
        std::string existing;
        rc = store_->Cas(kNumKey, cur, next, existing);
        if (rc == OK) {
            value = found;
            return OK;
        }
        if (rc != ERR_IN_USE) return rc;
    }
    return ERR_BUSY;
}

int GroupEngine::ReleaseNumber(int32_t value)
{
    if (value < 0 || (uint32_t)value >= kMaxRanks) return ERR_INVALID_PARAM;
    for (int attempt = 0; attempt < 4096; attempt++) {
        std::string cur;
        int rc = store_->Get(kNumKey, cur, 0);
        if (rc == ERR_NOT_EXIST) return OK;
        if (rc != OK) return rc;
        if (cur.size() != kMaxRanks / 8) return ERR;
        std::string next = cur;
        next[value / 8] = (char)((uint8_t)next[value / 8] & ~(1u << (value % 8)));
        std::string existing;
        rc = store_->Cas(kNumKey, cur, next, existing);
        if (rc == OK) return OK;
        if (rc != ERR_IN_USE) return rc;
    }
    return ERR_BUSY;
}

// ------------------------------------------------------------------------------------------------
int GroupEngine::ReadEvent(GroupInfo &info, bool &exists)
{
    std::string v;
    int rc = store_->Get(kEventKey, v, 0);
    if (rc == ERR_NOT_EXIST) {
        exists = false;
        info = GroupInfo();
        return OK;
    }
    if (rc != OK) return rc;
    exists = true;
    return De(v, info) ? OK : MF_FAIL(ERR, "EVENT record has %zu bytes, want %zu", v.size(), sizeof(GroupInfo));
}

int GroupEngine::StartListen()
{
    if (!opt_.dynamic || listening_.exchange(true)) return OK;
    listener_ = std::thread([this] {
        pthread_setname_np(pthread_self(), "mf-group-listen");
        ListenLoop();
    });
    auto alive = alive_;
    int rc = store_->Watch(
        kEventKey,
        [this, alive](int rc2, const std::string &, const std::string &v) {
            GroupInfo gi;
            if (!alive->load() || rc2 != OK || !De(v, gi)) return;
            std::lock_guard<std::mutex> g(qMu_);
            evQueue_.push_back(gi);
            qCv_.notify_all();
        },
        eventWatch_);
    if (rc != OK) return rc;
    return store_->WatchRankState(
        [this, alive](uint32_t rank) {
            if (!alive->load()) return;
            std::lock_guard<std::mutex> g(qMu_);
            downQueue_.push_back(rank);
            qCv_.notify_all();
        },
        rankWatch_);
}

void GroupEngine::StopListen()
{
    if (!listening_.exchange(false)) return;
    if (eventWatch_ != 0) store_->Unwatch(eventWatch_);
    if (rankWatch_ != 0) store_->Unwatch(rankWatch_);
    if (exitWatch_ != 0) store_->Unwatch(exitWatch_);
    {
        std::lock_guard<std::mutex> g(qMu_);
        qCv_.notify_all();
    }
    JoinOrDetach(listener_);
}

void GroupEngine::ListenLoop()
{
    while (listening_) {
        GroupInfo ev;
        uint32_t down = 0;
        int kind = 0;
        {
            std::unique_lock<std::mutex> lk(qMu_);
            qCv_.wait_for(lk, std::chrono::milliseconds(500),
                          [this] { return !listening_ || !evQueue_.empty() || !downQueue_.empty(); });
            if (!listening_) return;
            if (!evQueue_.empty()) {
                ev = evQueue_.front();
                evQueue_.pop_front();
                kind = 1;
            } else if (!downQueue_.empty()) {
                down = downQueue_.front();
                downQueue_.pop_front();
                kind = 2;
            }
        }
        if (kind == 1) HandleEvent(ev);
        else if (kind == 2) HandleRankDown(down);
    }
}

void GroupEngine::HandleEvent(const GroupInfo &ev)
{
    if (ev.version <= lastHandledVersion_ && ev.version != 0) return;
    lastHandledVersion_ = ev.version;
    if (ev.curEvent == EV_NULL || (ev.version & 1u) == 0) {
        // finalised: adopt the membership view
        if (joined_) {
            std::lock_guard<std::mutex> g(mu_);
            // a notification can arrive after this rank already posted a NEWER event of its own
            // (its main thread does not wait for the watch): never step back to an older record
            if (ev.Has(opt_.rank) && ev.version > info_.version) {
                info_ = ev;
                eventOpVersion_ = 0;
            }
        }
        changeEpoch_.fetch_add(1);
        return;
    }
    changeEpoch_.fetch_add(1);
    if (ev.submitRank == opt_.rank) return;  // the submitting thread drives its own event
    if (!joined_) return;
    if (ev.targetRank >= kMaxRanks || ev.submitRank >= kMaxRanks) {
        MF_WARN("group event %u names rank %u (from rank %u): outside the %u ranks a group can have, ignored", ev.curEvent, ev.targetRank, ev.submitRank,
                kMaxRanks);
        return;
    }
    ChangeFn cb;
    bool hadTarget;
    {
        std::lock_guard<std::mutex> g(mu_);
        hadTarget = info_.Has(ev.targetRank);
        if (ev.version > info_.version) {
            info_ = ev;
            eventOpVersion_ = ev.version;
            eventOpSn_ = 0;
        }
    }
    int rc = OK;
    switch (ev.curEvent) {
        case EV_JOIN:
            // A rank that re-joins under an id we still hold is first dropped, then imported afresh.
            // (the link-down handler: it drops the imports without the leave protocol's barrier)
            if (hadTarget && opt_.linkDownCb) opt_.linkDownCb(ev.targetRank);
            if (opt_.joinCb) rc = opt_.joinCb(ev.targetRank);
            break;
        case EV_UPDATE:
            if (opt_.updateCb) rc = opt_.updateCb(ev.targetRank);
            break;
        case EV_LEAVE:
            if (opt_.leaveCb) rc = opt_.leaveCb(ev.targetRank);
            break;
        case EV_LINK_DOWN:
            if (opt_.linkDownCb) rc = opt_.linkDownCb(ev.targetRank);
            break;
        default:
            break;
    }
    if (rc != OK) MF_WARN("group event %u for rank %u: handler returned %d", ev.curEvent, ev.targetRank, rc);
}

void GroupEngine::CleanStaleEvent(const GroupInfo &ev)
{
    // An event left in flight by a submitter that died is rolled back by whoever notices first.
    uint64_t now = NowMs();
    if (inflightVersion_ != ev.version) {
        inflightVersion_ = ev.version;
        inflightSinceMs_ = now;
        return;
    }
    if (now - inflightSinceMs_ < kStaleEventMs) return;
    bool alive = true;
    if (store_->QueryAlive(ev.submitRank, alive) != OK || alive) return;
    GroupInfo fixed = ev;
    fixed.version = ev.version + 1;
    fixed.curEvent = EV_NULL;
    fixed.Drop(ev.submitRank);
    if (ev.curEvent == EV_JOIN) fixed.Drop(ev.targetRank);
    fixed.groupSize = fixed.Count();
    std::string existing;
    if (store_->Cas(kEventKey, Ser(ev), Ser(fixed), existing) == OK)
        MF_WARN("rolled back stale group event %u left by dead rank %u", ev.curEvent, ev.submitRank);
}

int GroupEngine::SubmitEvent(EventType evType, uint32_t target, GroupInfo &posted)
{
    uint64_t deadline = NowMs() + JoinMaxMs();
    for (;;) {
        GroupInfo cur;
        bool exists = false;
        int rc = ReadEvent(cur, exists);
        if (rc != OK) return rc;
        if (exists && (cur.curEvent != EV_NULL || (cur.version & 1u))) {
            CleanStaleEvent(cur);
            if (NowMs() >= deadline) return MF_FAIL(ERR_TIMEOUT, "group is busy with event %u of rank %u", cur.curEvent, cur.submitRank);
            std::this_thread::sleep_for(std::chrono::milliseconds(RetryMs()));
            continue;
        }
        GroupInfo next = cur;
        next.version = cur.version + 1;
        next.curEvent = evType;
        next.targetRank = target;
        next.submitRank = opt_.rank;
        switch (evType) {
            case EV_JOIN: next.Put(target); break;
            case EV_LINK_DOWN: next.Drop(target); break;
            default: break;
        }
        if (evType == EV_LINK_DOWN && !cur.Has(target)) return ERR_NOT_EXIST;
        if ((evType == EV_LEAVE || evType == EV_UPDATE) && !cur.Has(target)) return MF_FAIL(ERR_NOT_EXIST, "rank %u is not a member", target);
        next.groupSize = next.Count();
        std::string existing;
        rc = store_->Cas(kEventKey, exists ? Ser(cur) : std::string(), Ser(next), existing);
        if (rc == OK) {
            posted = next;
            return OK;
        }
        if (rc != ERR_IN_USE) return rc;
        if (NowMs() >= deadline) return ERR_TIMEOUT;
    }
}

int GroupEngine::FinishEvent(const GroupInfo &posted, bool keepTarget)
{
    GroupInfo fin = posted;
    fin.version = posted.version + 1;
    fin.curEvent = EV_NULL;
    if (!keepTarget) fin.Drop(posted.targetRank);
    fin.groupSize = fin.Count();
    std::string existing;
    int rc = store_->Cas(kEventKey, Ser(posted), Ser(fin), existing);
    if (rc != OK) MF_WARN("finishing group event %u: CAS returned %d", posted.curEvent, rc);
    std::lock_guard<std::mutex> g(mu_);
    eventOpVersion_ = 0;
    if (fin.Has(opt_.rank)) info_ = fin;
    return rc;
}

int GroupEngine::Join()
{
    if (!opt_.dynamic) return OK;
    if (joined_) return MF_FAIL(ERR_REPEAT, "rank %u already joined", opt_.rank);
    MF_TRACE_BEGIN(TP_GROUP_JOIN);
    int rc = StartListen();
    GroupInfo posted;
    if (rc == OK) rc = SubmitEvent(EV_JOIN, opt_.rank, posted);
    if (rc == OK) {
        {
            std::lock_guard<std::mutex> g(mu_);
            info_ = posted;
            eventOpVersion_ = posted.version;
            eventOpSn_ = 0;
        }
        joined_ = true;
        int cbRc = opt_.joinCb ? opt_.joinCb(opt_.rank) : OK;
        if (cbRc != OK) {
            joined_ = false;
            FinishEvent(posted, false);  // roll ourselves back out
            rc = cbRc;
        } else {
            rc = FinishEvent(posted, true);
        }
    }
    MF_TRACE_END(TP_GROUP_JOIN, rc);
    return rc;
}

int GroupEngine::Update()
{
    if (!opt_.dynamic) return OK;
    if (!joined_) return ERR_NOT_STARTED;
    GroupInfo posted;
    int rc = SubmitEvent(EV_UPDATE, opt_.rank, posted);
    if (rc != OK) return rc;
    {
        std::lock_guard<std::mutex> g(mu_);
        info_ = posted;
        eventOpVersion_ = posted.version;
        eventOpSn_ = 0;
    }
    int cbRc = opt_.updateCb ? opt_.updateCb(opt_.rank) : OK;
    rc = FinishEvent(posted, true);
    return cbRc != OK ? cbRc : rc;
}

int GroupEngine::Leave()
{
    if (!opt_.dynamic) return OK;
    if (!joined_) return ERR_NOT_STARTED;
    MF_TRACE_BEGIN(TP_GROUP_LEAVE);
    GroupInfo posted;
    int rc = SubmitEvent(EV_LEAVE, opt_.rank, posted);
    if (rc == OK) {
        {
            std::lock_guard<std::mutex> g(mu_);
            info_ = posted;
            eventOpVersion_ = posted.version;
            eventOpSn_ = 0;
        }
        int cbRc = opt_.leaveCb ? opt_.leaveCb(opt_.rank) : OK;
        rc = FinishEvent(posted, false);
        joined_ = false;
        {
            std::lock_guard<std::mutex> g(mu_);
            info_ = GroupInfo();
        }
        if (cbRc != OK) rc = cbRc;
    }
    MF_TRACE_END(TP_GROUP_LEAVE, rc);
    return rc;
}

void GroupEngine::HandleRankDown(uint32_t rank)
{
    changeEpoch_.fetch_add(1);
    if (!joined_ || rank == opt_.rank) return;
    {
        std::lock_guard<std::mutex> g(mu_);
        if (!info_.Has(rank)) return;
    }
    GroupInfo posted;
    int rc = SubmitEvent(EV_LINK_DOWN, rank, posted);
    if (rc != OK) return;  // ERR_NOT_EXIST: another member already recorded it
    {
        std::lock_guard<std::mutex> g(mu_);
        info_ = posted;
    }
    if (opt_.linkDownCb) opt_.linkDownCb(rank);
    FinishEvent(posted, true);  // the bitmap already excludes the dead rank
}

}  // namespace group
}  // namespace mf
