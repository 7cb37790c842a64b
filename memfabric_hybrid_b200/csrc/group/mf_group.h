// Group engine: collective control-plane operations built only on config-store primitives.
//   static groups  : barrier (ADD counter + wait key), allgather (APPEND rank-tagged blobs, sorted),
//                    sub-group variants keyed by a user string, exit broadcast, unique-number bitmap
//   dynamic groups : join / update / leave / link-down as a CAS'd EVENT record that every member
//                    watches; an odd version means "event in flight", the submitter finalises it back
//                    to an even version once every member's callback ran.
// Store keys (under the caller's prefix): "<ver>_<sn>_BA|_BW|_GA|_GW", "<userKey>_<sn>_BA|...",
// "EVENT", "BMEX_<rank>", "AT_NUM", "EXIT".
// Parity: src/smem/csrc/net/smem_net_group_engine.{h,cpp} (barrier :145-209, allgather :211-275,
// sub-groups :277-320,522-570, alloc-number :617-675, listeners :905-1148, join/leave :1352-1534,
// reconnect :1549-1588, key GC :1590-1628).
#pragma once
#include "../store/mf_store.h"

namespace mf {
namespace group {

constexpr uint32_t kMaxRanks = 1024;
constexpr uint32_t kBitmapWords = kMaxRanks / 64;
constexpr uint32_t kKeyGcLag = 2;  // barrier/allgather keys are removed this many rounds later

enum EventType : int32_t {
    EV_JOIN = 0,
    EV_LEAVE = 1,
    EV_RECOVER = 2,
    EV_LINK_DOWN = 3,
    EV_UPDATE = 4,
    EV_NULL = 5,
    EV_STOP = 6,
};

#pragma pack(push, 4)
struct GroupInfo {
    uint32_t version = 0;
    uint32_t groupSize = 0;
    uint32_t curEvent = EV_NULL;
    uint32_t targetRank = 0;
    uint32_t submitRank = 0;
    uint64_t bitmap[kBitmapWords] = {0};
    bool Has(uint32_t r) const { return r < kMaxRanks && (bitmap[r / 64] >> (r % 64)) & 1ULL; }
    // (rank numbers arrive in records written by other processes: one outside the bitmap changes nothing)
    void Put(uint32_t r)
    {
        if (r < kMaxRanks) bitmap[r / 64] |= 1ULL << (r % 64);
    }
    void Drop(uint32_t r)
    {
        if (r < kMaxRanks) bitmap[r / 64] &= ~(1ULL << (r % 64));
    }
    uint32_t Count() const
    {
        uint32_t n = 0;
        for (uint32_t i = 0; i < kBitmapWords; i++) n += (uint32_t)__builtin_popcountll(bitmap[i]);  // packed: no references
        return n;
    }
};
#pragma pack(pop)
static_assert(sizeof(GroupInfo) == 20 + 8 * kBitmapWords, "EVENT record layout");

using ChangeFn = std::function<int(uint32_t rank)>;

struct GroupOption {
    uint32_t rankSize = 0;
    uint32_t rank = 0;
    uint64_t timeoutMs = 120000;
    bool dynamic = false;
    ChangeFn joinCb, updateCb, leaveCb, linkDownCb;
};

class GroupEngine : public std::enable_shared_from_this<GroupEngine> {
public:
    static std::shared_ptr<GroupEngine> Create(const store::StorePtr &st, const GroupOption &opt);
    GroupEngine(store::StorePtr st, const GroupOption &opt);
    ~GroupEngine();

    // ---- static collectives over the current member set
    int Barrier();
    int AllGather(const char *send, uint32_t sendSize, char *recv, uint32_t recvSize);
    int Barrier(const char *key, uint32_t rankSize, uint32_t rankId);
    int AllGather(const char *key, uint32_t rankSize, uint32_t rankId, const char *send, uint32_t sendSize, char *recv,
                  uint32_t recvSize);
    // Barrier among the members of an in-flight event (keys scoped by the event version).
    int EventBarrier();
    // AllGather of int results among event members; returns the first non-zero result.
    int EventGatherResult(int32_t mine);

    int BroadcastExit(int status);
    int RegisterExit(std::function<void(int)> cb);
    int AllocNumber(uint32_t limit, int32_t &value);
    int ReleaseNumber(int32_t value);

    // ---- dynamic membership
    int StartListen();
    void StopListen();
    int Join();
    int Update();
    int Leave();
    bool Joined() const { return joined_.load(); }
    GroupInfo Info();
    uint32_t Rank() const { return opt_.rank; }
    uint32_t RankSize();
    const store::StorePtr &Store() const { return store_; }
    // Counters that interrupt blocking waits when membership changes under them.
    uint32_t ChangeEpoch() const { return changeEpoch_.load(); }

private:
    struct Pending {
        GroupInfo info;
    };
    int WaitKey(const std::string &key, uint64_t timeoutMs, std::string &out);
    int BarrierImpl(const std::string &base, uint32_t size);
    int GatherImpl(const std::string &base, uint32_t size, uint32_t rank, const char *send, uint32_t sendSize,
                   char *recv, uint32_t recvSize);
    int SubmitEvent(EventType ev, uint32_t target, GroupInfo &posted);
    int FinishEvent(const GroupInfo &posted, bool keepTarget);
    void ListenLoop();
    void HandleEvent(const GroupInfo &info);
    void HandleRankDown(uint32_t rank);
    void CleanStaleEvent(const GroupInfo &info);
    int ReadEvent(GroupInfo &info, bool &exists);
    void GcKey(const std::string &base, uint32_t sn);

    store::StorePtr store_;
    GroupOption opt_;
    std::mutex mu_;
    GroupInfo info_;
    std::atomic<bool> joined_{false};
    uint32_t barrierSn_ = 0;
    uint32_t gatherSn_ = 0;
    uint32_t eventOpSn_ = 0;      // per in-flight event, reset when a new event starts
    uint32_t eventOpVersion_ = 0;
    std::map<std::string, uint32_t> subSn_;
    std::thread listener_;
    std::mutex qMu_;
    std::condition_variable qCv_;
    std::deque<GroupInfo> evQueue_;
    std::deque<uint32_t> downQueue_;
    std::atomic<bool> listening_{false};
    uint32_t eventWatch_ = 0, rankWatch_ = 0, exitWatch_ = 0;
    uint32_t lastHandledVersion_ = 0;
    std::atomic<uint32_t> changeEpoch_{0};
    std::function<void(int)> exitCb_;
    std::shared_ptr<std::atomic<bool>> alive_ = std::make_shared<std::atomic<bool>>(true);
    uint64_t inflightSinceMs_ = 0;
    uint32_t inflightVersion_ = 0;
};
using GroupPtr = std::shared_ptr<GroupEngine>;

}  // namespace group
}  // namespace mf
