// Highly available config store: several candidate processes share a distributed backend; one of
// them is elected leader and runs the StoreServer, the rest are followers whose calls are forwarded
// to the leader. Election: random back-off 100-1000 ms -> connect backend -> if the registered
// leader answers a TCP probe become follower -> else take the backend lock "backend", re-check, start
// a server on the first free port at or above the URL's port (restoring world size and alive ranks
// unless first leader), publish "ip:port" under the leader key with a 5 s lease that a 4 s health
// thread keeps renewing; a leader that cannot reach the backend demotes itself; a broken client link
// triggers re-election on one worker thread.
// Parity: src/smem/csrc/config_store/ha/smem_ha_config_store.cpp:155-298,304-373,406-536,551-698,
// doc/config_store_cluster_ha.md:189-407.
#pragma once
#include "mf_store.h"
#include "mf_store_backend.h"

namespace mf {
namespace store {

class HaConfigStore : public ConfigStore, public std::enable_shared_from_this<HaConfigStore> {
public:
    HaConfigStore(std::string ip, uint16_t basePort, uint32_t worldSize, uint32_t rank, BackendPtr backend,
                  bool candidate);
    ~HaConfigStore() override;
    int Startup(uint32_t timeoutMs);
    void Shutdown();
    bool IsLeader() const { return leader_.load(); }
    std::string LeaderAddress();
    // Test knobs (milliseconds): lease TTL, health period, back-off range.
    void SetTimings(uint32_t leaseMs, uint32_t healthMs, uint32_t backoffLoMs, uint32_t backoffHiMs);
    // Test hook: a leader stops serving as if its process died (no lease cleanup).
    void KillLeaderServer();

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
    bool Connected() const override;
    uint32_t Rank() const override { return rank_; }

private:
    int Elect(uint32_t timeoutMs);
    int BecomeLeader(bool first);
    int FollowLeader(const std::string &addr);
    void HealthLoop();
    void Demote();
    std::shared_ptr<TcpStoreClient> Client();
    void ScheduleReelect();

    std::string ip_;
    uint16_t basePort_;
    uint32_t worldSize_;
    uint32_t rank_;
    BackendPtr backend_;
    std::atomic<bool> candidate_;
    std::atomic<bool> leader_{false};
    std::atomic<bool> running_{false};
    std::mutex mu_;
    std::shared_ptr<StoreServer> server_;
    std::shared_ptr<TcpStoreClient> client_;
    std::string leaderAddr_;
    std::thread health_;
    std::thread elector_;
    std::mutex cvMu_;
    std::condition_variable cv_;
    std::atomic<bool> reelect_{false};
    std::atomic<bool> everFollowed_{false};
    std::vector<ReconnectFn> reconnectFns_;
    std::vector<BrokenFn> brokenFns_;
    struct SavedWatch {
        std::string key;
        WatchFn fn;
        RankDownFn rankFn;
        uint32_t innerId = 0;
    };
    std::map<uint32_t, SavedWatch> watches_;
    uint32_t nextWatch_ = 1;
    uint32_t leaseMs_ = 5000, healthMs_ = 4000, backoffLo_ = 100, backoffHi_ = 1000;
};

}  // namespace store
}  // namespace mf
