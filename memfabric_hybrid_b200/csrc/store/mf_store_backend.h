// Durable/distributed backends behind the config store. The store server persists its world size and
// alive-rank list here; the HA store elects a leader through it. Implementations: process-local map
// (tests and single-node runs) and an adapter over a user-supplied C op table (how etcd or any other
// service is attached without linking it).
// Parity: src/smem/csrc/config_store/backend/smem_config_store_backend.h:31-35,47-192,202-315,
// backend/smem_local_memory_backend.cpp, backend/smem_external_backend.cpp, src/smem/include/host/smem_def.h:44-96.
#pragma once
#include "../include/smem_def.h"
#include "mf_store.h"

namespace mf {
namespace store {

constexpr const char *kBackendKeyLeader = "/memfabric_hybrid/config_store/meta/leader";
constexpr const char *kBackendKeyLeaderStatus = "/memfabric_hybrid/config_store/meta/leader_status";
constexpr const char *kBackendKeyWorldSize = "/memfabric_hybrid/config_store/data/world_size";
constexpr const char *kBackendKeyAliveRanks = "/memfabric_hybrid/config_store/data/alive_rank_list";

class StoreBackend {
public:
    virtual ~StoreBackend() = default;
    virtual bool Distributed() const = 0;
    virtual int Connect() { return OK; }
    virtual int Put(const std::string &key, const std::string &value, uint32_t ttlMs) = 0;
    virtual int Get(const std::string &key, std::string &value) = 0;
    virtual int PrefixGet(const std::string &prefix, std::vector<std::pair<std::string, std::string>> &out) = 0;
    virtual int Delete(const std::string &key) = 0;
    virtual bool Exist(const std::string &key)
    {
        std::string v;
        return Get(key, v) == OK;
    }
    virtual int Clear(const std::string &prefix) = 0;
    virtual int Lock(const std::string &name) = 0;
    virtual int TryLock(const std::string &name) = 0;
    virtual int Unlock(const std::string &name) = 0;
};
using BackendPtr = std::shared_ptr<StoreBackend>;

// RAII guard over a backend's named lock.
class DistributedLockGuard {
public:
    DistributedLockGuard(BackendPtr b, std::string name) : b_(std::move(b)), name_(std::move(name))
    {
        held_ = b_ && b_->Lock(name_) == OK;
    }
    ~DistributedLockGuard()
    {
        if (held_) b_->Unlock(name_);
    }
    bool Held() const { return held_; }

private:
    BackendPtr b_;
    std::string name_;
    bool held_ = false;
};

// In-process backend with TTL support. Instances created with the same name share one map, so
// several "nodes" inside one test process see the same state.
class LocalMemoryBackend : public StoreBackend {
public:
    explicit LocalMemoryBackend(const std::string &name = "default", bool pretendDistributed = false);
    bool Distributed() const override { return distributed_; }
    int Connect() override;
    int Put(const std::string &key, const std::string &value, uint32_t ttlMs) override;
    int Get(const std::string &key, std::string &value) override;
    int PrefixGet(const std::string &prefix, std::vector<std::pair<std::string, std::string>> &out) override;
    int Delete(const std::string &key) override;
    int Clear(const std::string &prefix) override;
    int Lock(const std::string &name) override;
    int TryLock(const std::string &name) override;
    int Unlock(const std::string &name) override;
    // Test hook: make every call fail, as an unreachable service would.
    static void SetReachable(const std::string &name, bool reachable);
    static void Reset(const std::string &name);
    struct Shared;

private:
    std::shared_ptr<Shared> s_;
    bool distributed_;
};

// Adapter over smem_conf_store_backend_op_t.
class ExternalBackend : public StoreBackend {
public:
    ExternalBackend(const smem_conf_store_backend_op_t &ops, const std::string &name, const std::string &prefix);
    ~ExternalBackend() override;
    bool Distributed() const override;
    int Connect() override;
    int Put(const std::string &key, const std::string &value, uint32_t ttlMs) override;
    int Get(const std::string &key, std::string &value) override;
    int PrefixGet(const std::string &prefix, std::vector<std::pair<std::string, std::string>> &out) override;
    int Delete(const std::string &key) override;
    int Clear(const std::string &prefix) override;
    int Lock(const std::string &name) override;
    int TryLock(const std::string &name) override;
    int Unlock(const std::string &name) override;

private:
    smem_conf_store_backend_op_t ops_;
    std::string name_, prefix_;
    void *handle_ = nullptr;
};

// Registry of the user-supplied op table (smem_config_store_set_backend_op).
int SetExternalBackendOps(const smem_conf_store_backend_op_t *ops);
bool GetExternalBackendOps(smem_conf_store_backend_op_t &ops);

}  // namespace store
}  // namespace mf
