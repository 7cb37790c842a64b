// etcd v3 as the distributed backend of the highly available config store, spoken natively: the JSON gateway that every
// etcd member serves beside gRPC (POST /v3/kv/put, /v3/kv/range, /v3/kv/deleterange, /v3/kv/txn, /v3/lease/grant,
// /v3/lease/keepalive, /v3/lease/revoke, /v3/auth/authenticate) over plain HTTP/1.1, one short connection per call. No
// client library is linked or opened.
// Counterpart of the reference's etcd backend (src/smem/csrc/config_store/backend/smem_etcd_store_backend.cpp) and of
// the cgo client it opens at run time (src/util/etcd_client/etcd_store_backend/etcd_client_v3.go: put with a lease,
// get, prefix get, remove, named locks on sessions with a 10 s TTL).
#pragma once
#include <atomic>
#include <condition_variable>
#include <map>
#include <thread>

#include "mf_store_backend.h"

namespace mf {
namespace store {

class EtcdBackend : public StoreBackend {
public:
    // instance: keys are stored below /memfabric_hybrid/config_store/clusters/<instance>/ when it is not empty, so that
    // several pools share one etcd. user / password: etcd authentication (empty: none).
    EtcdBackend(std::string ip, uint16_t port, std::string instance, std::string user = "", std::string password = "");
    ~EtcdBackend() override;
    bool Distributed() const override { return true; }
    int Connect() override;
    // ttlMs > 0: the key is bound to a fresh lease of ceil(ttlMs / 1000) seconds and disappears when it runs out; writing
    // the key again renews it (the lease of the earlier write is revoked).
    int Put(const std::string &key, const std::string &value, uint32_t ttlMs) override;
    int Get(const std::string &key, std::string &value) override;
    int PrefixGet(const std::string &prefix, std::vector<std::pair<std::string, std::string>> &out) override;
    int Delete(const std::string &key) override;
    int Clear(const std::string &prefix) override;
    // A named lock is a key created in a transaction that succeeds only while the key does not exist, bound to a 10 s
    // lease that a thread of this object keeps alive: a holder that dies frees the lock when the lease runs out.
    // Lock waits up to 30 s.
    int Lock(const std::string &name) override;
    int TryLock(const std::string &name) override;
    int Unlock(const std::string &name) override;

    void SetTimeoutMs(uint32_t ms) { timeoutMs_ = ms; }
    std::string LastError();

private:
    struct Reply;
    int Call(const std::string &path, const std::string &body, Reply &reply);
    int CallOnce(const std::string &path, const std::string &body, Reply &reply, bool withToken);
    int Authenticate();
    int GrantLease(int64_t ttlSec, int64_t &id);
    void RevokeLease(int64_t id);
    int Acquire(const std::string &name, bool wait);
    std::string Qualify(const std::string &key) const;
    void KeepAliveLoop();
    void SetError(const std::string &e);

    std::string ip_;
    uint16_t port_;
    std::string root_;   // "" or /memfabric_hybrid/config_store/clusters/<instance>
    std::string user_, password_, api_;
    std::atomic<uint32_t> timeoutMs_{3000};
    std::mutex mu_;                              // token_, lastError_, putLeases_, locks_
    std::string token_, lastError_;
    std::map<std::string, int64_t> putLeases_;   // qualified key -> lease of our last write with a TTL
    std::map<std::string, int64_t> locks_;       // lock name -> lease that holds it
    std::string owner_;                          // value written into lock keys: host:pid:object
    std::thread keepAlive_;
    std::mutex kaMu_;
    std::condition_variable kaCv_;
    bool stop_ = false;
};

}  // namespace store
}  // namespace mf
