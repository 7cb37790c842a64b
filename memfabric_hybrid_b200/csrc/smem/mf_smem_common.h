// Shared pieces of the smem C API layer: limits, handle registry, blob packing of exchange infos.
// Parity: src/smem/csrc/common/smem_types.h:55-64 (limits), smem_bm_entry.cpp:178-197 (exchange blobs).
#pragma once
#include <set>

#include "../group/mf_group.h"
#include "../hybm/mf_entity.h"
#include "../include/smem.h"
#include "../store/mf_store.h"

namespace mf {
namespace smem {

constexpr uint32_t kIdMax = 63;
constexpr uint64_t kHbmMax = 256ULL << 30;   // per rank (a B200 has 180 GB)
constexpr uint64_t kDramMax = 2ULL << 40;    // per rank
constexpr uint32_t kDefaultTimeoutSec = 120;

// Translates internal result codes to the public SMEM_* range (they share values by construction).
inline int32_t Pub(int rc)
{
    switch (rc) {
        case ERR_BUSY: return SMEM_TIMEOUT;
        case ERR_RECONNECT: return SMEM_NOT_CONNECTED;
        default: return rc;
    }
}

// [u32 count]{[u32 len][bytes]}*
inline std::string PackInfos(const std::vector<hybm_exchange_info> &v)
{
    std::string s;
    uint32_t n = (uint32_t)v.size();
    s.append(reinterpret_cast<const char *>(&n), sizeof(n));
    for (auto &e : v) {
        s.append(reinterpret_cast<const char *>(&e.descLen), sizeof(e.descLen));
        s.append(reinterpret_cast<const char *>(e.desc), e.descLen);
    }
    return s;
}

inline bool UnpackInfos(const std::string &s, std::vector<hybm_exchange_info> &v)
{
    size_t off = 0;
    uint32_t n = 0;
    if (s.size() < sizeof(n)) return false;
    memcpy(&n, s.data(), sizeof(n));
    off += sizeof(n);
    if (n > 4096) return false;
    for (uint32_t i = 0; i < n; i++) {
        hybm_exchange_info e;
        if (off + sizeof(e.descLen) > s.size()) return false;
        memcpy(&e.descLen, s.data() + off, sizeof(e.descLen));
        off += sizeof(e.descLen);
        if (e.descLen > sizeof(e.desc) || off + e.descLen > s.size()) return false;
        memcpy(e.desc, s.data() + off, e.descLen);
        off += e.descLen;
        v.push_back(e);
    }
    return true;
}

// Registry of live handles of one API so that a stale or foreign pointer is refused, not followed.
template <typename T> class HandleTable {
public:
    void *Add(const std::shared_ptr<T> &p)
    {
        std::lock_guard<std::mutex> g(mu_);
        map_[p.get()] = p;
        return p.get();
    }
    std::shared_ptr<T> Find(void *h)
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = map_.find(h);
        return it == map_.end() ? nullptr : it->second;
    }
    std::shared_ptr<T> Take(void *h)
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = map_.find(h);
        if (it == map_.end()) return nullptr;
        auto p = it->second;
        map_.erase(it);
        return p;
    }
    std::vector<std::shared_ptr<T>> TakeAll()
    {
        std::lock_guard<std::mutex> g(mu_);
        std::vector<std::shared_ptr<T>> v;
        for (auto &kv : map_) v.push_back(kv.second);
        map_.clear();
        return v;
    }

private:
    std::mutex mu_;
    std::map<void *, std::shared_ptr<T>> map_;
};

// smem_init bookkeeping shared by bm/shm/trans.
bool SmemInited();

}  // namespace smem
}  // namespace mf
