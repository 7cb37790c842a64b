// SMA: the caching allocator that serves PyTorch (through its pluggable-allocator hooks) from the
// symmetric heap.
//
//   malloc(size, stream): round the size (512 B steps below the small threshold, 2 MiB steps above), look
//     for a cached block of that stream that fits without wasting more than `max_split`, else carve from
//     the SplitMemoryHeap; when the heap is exhausted, wait for the device (hook), return every cached
//     block of every stream to the heap and try once more.
//   free(ptr, stream): the block goes to the cache of the stream it was allocated on. Work already queued
//     on that stream may still touch it, and a later malloc on the SAME stream is ordered behind that
//     work, so reuse needs no event. Blocks never move between streams without a device-wide wait.
//
// Because the policy depends only on the call sequence, ranks that allocate in lockstep get identical
// offsets inside their slices (a symmetric tensor needs no address exchange).
//
// Configuration (environment ZBAL_ALLOC_CONF, "key:value,key:value" as in PyTorch's allocator settings):
//   small_heap_threshold   bytes; requests below it grow from the low end (default 1 MiB)
//   max_split_size_mb      a cached block may serve a request only if it wastes less than this (default 20)
//   round_large_mb         rounding step of large requests (default 2)
//   garbage_collection_threshold   fraction of the heap in use+cached above which free() of a large block
//                          returns it to the heap at once instead of caching it (default 0 = off)
//
// Private pools (CUDA-graph capture): between begin_pool and end_pool, allocations of the capturing stream are
// tagged with the pool; a tagged block that is freed is parked in the pool and only that pool may reuse it,
// until release_pool returns the parked blocks to the heap. Neither empty_cache nor heap exhaustion touches a
// pool, because a graph replays with the addresses it captured.
//
// Parity of role: app/zbal/src/csrc/sma/zbal_sma_device.cpp, zbal_sma_config.h:20-102,
// app/zbal/src/include/zbal_mem_allocator.h of the reference.
#include <dlfcn.h>

#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <sstream>
#include <unordered_map>

#include "../include/zbal_mem_allocator.h"
#include "../util/mf_util.h"
#include "../hybm/mf_device.h"
#include "zbal_sma_heap.h"

namespace zbal {
namespace {

// Keys of ZBAL_ALLOC_CONF / ZBAL_NPU_ALLOC_CONF (the reference's set, app/zbal/src/csrc/sma/zbal_sma_config.h:20-102,
// app/zbal/doc/user_guide/env.md, plus round_large_mb):
//   max_split_size_mb            cached blocks above this size are only reused whole
//   garbage_collection_threshold fraction of the heap in use above which cached blocks are returned first
//   segment_size_mb              granule that large requests are rounded to (alias: round_large_mb), default 2
//   small_heap_threshold         requests below it come from the low end of the heap, default 1 MiB
//   small_heap_size              bytes of the low end that such requests may occupy, default 512000 KiB
//   use_sma_allocator            False: the pluggable entry points bypass the heap (plain device allocations)
//   use_vmm_for_static_memory    True: requests above max_split_size_mb (weights, KV cache: large and long-lived)
//                                get their own device allocation outside the heap and never fragment it
//   expandable_segments          True: a request that the heap cannot serve (after the caches were returned) asks the grow
//                                hook for another segment and is tried again; the heap then spans several address ranges
//   max_segments                 ranges the heap may grow to (the first one included), default 8
struct Config {
    uint64_t smallThreshold = 1ull << 20;
    uint64_t maxSplit = 20ull << 20;
    uint64_t roundLarge = 2ull << 20;
    uint64_t smallHeapSize = 524288000ull;
    double gcThreshold = 0.0;
    bool useSma = true;
    bool vmmForStatic = false;
    bool expandable = false;
    uint64_t maxSegments = 8;
};

// Asked for another segment when the heap is exhausted: returns 0 after it added one with zbal_sma_add_segment.
std::mutex g_hookMu;
zbal_sma_grow_hook_t g_growHook = nullptr;
void *g_growCtx = nullptr;

bool ParseBool(const std::string &v, bool &out)
{
    if (v == "True" || v == "true" || v == "1") out = true;
    else if (v == "False" || v == "false" || v == "0") out = false;
    else return false;
    return true;
}

Config ParseConf(uint64_t optThreshold)
{
    Config c;
    if (optThreshold) c.smallThreshold = optThreshold;
    const std::string s = mf::EnvStr("ZBAL_ALLOC_CONF", "ZBAL_NPU_ALLOC_CONF", "");
    for (const auto &kv : mf::Split(s, ',')) {
        const auto p = kv.find(':');
        if (p == std::string::npos) continue;
        const std::string k = kv.substr(0, p), v = kv.substr(p + 1);
        uint64_t u = 0;
        if (k == "small_heap_threshold" && mf::ParseU64(v, u) && u >= 4096) c.smallThreshold = u;
        else if (k == "max_split_size_mb" && mf::ParseU64(v, u) && u >= 1) c.maxSplit = u << 20;
        else if ((k == "round_large_mb" || k == "segment_size_mb") && mf::ParseU64(v, u) && u >= 1 && u <= 1024) c.roundLarge = u << 20;
        else if (k == "small_heap_size" && mf::ParseU64(v, u)) c.smallHeapSize = u;
        else if (k == "use_sma_allocator" && ParseBool(v, c.useSma)) {}
        else if (k == "use_vmm_for_static_memory" && ParseBool(v, c.vmmForStatic)) {}
        else if (k == "expandable_segments" && ParseBool(v, c.expandable)) {}
        else if (k == "max_segments" && mf::ParseU64(v, u) && u >= 1 && u <= 64) c.maxSegments = u;
        else if (k == "garbage_collection_threshold") c.gcThreshold = atof(v.c_str());
        else MF_WARN("ZBAL_ALLOC_CONF: ignoring '%s'", kv.c_str());
    }
    return c;
}

struct HistoryEntry {
    uint8_t kind;  // 0 malloc from heap, 1 malloc from cache, 2 free to cache, 3 free to heap, 4 empty_cache, 5 failed malloc
    uint64_t addr, size, requested, stream;
};

using PoolId = std::pair<uint64_t, uint64_t>;
const PoolId kNoPool{0, 0};

struct Pool {
    std::multimap<uint64_t, uint64_t> parked;  // size -> addr
    uint64_t parkedBytes = 0;
    bool routing = false;
    zbal_pool_filter_t filter = nullptr;
    void *ctx = nullptr;
};

struct LiveBlock {
    uint64_t size, stream;
    PoolId pool;
};

class Sma {
public:
    Sma(uint64_t base, uint64_t size, const Config &cfg, int device, bool simulated)
        : heap_(base, size, cfg.smallThreshold), cfg_(cfg), device_(device), simulated_(simulated)
    {
        // the small side may take at most half of a heap that is smaller than twice the configured size
        heap_.SetSmallLimit(std::min<uint64_t>(cfg.smallHeapSize, size / 2));
    }
    const Config &Conf() const { return cfg_; }
    bool Simulated() const { return simulated_; }

    uint64_t Round(uint64_t size) const
    {
        if (size == 0) size = 1;
        if (size < cfg_.smallThreshold) return mf::AlignUp(size, SplitMemoryHeap::kMinBlock);
        return mf::AlignUp(size, cfg_.roundLarge);
    }

    void *Malloc(uint64_t requested, uint64_t stream)
    {
        const uint64_t size = Round(requested);
        std::unique_lock<std::mutex> g(mu_);
        st_.mallocCalls++;
        const PoolId pool = RoutedPool(stream);
        if (pool != kNoPool) return PoolMalloc(pool, size, requested, stream);
        auto &cache = cache_[stream];
        auto it = cache.lower_bound(size);
        if (it != cache.end()) {
            // small classes are multiples of 512 B and must match exactly; a large cached block may serve a
            // request up to 25 % smaller, as long as the waste stays under max_split
            const uint64_t waste = it->first - size;
            const bool hit = size < cfg_.smallThreshold ? waste == 0 : (waste < cfg_.maxSplit && waste <= it->first / 4);
            if (hit) {
                const uint64_t addr = it->second, bsz = it->first;
                cache.erase(it);
                cached_ -= bsz;
                Hand(addr, bsz, stream, kNoPool);
                st_.cacheHits++;
                Note(1, addr, bsz, requested, stream);
                return reinterpret_cast<void *>(addr);
            }
        }
        uint64_t addr = heap_.AlignedAllocate(size, size < cfg_.smallThreshold ? 512 : 4096);
        if (addr == 0 && cached_ > 0) {
            DeviceWait();
            FlushLocked();
            addr = heap_.AlignedAllocate(size, size < cfg_.smallThreshold ? 512 : 4096);
        }
        if (addr == 0 && cfg_.expandable && heap_.Regions() < cfg_.maxSegments) {
            // another segment: the hook runs without the allocator's lock (it calls back into AddSegment, and with a
            // symmetric heap it is a collective step that may take a while)
            zbal_sma_grow_hook_t hook;
            void *ctx;
            {
                std::lock_guard<std::mutex> h(g_hookMu);
                hook = g_growHook;
                ctx = g_growCtx;
            }
            if (hook != nullptr) {
                g.unlock();
                const int rc = hook(size, ctx);
                g.lock();
                if (rc == 0) {
                    st_.segmentsAdded++;
                    addr = heap_.AlignedAllocate(size, size < cfg_.smallThreshold ? 512 : 4096);
                }
            }
        }
        if (addr == 0) {
            st_.failedMallocs++;
            Note(5, 0, size, requested, stream);
            mf::LastError::Set(Z_NO_MEMORY, "symmetric heap exhausted: %lu bytes requested, %lu in use of %lu, largest free block %lu",
                               (unsigned long)size, (unsigned long)inUse_, (unsigned long)heap_.TotalSize(),
                               (unsigned long)heap_.LargestFree());
            return nullptr;
        }
        st_.heapCarves++;
        Hand(addr, size, stream, kNoPool);
        Note(0, addr, size, requested, stream);
        return reinterpret_cast<void *>(addr);
    }

    int BeginPool(PoolId id, zbal_pool_filter_t filter, void *ctx)
    {
        if (id == kNoPool) return Z_INVALID_PARAM;
        std::lock_guard<std::mutex> g(mu_);
        Pool &p = pools_[id];
        p.routing = true;
        p.filter = filter;
        p.ctx = ctx;
        return Z_OK;
    }
    int EndPool(PoolId id)
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = pools_.find(id);
        if (it == pools_.end()) return Z_INVALID_PARAM;
        it->second.routing = false;
        it->second.filter = nullptr;
        it->second.ctx = nullptr;
        return Z_OK;
    }
    int ReleasePool(PoolId id)
    {
        std::lock_guard<std::mutex> g(mu_);
        auto it = pools_.find(id);
        if (it == pools_.end()) return Z_INVALID_PARAM;
        if (!it->second.parked.empty()) DeviceWait();  // a replay in flight may still touch the parked blocks
        for (auto &kv : it->second.parked) {
            heap_.Release(kv.second);
            Note(3, kv.second, kv.first, 0, 0);
        }
        pools_.erase(it);
        for (auto &kv : live_)
            if (kv.second.pool == id) kv.second.pool = kNoPool;
        return Z_OK;
    }

    bool Free(void *ptr)
    {
        const uint64_t addr = reinterpret_cast<uint64_t>(ptr);
        std::lock_guard<std::mutex> g(mu_);
        auto it = live_.find(addr);
        if (it == live_.end()) return false;
        const uint64_t size = it->second.size, stream = it->second.stream;
        const PoolId pool = it->second.pool;
        live_.erase(it);
        inUse_ -= size;
        st_.freeCalls++;
        if (pool != kNoPool) {
            auto pit = pools_.find(pool);
            if (pit != pools_.end()) {
                pit->second.parked.emplace(size, addr);
                pit->second.parkedBytes += size;
                Note(2, addr, size, 0, stream);
                return true;
            }
        }
        const bool gc = cfg_.gcThreshold > 0.0 && size >= cfg_.smallThreshold &&
                        (double)(inUse_ + cached_ + size) > cfg_.gcThreshold * (double)heap_.TotalSize();
        if (gc) {
            // the block may still be in use by queued work: wait before it can be carved for another stream
            DeviceWait();
            heap_.Release(addr);
            Note(3, addr, size, 0, stream);
        } else {
            cache_[stream].emplace(size, addr);
            cached_ += size;
            Note(2, addr, size, 0, stream);
        }
        return true;
    }

    void EmptyCache(bool checkError)
    {
        std::lock_guard<std::mutex> g(mu_);
        DeviceWait();
        FlushLocked();
        Note(4, 0, 0, 0, 0);
        if (checkError && !live_.empty())
            mf::LastError::Set(Z_ERROR, "empty_cache: %zu blocks (%lu bytes) are still in use", live_.size(), (unsigned long)inUse_);
    }

    bool AddSegment(uint64_t base, uint64_t size) { return heap_.AddRegion(base, size); }

    void Stats(zbal_sma_stats_t &o)
    {
        std::lock_guard<std::mutex> g(mu_);
        o = st_;
        o.segments = heap_.Regions();
        o.heapSize = heap_.TotalSize();
        o.inUseBytes = inUse_;
        o.cachedBytes = cached_;
        o.peakInUseBytes = peak_;
        o.largestFreeBlock = heap_.LargestFree();
        o.poolCount = pools_.size();
        o.poolCachedBytes = 0;
        for (const auto &kv : pools_) o.poolCachedBytes += kv.second.parkedBytes;
    }
    void ResetPeak()
    {
        std::lock_guard<std::mutex> g(mu_);
        peak_ = inUse_;
    }
    void Record(bool on, uint32_t maxEntries)
    {
        std::lock_guard<std::mutex> g(mu_);
        record_ = on;
        maxHistory_ = maxEntries ? maxEntries : 65536;
        if (!on) history_.clear();
    }

    std::string Snapshot()
    {
        std::lock_guard<std::mutex> g(mu_);
        std::ostringstream o;
        o << "{\"heap\":{\"base\":" << heap_.Base() << ",\"size\":" << heap_.TotalSize() << ",\"threshold\":" << heap_.Threshold()
          << ",\"round_large\":" << cfg_.roundLarge << ",\"max_split\":" << cfg_.maxSplit << ",\"device\":" << device_
          << ",\"simulated\":" << (simulated_ ? "true" : "false") << ",\"in_use\":" << inUse_ << ",\"cached\":" << cached_
          << ",\"peak\":" << peak_ << "},\"segments\":[";
        bool first = true;
        for (const auto &r : heap_.RegionList()) {
            o << (first ? "" : ",") << "{\"base\":" << r.first << ",\"size\":" << r.second << "}";
            first = false;
        }
        o << "],\"blocks\":[";
        first = true;
        for (const auto &b : heap_.Blocks()) {
            const char *state = "free";
            uint64_t stream = 0;
            if (b.used) {
                auto it = live_.find(b.addr);
                state = it != live_.end() ? "active" : "cached";
                if (it != live_.end()) stream = it->second.stream;
            }
            o << (first ? "" : ",") << "{\"addr\":" << b.addr << ",\"size\":" << b.size << ",\"state\":\"" << state << "\",\"stream\":" << stream
              << "}";
            first = false;
        }
        o << "],\"history\":[";
        first = true;
        static const char *kinds[] = {"malloc_heap", "malloc_cache", "free_cache", "free_heap", "empty_cache", "malloc_failed"};
        for (const auto &h : history_) {
            o << (first ? "" : ",") << "{\"op\":\"" << kinds[h.kind] << "\",\"addr\":" << h.addr << ",\"size\":" << h.size
              << ",\"requested\":" << h.requested << ",\"stream\":" << h.stream << "}";
            first = false;
        }
        o << "]}";
        return o.str();
    }

    bool Owns(uint64_t addr) const { return addr >= heap_.Base() && addr < heap_.Base() + heap_.TotalSize(); }

private:
    PoolId RoutedPool(uint64_t stream) const
    {
        for (const auto &kv : pools_)
            if (kv.second.routing && (kv.second.filter == nullptr || kv.second.filter(kv.second.ctx, reinterpret_cast<zbal_stream_t>(stream))))
                return kv.first;
        return kNoPool;
    }
    // Exact size classes inside a pool: a capture repeats the same shapes, and a replay must never see a block split.
    void *PoolMalloc(const PoolId &id, uint64_t size, uint64_t requested, uint64_t stream)
    {
        Pool &p = pools_[id];
        auto it = p.parked.find(size);
        uint64_t addr = 0;
        if (it != p.parked.end()) {
            addr = it->second;
            p.parked.erase(it);
            p.parkedBytes -= size;
            st_.cacheHits++;
            Note(1, addr, size, requested, stream);
        } else {
            addr = heap_.AlignedAllocate(size, size < cfg_.smallThreshold ? 512 : 4096);
            if (addr == 0 && cached_ > 0) {
                // no device-wide wait here: it is illegal while a stream is capturing. The stream caches are
                // flushed only if nothing is capturing work that could still touch them, which the caller
                // guarantees by emptying the cache before the capture (torch.cuda.graph does).
                st_.failedMallocs++;
                Note(5, 0, size, requested, stream);
                mf::LastError::Set(Z_NO_MEMORY, "symmetric heap exhausted inside a private pool: %lu bytes requested, %lu cached outside "
                                   "the pool (empty the cache before capturing)", (unsigned long)size, (unsigned long)cached_);
                return nullptr;
            }
            if (addr == 0) {
                st_.failedMallocs++;
                Note(5, 0, size, requested, stream);
                mf::LastError::Set(Z_NO_MEMORY, "symmetric heap exhausted: %lu bytes requested, %lu in use of %lu", (unsigned long)size,
                                   (unsigned long)inUse_, (unsigned long)heap_.TotalSize());
                return nullptr;
            }
            st_.heapCarves++;
            Note(0, addr, size, requested, stream);
        }
        Hand(addr, size, stream, id);
        return reinterpret_cast<void *>(addr);
    }
    void Hand(uint64_t addr, uint64_t size, uint64_t stream, const PoolId &pool)
    {
        live_[addr] = {size, stream, pool};
        inUse_ += size;
        if (inUse_ > peak_) peak_ = inUse_;
    }
    void FlushLocked()
    {
        for (auto &s : cache_)
            for (auto &kv : s.second) heap_.Release(kv.second);
        cache_.clear();
        cached_ = 0;
    }
    void Note(uint8_t kind, uint64_t addr, uint64_t size, uint64_t requested, uint64_t stream)
    {
        if (!record_) return;
        if (history_.size() >= maxHistory_) history_.pop_front();
        history_.push_back({kind, addr, size, requested, stream});
    }
    void DeviceWait()
    {
        if (simulated_) return;
        // exported by the CUDA library once it is loaded; without it there is no device work to wait for
        using Fn = int (*)(int);
        static Fn fn = reinterpret_cast<Fn>(mf::hybm::CudaSymbol("mf_cuda_device_sync"));
        if (fn != nullptr) fn(device_);
    }

    SplitMemoryHeap heap_;
    const Config cfg_;
    const int device_;
    const bool simulated_;
    std::mutex mu_;
    std::unordered_map<uint64_t, std::multimap<uint64_t, uint64_t>> cache_;  // stream -> size -> addr
    std::unordered_map<uint64_t, LiveBlock> live_;                           // addr -> (size, stream, pool)
    std::map<PoolId, Pool> pools_;
    uint64_t inUse_ = 0, cached_ = 0, peak_ = 0;
    zbal_sma_stats_t st_{};
    bool record_ = false;
    size_t maxHistory_ = 65536;
    std::deque<HistoryEntry> history_;
};

std::mutex g_mu;
std::shared_ptr<Sma> g_sma;

std::shared_ptr<Sma> Get()
{
    std::lock_guard<std::mutex> g(g_mu);
    return g_sma;
}

}  // namespace
}  // namespace zbal

using namespace zbal;

extern "C" {

namespace {
std::mutex g_outside_mu;
std::map<uint64_t, uint64_t> g_outside;  // device allocations handed out by the pluggable entry points outside the heap
}  // namespace

int32_t zbal_sma_init(zbal_allocator_options_t *options, int32_t flags)
{
    (void)flags;
    if (options == nullptr || options->size < (1ull << 20) || options->baseAddress == 0)
        return MF_FAIL(Z_INVALID_PARAM, "zbal_sma_init: need a base address and at least 1 MiB");
    std::lock_guard<std::mutex> g(g_mu);
    if (g_sma) return MF_FAIL(Z_ALREADY_INITIALIZED, "zbal_sma_init: allocator already initialised");
    g_sma = std::make_shared<Sma>(options->baseAddress, options->size, ParseConf(options->smallThreshold), options->deviceId, false);
    return Z_OK;
}

void zbal_sma_uninit(int32_t flags)
{
    (void)flags;
    std::lock_guard<std::mutex> g(g_mu);
    g_sma.reset();
}

int32_t zbal_sma_add_segment(uint64_t base, uint64_t size)
{
    auto s = Get();
    if (!s) return MF_FAIL(Z_NOT_INITIALIZED, "zbal_sma_add_segment before zbal_sma_init");
    if (base == 0 || size < (1ull << 20)) return MF_FAIL(Z_INVALID_PARAM, "a segment needs a base address and at least 1 MiB");
    if (!s->AddSegment(base, size)) return MF_FAIL(Z_INVALID_PARAM, "segment [%lx, +%lu) overlaps the heap or is misaligned", (unsigned long)base, (unsigned long)size);
    return Z_OK;
}

void zbal_sma_set_grow_hook(zbal_sma_grow_hook_t hook, void *ctx)
{
    std::lock_guard<std::mutex> h(g_hookMu);
    g_growHook = hook;
    g_growCtx = ctx;
}

void zbal_simulate_init(int64_t addr, int64_t size)
{
    std::lock_guard<std::mutex> g(g_mu);
    g_sma = std::make_shared<Sma>((uint64_t)addr, (uint64_t)size, ParseConf(0), 0, true);
}

void zbal_pluggable_init(int32_t device_count)
{
    (void)device_count;  // one device per process: nothing to size
}

void *zbal_pluggable_malloc(size_t size, int32_t device, zbal_stream_t stream)
{
    (void)device;
    auto s = Get();
    if (!s) {
        mf::LastError::Set(Z_NOT_INITIALIZED, "zbal_pluggable_malloc before zbal_sma_init");
        return nullptr;
    }
    // outside the heap: the whole allocator switched off, or "static" (large, long-lived) memory kept out of it
    const Config &c = s->Conf();
    if (!s->Simulated() && (!c.useSma || (c.vmmForStatic && size > c.maxSplit))) {
        mf::hybm::DeviceBackend *dev = mf::hybm::CurrentBackend();
        uint64_t p = 0;
        if (dev == nullptr || dev->Malloc(size, &p) != 0 || p == 0) {
            MF_FAIL(Z_NO_MEMORY, "device allocation of %zu bytes outside the heap failed", size);
            return nullptr;
        }
        std::lock_guard<std::mutex> g(g_outside_mu);
        g_outside[p] = size;
        return reinterpret_cast<void *>(p);
    }
    return s->Malloc(size, reinterpret_cast<uint64_t>(stream));
}

void zbal_pluggable_free(void *ptr, size_t size, int32_t device, zbal_stream_t stream)
{
    (void)size;
    (void)device;
    (void)stream;
    auto s = Get();
    if (ptr == nullptr) return;
    {
        std::unique_lock<std::mutex> g(g_outside_mu);
        auto it = g_outside.find(reinterpret_cast<uint64_t>(ptr));
        if (it != g_outside.end()) {
            g_outside.erase(it);
            g.unlock();
            if (mf::hybm::DeviceBackend *dev = mf::hybm::CurrentBackend()) dev->Free(reinterpret_cast<uint64_t>(ptr));
            return;
        }
    }
    if (!s) return;
    if (!s->Free(ptr)) MF_WARN("zbal_pluggable_free: %p was not allocated by this allocator", ptr);
}

void zbal_pluggable_empty_cache(bool check_error)
{
    auto s = Get();
    if (s) s->EmptyCache(check_error);
}

int32_t zbal_sma_begin_pool(uint64_t pool_hi, uint64_t pool_lo, zbal_pool_filter_t filter, void *ctx)
{
    auto s = Get();
    return s ? s->BeginPool({pool_hi, pool_lo}, filter, ctx) : (int32_t)Z_NOT_INITIALIZED;
}

int32_t zbal_sma_end_pool(uint64_t pool_hi, uint64_t pool_lo)
{
    auto s = Get();
    return s ? s->EndPool({pool_hi, pool_lo}) : (int32_t)Z_NOT_INITIALIZED;
}

int32_t zbal_sma_release_pool(uint64_t pool_hi, uint64_t pool_lo)
{
    auto s = Get();
    return s ? s->ReleasePool({pool_hi, pool_lo}) : (int32_t)Z_NOT_INITIALIZED;
}

int32_t zbal_sma_get_stats(zbal_sma_stats_t *stats)
{
    auto s = Get();
    if (!s || stats == nullptr) return Z_NOT_INITIALIZED;
    s->Stats(*stats);
    return Z_OK;
}

void zbal_sma_reset_peak(void)
{
    auto s = Get();
    if (s) s->ResetPeak();
}

void zbal_sma_record_history(bool enable, uint32_t max_entries)
{
    auto s = Get();
    if (s) s->Record(enable, max_entries);
}

int64_t zbal_sma_snapshot(char *buf, int64_t cap)
{
    auto s = Get();
    if (!s) return Z_NOT_INITIALIZED;
    const std::string j = s->Snapshot();
    if (buf != nullptr && cap > 0) {
        const size_t n = std::min<size_t>(j.size(), (size_t)cap - 1);
        memcpy(buf, j.data(), n);
        buf[n] = 0;
    }
    return (int64_t)j.size() + 1;
}

}  // extern "C"
