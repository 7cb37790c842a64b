#include "zbal_sma_heap.h"

#include <algorithm>

namespace zbal {

SplitMemoryHeap::SplitMemoryHeap(uint64_t base, uint64_t size, uint64_t threshold)
    : base_(base), size_(size / kMinBlock * kMinBlock), threshold_(threshold == 0 ? (1ull << 20) : threshold)
{
    if (size_ > 0) InsertFree(base_, size_);
    regions_.emplace_back(base_, size_);
}

void SplitMemoryHeap::InsertFreeMerged(uint64_t addr, uint64_t size)
{
    auto next = free_.lower_bound(addr);
    if (next != free_.begin()) {
        auto prev = std::prev(next);
        if (prev->first + prev->second == addr) {
            const uint64_t pa = prev->first, ps = prev->second;
            EraseFree(pa, ps);
            addr = pa;
            size += ps;
        }
    }
    next = free_.find(addr + size);
    if (next != free_.end()) {
        const uint64_t na = next->first, ns = next->second;
        EraseFree(na, ns);
        size += ns;
    }
    InsertFree(addr, size);
}

bool SplitMemoryHeap::AddRegion(uint64_t base, uint64_t size)
{
    size = size / kMinBlock * kMinBlock;
    if (size == 0 || (base % kMinBlock) != 0) return false;
    std::lock_guard<std::mutex> g(mu_);
    for (const auto &r : regions_)
        if (base < r.first + r.second && r.first < base + size) return false;
    regions_.emplace_back(base, size);
    size_ += size;
    InsertFreeMerged(base, size);
    return true;
}

size_t SplitMemoryHeap::Regions() const
{
    std::lock_guard<std::mutex> g(mu_);
    return regions_.size();
}

std::vector<std::pair<uint64_t, uint64_t>> SplitMemoryHeap::RegionList() const
{
    std::lock_guard<std::mutex> g(mu_);
    return regions_;
}

int SplitMemoryHeap::BucketOf(uint64_t size)
{
    return size == 0 ? 0 : 63 - __builtin_clzll(size);
}

void SplitMemoryHeap::InsertFree(uint64_t addr, uint64_t size)
{
    free_[addr] = size;
    buckets_[BucketOf(size)].insert(addr);
}

void SplitMemoryHeap::EraseFree(uint64_t addr, uint64_t size)
{
    free_.erase(addr);
    buckets_[BucketOf(size)].erase(addr);
}

bool SplitMemoryHeap::Pick(uint64_t size, uint64_t align, bool low, uint64_t &blockAddr, uint64_t &blockSize, uint64_t &at) const
{
    bool found = false;
    auto consider = [&](uint64_t addr) {
        const uint64_t bsz = free_.find(addr)->second;
        uint64_t pos;
        if (low) {
            pos = (addr + align - 1) & ~(align - 1);
            if (pos + size > addr + bsz) return false;
            if (smallLimit_ != 0 && pos + size > base_ + smallLimit_) return false;   // the small side is full
        } else {
            if (bsz < size) return false;
            pos = (addr + bsz - size) & ~(align - 1);
            if (pos < addr) return false;
        }
        if (!found || (low ? pos < at : pos > at)) {
            found = true;
            blockAddr = addr;
            blockSize = bsz;
            at = pos;
        }
        return true;
    };
    const int first = BucketOf(size);
    for (int b = first; b < kBuckets; b++) {
        const auto &s = buckets_[b];
        if (s.empty()) continue;
        // walk from the preferred end until one block of this class fits; blocks of a higher class fit
        // unless alignment eats the slack, so the walk is short
        if (low) {
            for (auto it = s.begin(); it != s.end(); ++it)
                if (consider(*it)) break;
        } else {
            for (auto it = s.rbegin(); it != s.rend(); ++it)
                if (consider(*it)) break;
        }
    }
    return found;
}

uint64_t SplitMemoryHeap::AlignedAllocate(uint64_t size, uint64_t align)
{
    if (size == 0) size = kMinBlock;
    size = (size + kMinBlock - 1) / kMinBlock * kMinBlock;
    if (align < kMinBlock) align = kMinBlock;
    if ((align & (align - 1)) != 0) return 0;
    std::lock_guard<std::mutex> g(mu_);
    const bool low = size < threshold_;
    uint64_t baddr = 0, bsize = 0, at = 0;
    if (!Pick(size, align, low, baddr, bsize, at)) {
        if (!(low && smallLimit_ != 0 && Pick(size, align, false, baddr, bsize, at))) return 0;
    }
    EraseFree(baddr, bsize);
    if (at > baddr) InsertFree(baddr, at - baddr);
    const uint64_t end = at + size, bend = baddr + bsize;
    if (bend > end) InsertFree(end, bend - end);
    used_[at] = size;
    inUse_ += size;
    return at;
}

uint64_t SplitMemoryHeap::Release(uint64_t addr)
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = used_.find(addr);
    if (it == used_.end()) return 0;
    uint64_t size = it->second;
    const uint64_t released = size;
    used_.erase(it);
    inUse_ -= size;
    InsertFreeMerged(addr, size);  // with the free block that ends at addr and the one that starts at addr + size
    return released;
}

uint64_t SplitMemoryHeap::AllocatedSize(uint64_t addr) const
{
    std::lock_guard<std::mutex> g(mu_);
    auto it = used_.find(addr);
    return it == used_.end() ? 0 : it->second;
}

uint64_t SplitMemoryHeap::InUseSize() const
{
    std::lock_guard<std::mutex> g(mu_);
    return inUse_;
}

uint64_t SplitMemoryHeap::LargestFree() const
{
    std::lock_guard<std::mutex> g(mu_);
    for (int b = kBuckets - 1; b >= 0; b--) {
        uint64_t best = 0;
        for (uint64_t a : buckets_[b]) best = std::max(best, free_.find(a)->second);
        if (best) return best;
    }
    return 0;
}

size_t SplitMemoryHeap::FreeBlocks() const
{
    std::lock_guard<std::mutex> g(mu_);
    return free_.size();
}

std::vector<SplitMemoryHeap::BlockInfo> SplitMemoryHeap::Blocks() const
{
    std::lock_guard<std::mutex> g(mu_);
    std::vector<BlockInfo> out;
    out.reserve(free_.size() + used_.size());
    for (auto &kv : free_) out.push_back({kv.first, kv.second, false});
    for (auto &kv : used_) out.push_back({kv.first, kv.second, true});
    std::sort(out.begin(), out.end(), [](const BlockInfo &a, const BlockInfo &b) { return a.addr < b.addr; });
    return out;
}

}  // namespace zbal
