// SplitMemoryHeap: the address-space manager under the symmetric allocator.
//
// One contiguous range [base, base + size). Free blocks are kept twice: in an address-ordered map (so a
// released block finds both neighbours in O(log n) and coalesces) and in power-of-two size buckets
// (bucket = floor(log2(size)), each ordered by address). Requests below `threshold` are carved from the
// LOW end of the lowest fitting block, all others from the HIGH end of the highest fitting block, so the
// many small, short-lived blocks never fragment the region the large activations and KV blocks live in.
// The choice depends only on the sequence of calls, never on timing: ranks that run the same sequence get
// the same offsets, which is what lets kernels reach a peer's copy of a tensor with one stride.
//
// Parity of role: app/zbal/src/csrc/sma/zbal_sma_mm_heap.h:71-146 of the reference.
#pragma once
#include <cstdint>
#include <map>
#include <mutex>
#include <set>
#include <vector>

namespace zbal {

class SplitMemoryHeap {
public:
    static constexpr uint64_t kMinBlock = 512;
    static constexpr int kBuckets = 64;

    SplitMemoryHeap(uint64_t base, uint64_t size, uint64_t threshold);

    // Returns 0 when no block fits. `align` must be a power of two >= kMinBlock (smaller values are raised).
    uint64_t AlignedAllocate(uint64_t size, uint64_t align = kMinBlock);
    // Returns the size of the released block, 0 if addr was not handed out by this heap.
    uint64_t Release(uint64_t addr);
    uint64_t AllocatedSize(uint64_t addr) const;
    // Adds another range [base, base + size) of usable addresses (an expansion segment). It may or may not touch a
    // range the heap already has; free space that touches is merged. False when it overlaps what the heap manages.
    bool AddRegion(uint64_t base, uint64_t size);
    size_t Regions() const;
    std::vector<std::pair<uint64_t, uint64_t>> RegionList() const;  // (base, size) in the order they were added

    uint64_t Base() const { return base_; }
    uint64_t TotalSize() const { return size_; }
    uint64_t InUseSize() const;
    uint64_t LargestFree() const;
    size_t FreeBlocks() const;
    uint64_t Threshold() const { return threshold_; }
    // Bytes from the low end that blocks below the threshold may occupy (0: no limit). A small request that no longer
    // fits below the limit is carved from the high end like a large one.
    void SetSmallLimit(uint64_t bytes) { smallLimit_ = bytes; }
    uint64_t SmallLimit() const { return smallLimit_; }
    // (addr, size, used) of every block in address order
    struct BlockInfo {
        uint64_t addr, size;
        bool used;
    };
    std::vector<BlockInfo> Blocks() const;

private:
    static int BucketOf(uint64_t size);
    void InsertFree(uint64_t addr, uint64_t size);
    void EraseFree(uint64_t addr, uint64_t size);
    void InsertFreeMerged(uint64_t addr, uint64_t size);  // joins the free neighbours that touch [addr, addr + size)
    // picks a free block for (size, align); low=true prefers the lowest address, else the highest
    bool Pick(uint64_t size, uint64_t align, bool low, uint64_t &blockAddr, uint64_t &blockSize, uint64_t &at) const;

    const uint64_t base_;
    uint64_t size_;
    const uint64_t threshold_;
    std::vector<std::pair<uint64_t, uint64_t>> regions_;  // (base, size) in the order they were added
    mutable std::mutex mu_;
    std::map<uint64_t, uint64_t> free_;        // addr -> size
    std::set<uint64_t> buckets_[kBuckets];     // addresses of the free blocks of each size class
    std::map<uint64_t, uint64_t> used_;        // addr -> size
    uint64_t inUse_ = 0;
    uint64_t smallLimit_ = 0;
};

}  // namespace zbal
