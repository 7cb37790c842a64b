// Memory segments: one per (entity, memory type). A segment reserves the GVA window
// [base, base + slot * ranks), places this rank's slices in its own slot, exports them as blobs and
// maps peers' slices at their slots.
//   HostShmSegment — pooled DRAM: POSIX shared-memory files mapped with MAP_FIXED; when a GPU is
//                    attached every mapped range is also registered (pinned + device-mapped) so that
//                    copy engines and kernels reach it at PCIe speed.
//   VmmSegment     — pooled HBM: physical allocations from the device backend's VMM interface,
//                    exported as POSIX file descriptors that travel over a Unix-domain socket
//                    (SCM_RIGHTS) because the store blobs can carry no descriptors.
// Parity: src/hybm/csrc/mm/hybm_mem_segment.h, hybm_host_shm_segment.cpp:35-143,390-540,
// hybm_vmm_based_segment.cpp:71-101,252-336,395-445,470-631,650-687.
#pragma once
#include <functional>
#include <memory>
#include <thread>

#include "mf_device.h"
#include "mf_hybm_types.h"

namespace mf {
namespace hybm {

// Passes file descriptors between processes of one host. Each process serves its published
// descriptors on an abstract Unix socket; importers connect, send a token and get the descriptor.
class FdChannel {
public:
    static FdChannel &Get();
    const std::string &Name();                 // starts the server thread on first use
    uint64_t Publish(int fd);                  // keeps a dup until Withdraw
    void Withdraw(uint64_t token);
    static int Fetch(const std::string &name, uint64_t token, int *fd);
    void Stop();

private:
    void Serve();
    std::mutex mu_;
    std::string name_;
    int listenFd_ = -1;
    std::thread th_;
    std::atomic<bool> run_{false};
    std::map<uint64_t, int> fds_;
    uint64_t next_ = 1;
};

struct SegmentOptions {
    uint32_t entityId = 0;
    uint32_t rank = 0;
    uint32_t rankCount = 0;
    uint64_t slot = 0;  // per-rank bytes in the window
    uint64_t publicSlot = 0;  // != 0: compact mode (56-bit addresses): callers see slots of this size, `slot` is what each rank gets in this process
    hybm_mem_type type = HYBM_MEM_TYPE_DEVICE;
    uint32_t flags = 0;
    int shmFd = -1;
    DeviceBackend *dev = nullptr;
};

struct PeerSlice {
    uint32_t rank = 0;
    uint32_t index = 0;
    uint64_t offset = 0;
    uint64_t size = 0;
    std::string source;  // shm file name, or fd-channel name
    uint64_t token = 0;  // fd-channel token
    int32_t pid = 0;
    bool mapped = false;
    PhysHandle phys = 0;
};

class Segment {
public:
    explicit Segment(const SegmentOptions &o) : opt_(o), mappedBytes_(o.rankCount) {}
    virtual ~Segment() = default;
    static std::shared_ptr<Segment> Create(const SegmentOptions &o);

    int Reserve(uint32_t attempt);
    int Unreserve();
    int AllocLocal(uint64_t size, std::shared_ptr<MemSlice> &out);
    int FreeLocal(const std::shared_ptr<MemSlice> &s);
    int Export(const MemSlice &s, hybm_exchange_info *out);
    int Import(const hybm_exchange_info &in, uint64_t *addr);
    int Mmap();
    void UnmapAll();
    int RemoveImported(uint32_t rank);
    uint64_t Base() const { return base_; }
    uint64_t Slot() const { return opt_.slot; }
    // The window as callers see it: the same as Base() / Slot() unless the segment is compact (see kGva56Base).
    bool Compact() const { return opt_.publicSlot != 0; }
    uint64_t PubBase() const { return Compact() ? pubBase_ : base_; }
    uint64_t PubSlot() const { return Compact() ? opt_.publicSlot : opt_.slot; }
    // address inside this process of (rank, offset) / address a caller sees for an address of this process
    uint64_t LocalOf(uint32_t rank, uint64_t offset) const { return base_ + opt_.slot * rank + offset; }
    uint64_t ToPublic(uint64_t va) const
    {
        if (!Compact()) return va;
        const uint64_t rel = va - base_, r = rel / opt_.slot;
        return pubBase_ + r * opt_.publicSlot + (rel - r * opt_.slot);
    }
    uint64_t LocalBytes() const { return localUsed_; }
    hybm_mem_type Type() const { return opt_.type; }
    bool RankMapped(uint32_t rank);
    // Bytes of `rank`'s slot that are mapped here, contiguous from the slot start (lock-free read; the
    // copy path uses it to refuse a range that would run into unmapped address space).
    uint64_t MappedBytes(uint32_t rank) const
    {
        return rank < mappedBytes_.size() ? mappedBytes_[rank].load(std::memory_order_acquire) : 0;
    }
    std::vector<std::shared_ptr<MemSlice>> LocalSlices();

protected:
    virtual int ReserveRange(uint64_t hint, uint64_t size) = 0;
    virtual int ReleaseRange(uint64_t base, uint64_t size) = 0;
    virtual int MapLocal(MemSlice &s, std::string &source, uint64_t &token) = 0;
    virtual int UnmapLocal(MemSlice &s) = 0;
    virtual int MapPeer(PeerSlice &p) = 0;
    virtual int UnmapPeer(PeerSlice &p) = 0;
    virtual uint64_t Granule() const = 0;

    SegmentOptions opt_;
    uint64_t base_ = 0;
    uint64_t pubBase_ = 0;
    uint64_t localUsed_ = 0;
    std::mutex mu_;
    struct LocalRec {
        std::shared_ptr<MemSlice> slice;
        std::string source;
        uint64_t token = 0;
    };
    std::vector<LocalRec> locals_;
    std::vector<PeerSlice> peers_;
    std::vector<std::atomic<uint64_t>> mappedBytes_;
    void RecomputeMapped(uint32_t rank);  // mu_ held
};
using SegmentPtr = std::shared_ptr<Segment>;

}  // namespace hybm
}  // namespace mf
