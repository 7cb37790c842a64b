// Data operators: how bytes move once both ends of a copy are resolved.
//   SM kernel   — device<->device (local or peer HBM over NVLink) and device<->pinned pooled DRAM for
//                 batches of small segments: items are cut into equal work chunks, written into a
//                 pinned descriptor ring the kernel reads directly, one launch per batch
//   copy engine — device<->host legs of large or unpinned buffers: one async memcpy per item
//   host memcpy — host<->host through the mapped shared memory, split over a thread pool when large
//   process VM  — a peer's registered *host* buffer: process_vm_readv / process_vm_writev
// The compose operator picks per item, coalesces address-adjacent items first, and falls back from
// the kernel to the copy engine when a launch fails.
// Parity: src/hybm/csrc/data_operation/host/hybm_compose_data_op.cpp:26-291 (selection + fallback),
// hybm_data_op_sdma.cpp:403-463,590-805 (coalescing, param ring, async/wait),
// hybm_data_op_host_shm.cpp:41-178 (host memcpy leg).
#pragma once
#include <atomic>
#include <memory>
#include <mutex>
#include <vector>

#include "mf_device.h"
#include "mf_hybm_types.h"

namespace mf {
namespace hybm {

enum EpKind : uint8_t {
    EP_HOST = 0,         // ordinary host memory of this process
    EP_HOST_PINNED = 1,  // pooled DRAM: mapped in this process, pinned and device-visible when a GPU is attached
    EP_DEVICE = 2,       // device memory reachable from this process (local, pooled or IPC-mapped)
    EP_REMOTE_VM = 3,    // host memory of another process, reached through process_vm_*
};

struct Endpoint {
    uint64_t addr = 0;
    EpKind kind = EP_HOST;
    int32_t pid = 0;
};

struct ResolvedCopy {
    Endpoint src, dst;
    uint64_t len = 0;
    uint32_t index = 0;  // position in the caller's batch (for per-item results)
};

struct DataOpStats {
    uint64_t kernelLaunches = 0, kernelItems = 0, engineCopies = 0, hostCopies = 0, vmCopies = 0, coalesced = 0;
};

// A batch whose descriptors were validated, merged and cut into work chunks ONCE and live in pinned memory of their
// own: submitting it again is one kernel launch with no host work per descriptor, and because nothing is written at
// submission time the launch may be recorded into a CUDA graph (the low-latency submission path: the counterpart of the
// reference's own task-scheduler stream, src/hybm/csrc/ts_engine/hybm_stream.cpp, whose point is to cut the per-copy
// host cost).
struct PreparedBatch {
    CopyItem *desc = nullptr;  // pinned, device-visible
    uint32_t count = 0;
    uint64_t bytes = 0;
    bool bulkOk = false;
    uint64_t mapGen = 0;       // membership generation of the entity when it was built
};

class ComposeDataOp {
public:
    ComposeDataOp(DeviceBackend *dev, uint32_t opMask);
    ~ComposeDataOp();
    // Runs the batch. perItem (optional) receives one code per original index.
    int Submit(std::vector<ResolvedCopy> &items, void *userStream, uint32_t flags, int32_t *perItem);
    int Quant(const std::vector<QuantItem> &items, uint32_t unit, int inputFp16, int mode, void *userStream);
    int Wait();
    // items: device<->device copies, already validated. Builds the descriptor block of a PreparedBatch.
    int Prepare(const std::vector<ResolvedCopy> &items, PreparedBatch &out);
    int LaunchPrepared(const PreparedBatch &b, void *stream);
    void ReleasePrepared(PreparedBatch &b);
    // Runs the copy right here when it is a host-to-host memcpy below the size at which it would be split over the
    // thread pool, and says whether it did. Takes no lock: nothing of the operator's state is involved.
    bool HostFast(const ResolvedCopy &c);
    DataOpStats Stats() const
    {
        DataOpStats s = stats_;
        s.hostCopies += fastHost_.load(std::memory_order_relaxed);
        s.kernelLaunches += fastLaunches_.load(std::memory_order_relaxed);
        s.kernelItems += fastItems_.load(std::memory_order_relaxed);
        return s;
    }
    // Tunables (env MF_XCOPY_CHUNK_KB, MF_XCOPY_RING_MB, MF_HOST_COPY_THREADS, MF_XCOPY_ENGINE_MIN_MB).
    uint64_t ChunkBytes() const { return chunk_; }

private:
    int RunHost(const ResolvedCopy &c);
    int RunVm(const ResolvedCopy &c);
    int RunKernel(const std::vector<const ResolvedCopy *> &items, void *stream);
    int RunEngine(const ResolvedCopy &c, void *stream);
    int EnsureRing();
    int CheckCopyStatus();  // ERR_TIMEOUT when a copy kernel reported a wait that ran out since the last check
    void *StreamFor(void *userStream, uint32_t flags);

    DeviceBackend *dev_;
    uint32_t mask_;
    std::mutex mu_;
    void *stream_ = nullptr;  // internal stream
    CopyItem *ring_ = nullptr;
    uint64_t ringCap_ = 0;   // items
    uint64_t ringHead_ = 0;
    std::vector<void *> ringUsers_;  // streams with launches that may still read ring slots
    uint64_t chunk_;
    uint64_t hostSplit_;
    uint64_t engineMin_ = 0;  // device<->device items of at least this many bytes go to a copy engine (0: never)
    std::unique_ptr<ThreadPool> pool_;
    DataOpStats stats_;
    std::atomic<uint64_t> fastHost_{0}, fastLaunches_{0}, fastItems_{0};
    bool pending_ = false;
    friend class KernelBatch;
};

// Streaming writer for the hot case (every item goes to the SM kernel): the caller validates an item
// and hands it over; neighbours that continue one another are merged, the result is cut into work
// chunks written straight into the descriptor ring, and one launch covers the batch. No per-item
// allocation, no intermediate list. Holds the operator's lock for its lifetime.
class KernelBatch {
public:
    KernelBatch(ComposeDataOp &op, void *userStream, uint32_t flags, uint64_t totalBytes);
    bool Ready() const { return rc_ == OK; }
    inline void Add(uint64_t src, uint64_t dst, uint64_t len)
    {
        if (pendLen_ != 0 && pendSrc_ + pendLen_ == src && pendDst_ + pendLen_ == dst) {
            pendLen_ += len;
            op_.stats_.coalesced++;
            alignMask_ |= len;
            return;
        }
        if (pendLen_ != 0) Emit();
        alignMask_ |= src | dst | len;
        pendSrc_ = src;
        pendDst_ = dst;
        pendLen_ = len;
    }
    int Finish();

private:
    inline void Emit()
    {
        uint64_t off = 0;
        while (off < pendLen_) {
            if (op_.ringHead_ >= op_.ringCap_) Wrap();
            uint64_t n = pendLen_ - off < chunk_ ? pendLen_ - off : chunk_;
            op_.ring_[op_.ringHead_++] = CopyItem{pendSrc_ + off, pendDst_ + off, n};
            off += n;
        }
        pendLen_ = 0;
    }
    void Wrap();
    int Launch();
    ComposeDataOp &op_;
    std::unique_lock<std::mutex> lock_;
    void *stream_ = nullptr;
    uint32_t flags_;
    uint64_t chunk_ = 0;
    uint64_t first_ = 0;
    uint64_t pendSrc_ = 0, pendDst_ = 0, pendLen_ = 0;
    uint64_t alignMask_ = 0;  // OR of every address and length handed in: low four bits clear = bulk-copy kernel allowed
    int rc_ = OK;
};

}  // namespace hybm
}  // namespace mf
