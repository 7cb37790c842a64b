// Memory entity: owns the segments (pooled HBM and/or DRAM) of one pool instance, the imported peers,
// user-registered buffers and the data operators that move bytes between any two of them.
// Bring-up order used by the smem layer: Create -> ReserveMemSpace -> AllocLocal -> Export ->
// (blobs travel through the config store) -> Import -> Mmap -> CopyData/BatchCopyData.
// Parity: src/hybm/csrc/entity/hybm_entity_default.{h,cpp}:42-129,186-327,343-466,531-667,709-849,
// src/hybm/csrc/entity/hybm_entity_tag_info.h:24-56, src/hybm/csrc/hybm_data_op_entry.cpp:22-140.
#pragma once
#include <atomic>

#include "mf_data_op.h"
#include "mf_segment.h"

namespace mf {
namespace hybm {

struct PeerEntity {
    uint32_t rank = 0;
    uint32_t role = 0;
    int32_t pid = 0;
    int32_t devId = -1;
    std::string host;  // boot id: equal on processes of one machine
    std::string tag;
};

// A buffer registered by a peer (Trans / register_user_mem): reachable either through a CUDA IPC
// mapping (device memory) or through process_vm_readv/writev (host memory).
struct RemoteRegion {
    uint32_t rank = 0;
    uint64_t remoteAddr = 0;
    uint64_t size = 0;
    bool device = false;
    int32_t pid = 0;
    uint64_t mapped = 0;      // local address of the IPC mapping of the allocation base (device regions)
    uint64_t mappedBase = 0;  // remote address that `mapped` corresponds to
    uint8_t ipc[64] = {0};
};

class Entity : public std::enable_shared_from_this<Entity> {
public:
    static std::shared_ptr<Entity> Create(uint16_t id, const hybm_options &opt);
    Entity(uint16_t id, const hybm_options &opt, DeviceBackend *dev);
    ~Entity();

    uint16_t Id() const { return id_; }
    const hybm_options &Options() const { return opt_; }
    DeviceBackend *Device() const { return dev_; }

    int ReserveMemSpace(uint32_t attempt);
    int UnreserveMemSpace();
    void *MemoryPtr(hybm_mem_type t);
    int AllocLocal(hybm_mem_type t, uint64_t size, uint32_t flags, MemSlice **out);
    int FreeLocal(MemSlice *s);
    int RegisterLocal(const void *ptr, uint64_t size, uint32_t flags, MemSlice **out);
    int UnregisterLocal(uint64_t addr);
    int Export(const MemSlice *s, hybm_exchange_info *out);
    int Import(const hybm_exchange_info infos[], uint32_t count, void *addresses[]);
    int Mmap();
    void Unmap();
    int RemoveImported(uint32_t rank);
    int SetExtraContext(const void *ctx, uint32_t size);
    int ReachTypes(uint32_t rank, uint32_t &types);
    uint64_t LocalBytes(hybm_mem_type t);
    SegmentPtr SegmentOf(hybm_mem_type t) { return t == HYBM_MEM_TYPE_HOST ? dram_ : hbm_; }

    int CopyData(const hybm_copy_params &p, hybm_data_copy_direction dir, void *stream, uint32_t flags);
    int BatchCopyData(const hybm_batch_copy_params &p, hybm_data_copy_direction dir, void *stream, uint32_t flags,
                      int32_t *perItem = nullptr);
    int QuantCopy(const hybm_quant_copy_params &p, int mode = 0);
    int Wait();
    // Prepared batches (device-to-device directions): validated once, submitted by one launch each time.
    int PrepareBatch(const hybm_batch_copy_params &p, hybm_data_copy_direction dir, PreparedBatch &out);
    int LaunchPrepared(const PreparedBatch &b, void *stream);
    void ReleasePrepared(PreparedBatch &b) { ops_->ReleasePrepared(b); }
    // Runs copies whose two ends the caller already resolved (the Trans layer, after translating a
    // peer's addresses).
    int SubmitResolved(std::vector<ResolvedCopy> &items, void *stream, uint32_t flags)
    {
        return ops_->Submit(items, stream, flags, nullptr);
    }
    int SubmitQuant(const std::vector<QuantItem> &items, uint32_t unit, int fp16, int mode, void *stream)
    {
        return ops_->Quant(items, unit, fp16, mode, stream);
    }
    DataOpStats CopyStats() const { return ops_->Stats(); }

    // Translates an address valid in `rank`'s process (a buffer it registered) for use here.
    int TranslateRemote(uint32_t rank, uint64_t addr, uint64_t len, RemoteRegion &out, uint64_t &local);
    std::vector<PeerEntity> Peers();

private:
    // Resolves one side of a copy to how it can be accessed. Returns OK or an error for a bad range.
    int Resolve(uint64_t addr, uint64_t len, bool isSrc, hybm_data_copy_direction dir, Endpoint &ep);
    // local (optional): where the range is mapped in this process (the address itself unless the segment is compact)
    bool InPool(const SegmentPtr &seg, uint64_t addr, uint64_t len, int &err, uint64_t *local = nullptr) const;
    bool PinnedHost(uint64_t addr, uint64_t len);
    void PublishCopyWindow();  // MF_XCOPY_DEBUG=1: hands the copy kernels the pool window they check descriptors against
    std::mutex pinMu_;
    uint64_t pinLo_ = 0, pinHi_ = 0, pinStampMs_ = 0;  // last host range found pinned and device-addressable, and when

    uint16_t id_;
    hybm_options opt_;
    DeviceBackend *dev_;
    SegmentPtr hbm_, dram_;
    std::mutex mu_;
    std::vector<std::unique_ptr<MemSlice>> slices_;          // handles given to callers
    std::map<MemSlice *, std::shared_ptr<MemSlice>> pooled_; // handle -> segment slice
    std::map<uint64_t, std::unique_ptr<MemSlice>> userSlices_;
    std::map<uint32_t, PeerEntity> peers_;
    std::map<uint32_t, std::map<uint64_t, RemoteRegion>> remote_;  // rank -> remoteAddr -> region
    std::string extraCtx_;
    std::unique_ptr<ComposeDataOp> ops_;
    uint64_t transCursor_ = 0;
    std::atomic<uint64_t> mapGen_{1};  // grows whenever a mapping goes away: prepared batches built before are refused
};
using EntityPtr = std::shared_ptr<Entity>;

// Process-level init of the memory layer (device backend, tracer, fail points).
int HybmInit(uint16_t deviceId, uint64_t flags);
void HybmUninit();
bool HybmInited();

}  // namespace hybm
}  // namespace mf
