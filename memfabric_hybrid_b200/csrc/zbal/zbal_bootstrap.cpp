// zbal bootstrap and library-wide calls.
//
// zbal_bootstrap: smem_init -> smem_shm_init (config store; rank 0 hosts it when asked) ->
// smem_shm_create (one symmetric object for the job: every rank's slice mapped at
// base + rank * symmetricSize by all ranks). The local slice is then split:
//
//   [ communicator slots: commGroupCap x commSlotBytes ][ allocator heap (SMA) ... ]
//
// and the allocator is initialised on the heap part. Slot i of the communicator area has the same
// offset on every rank, so a communicator's flags and staging are reachable on a peer with one
// multiply-add. Parity of role: app/zbal/src/csrc/bootstrap/zbal_mem_mf_bootstrap.cpp:85-295,
// app/zbal/src/include/zbal_def.h:75-98 of the reference.
#include <cstring>

#include "../hybm/mf_device.h"
#include "../include/smem.h"
#include "../include/smem_shm_device.cuh"
#include "../util/mf_util.h"
#include "zbal_state.h"

namespace zbal {

State &S()
{
    static State *s = new State();  // never destroyed: entry points may run during interpreter teardown
    return *s;
}

const Launchers *GetLaunchers()
{
    static Launchers l;
    static std::once_flag once;
    std::call_once(once, [] {
        using mf::hybm::CudaSymbol;
        l.coll = reinterpret_cast<decltype(l.coll)>(CudaSymbol("mf_coll_launch"));
        l.a2a = reinterpret_cast<decltype(l.a2a)>(CudaSymbol("mf_coll_alltoallv"));
        l.send = reinterpret_cast<decltype(l.send)>(CudaSymbol("mf_coll_send"));
        l.recv = reinterpret_cast<decltype(l.recv)>(CudaSymbol("mf_coll_recv"));
        l.barrier = reinterpret_cast<decltype(l.barrier)>(CudaSymbol("mf_coll_barrier"));
        l.argsSize = reinterpret_cast<decltype(l.argsSize)>(CudaSymbol("mf_coll_args_size"));
        l.smCount = reinterpret_cast<decltype(l.smCount)>(CudaSymbol("mf_cuda_sm_count"));
        l.ok = l.coll && l.a2a && l.send && l.recv && l.barrier && l.argsSize && l.argsSize() == sizeof(MfCollArgs);
    });
    if (!l.ok) {
        mf::LastError::Set(Z_NOT_SUPPORTED, "the CUDA kernel library is missing or its argument layout differs from this build");
        return nullptr;
    }
    return &l;
}

}  // namespace zbal

using namespace zbal;

extern "C" {

const char *zbal_version(void) { return "zbal-b200 1.0.0"; }

int32_t zbal_set_logger(void (*func)(int, const char *))
{
    mf::Logger::Get().SetSink(func);
    return Z_OK;
}

int32_t zbal_set_logger_level(int level)
{
    if (level < mf::LOG_DEBUG || level > mf::LOG_OFF) return MF_FAIL(Z_INVALID_PARAM, "log level %d is outside 0..4", level);
    mf::Logger::Get().SetLevel(level);
    return Z_OK;
}

const char *zbal_get_last_error_msg(void) { return mf::LastError::Msg(); }
const char *zbal_get_and_clear_last_error_msg(void) { return mf::LastError::TakeMsg(); }

int32_t zbal_bootstrap_options_init(zbal_bootstrap_options_t *o)
{
    if (o == nullptr) return MF_FAIL(Z_INVALID_PARAM, "options is NULL");
    memset(o, 0, sizeof(*o));
    o->btType = ZBAL_BT_MEMFABRIC;
    o->worldSize = 1;
    o->deviceId = 0;
    o->startConfigServer = true;
    o->deviceMemorySize = 1ull << 30;
    o->dataOperationType = ZBAL_DATA_OP_MTE;
    o->commMetaSpaceSize = 0;
    o->commGroupCap = ZBAL_GROUP_CAP_DEFAULT;
    return Z_OK;
}

int32_t zbal_is_bootstrapped(void)
{
    std::lock_guard<std::mutex> g(S().mu);
    return S().up ? 1 : 0;
}

int32_t zbal_bootstrap_get_output(zbal_bootstrap_output_t *output)
{
    std::lock_guard<std::mutex> g(S().mu);
    if (!S().up || output == nullptr) return Z_NOT_INITIALIZED;
    *output = S().out;
    return Z_OK;
}

static int GrowHook(uint64_t need, void *ctx);

int32_t zbal_bootstrap(zbal_bootstrap_options_t *o, zbal_bootstrap_output_t *output)
{
    if (o == nullptr) return MF_FAIL(Z_INVALID_PARAM, "options is NULL");
    if (o->worldSize == 0 || o->rankId >= o->worldSize || o->worldSize > 16)
        return MF_FAIL(Z_INVALID_PARAM, "rank %u of world %u: the world must have 1..16 ranks", o->rankId, o->worldSize);
    if (o->commGroupCap == 0) o->commGroupCap = ZBAL_GROUP_CAP_DEFAULT;
    if (o->commGroupCap > ZBAL_GROUP_CAP_MAX) return MF_FAIL(Z_INVALID_PARAM, "commGroupCap %u exceeds %u", o->commGroupCap, ZBAL_GROUP_CAP_MAX);
    if (o->ipPort[0] == 0) return MF_FAIL(Z_INVALID_PARAM, "ipPort is empty");
    State &st = S();
    {
        std::lock_guard<std::mutex> g(st.mu);
        if (st.up) return MF_FAIL(Z_ALREADY_INITIALIZED, "zbal is already bootstrapped");
    }
    // slot size of a communicator: signals + 5 staging buffers
    const uint64_t minSlot = kSignalBytes + kStageCount * (256ull << 10);
    const uint64_t maxSlot = kSignalBytes + kStageCount * (32ull << 20);
    uint64_t slot = o->commMetaSpaceSize;
    if (slot == 0) slot = std::min(maxSlot, std::max(minSlot, o->deviceMemorySize / 4 / o->commGroupCap));
    slot = mf::AlignDown(slot, 2ull << 20);
    if (slot < minSlot) slot = mf::AlignUp(minSlot, 2ull << 20);
    const uint64_t commArea = slot * o->commGroupCap;
    if (commArea + (2ull << 20) > o->deviceMemorySize)
        return MF_FAIL(Z_INVALID_PARAM, "deviceMemorySize %lu cannot hold %u communicator slots of %lu bytes plus a heap",
                       (unsigned long)o->deviceMemorySize, o->commGroupCap, (unsigned long)slot);

    int rc = smem_init(0);
    if (rc != 0) return MF_FAIL(Z_ERROR, "smem_init failed (%d)", rc);
    smem_shm_config_t cfg;
    smem_shm_config_init(&cfg);
    cfg.startConfigStoreServer = o->startConfigServer && o->rankId == 0;
    rc = smem_shm_init(o->ipPort, o->worldSize, o->rankId, (uint16_t)o->deviceId, &cfg);
    if (rc != 0) {
        smem_uninit();
        return MF_FAIL(Z_ERROR, "smem_shm_init(%s) failed (%d): %s", o->ipPort, rc, mf::LastError::Msg());
    }
    void *gva = nullptr;
    smem_shm_t shm = smem_shm_create(0, o->worldSize, o->rankId, o->deviceMemorySize, SMEMS_DATA_OP_MTE, 0, &gva);
    if (shm == nullptr) {
        smem_shm_uninit(0);
        smem_uninit();
        return MF_FAIL(Z_ERROR, "smem_shm_create failed: %s", mf::LastError::Msg());
    }
    zbal_bootstrap_output_t out{};
    out.baseGva = reinterpret_cast<uint64_t>(gva);
    out.symmetricSize = smem_shm_get_symmetric_size(shm);
    out.localGva = out.baseGva + (uint64_t)o->rankId * out.symmetricSize;
    out.commAreaSize = commArea;
    out.heapGva = out.localGva + commArea;
    out.heapSize = o->deviceMemorySize - commArea;
    out.worldSize = o->worldSize;
    out.rankId = o->rankId;
    smem_shm_device_ctx_t dctx{};
    const uint64_t mcBase = smem_shm_get_device_context(shm, &dctx, sizeof(dctx)) == 0 ? dctx.mc_base : 0;

    // the communicator area starts zeroed on every rank before anybody may signal
    auto *be = mf::hybm::CurrentBackend();
    if (be != nullptr) {
        be->BindThread();
        be->MemsetAsync(out.localGva, 0, commArea, nullptr);
        be->StreamSync(nullptr);
    }
    rc = smem_shm_control_barrier(shm);
    if (rc != 0) {
        smem_shm_destroy(shm, 0);
        smem_shm_uninit(0);
        smem_uninit();
        return MF_FAIL(Z_ERROR, "bootstrap barrier failed (%d)", rc);
    }
    zbal_allocator_options_t ao{};
    ao.baseAddress = out.heapGva;
    ao.size = out.heapSize;
    ao.deviceId = o->deviceId;
    const bool ownSma = zbal_sma_init(&ao, 0) == Z_OK;
    if (ownSma) zbal_sma_set_grow_hook(GrowHook, nullptr);  // used only with ZBAL_ALLOC_CONF=expandable_segments:True
    {
        std::lock_guard<std::mutex> g(st.mu);
        st.opts = *o;
        st.out = out;
        st.shm = shm;
        st.commSlotBytes = slot;
        st.ownSma = ownSma;
        st.mcBase = mcBase;
        st.spinLimit = (uint32_t)mf::EnvInt("ZBAL_SPIN_LIMIT", nullptr, 1 << 22, 1024, 1u << 30);
        st.up = true;
    }
    // the world communicator always takes slot 0
    zbal_comm_options_t co{};
    snprintf(co.name, sizeof(co.name), "zbal_world");
    co.firstRank = 0;
    co.rankStep = 1;
    co.groupSize = o->worldSize;
    zbal_comm_t world = nullptr;
    rc = zbal_comm_create(&co, &world);
    if (rc != Z_OK) {
        zbal_unbootstrap(0);
        return rc;
    }
    if (output != nullptr) *output = out;
    MF_INFO("zbal up: rank %u/%u, slice %lu MiB (communicators %lu MiB in %u slots, heap %lu MiB)", o->rankId, o->worldSize,
            (unsigned long)(o->deviceMemorySize >> 20), (unsigned long)(commArea >> 20), o->commGroupCap, (unsigned long)(out.heapSize >> 20));
    return Z_OK;
}

// Collective: every rank adds one more symmetric segment to the allocator's heap. The segment is another symmetric object
// with the slot size of the first one, so that rank r's copy of an address p of this rank is p + (r - me) * symmetricSize
// in every segment, and the kernels' one-stride addressing holds across them.
int32_t zbal_heap_expand(uint64_t *segmentBase, uint64_t *segmentBytes)
{
    State &st = S();
    zbal_bootstrap_options_t o;
    zbal_bootstrap_output_t out;
    smem_shm_t first;
    uint32_t id;
    {
        std::lock_guard<std::mutex> g(st.mu);
        if (!st.up) return MF_FAIL(Z_NOT_INITIALIZED, "zbal_heap_expand before zbal_bootstrap");
        if (!st.ownSma) return MF_FAIL(Z_NOT_SUPPORTED, "the heap belongs to an allocator that zbal_bootstrap did not create");
        o = st.opts;
        out = st.out;
        first = st.shm;
        // object 0 is the first segment; expansions count down from the highest id, away from ids an application may use
        if (st.extraShm.size() >= 32) return MF_FAIL(Z_NO_MEMORY, "the symmetric heap already has %zu expansion segments", st.extraShm.size());
        id = 63u - (uint32_t)st.extraShm.size();
    }
    void *gva = nullptr;
    smem_shm_t shm = smem_shm_create(id, o.worldSize, o.rankId, o.deviceMemorySize, SMEMS_DATA_OP_MTE, 0, &gva);
    if (shm == nullptr) return MF_FAIL(Z_NO_MEMORY, "zbal_heap_expand: segment %u could not be created: %s", id, mf::LastError::Msg());
    // one stride for all segments needs the same slot size and, on every rank, the same distance between the objects
    const uint64_t base = reinterpret_cast<uint64_t>(gva);
    int64_t delta = (int64_t)(base - out.baseGva);
    std::vector<int64_t> all(o.worldSize, 0);
    int rc = smem_shm_control_allgather(first, reinterpret_cast<const char *>(&delta), sizeof(delta), reinterpret_cast<char *>(all.data()),
                                        (uint32_t)(sizeof(delta) * o.worldSize));
    bool same = rc == 0 && smem_shm_get_symmetric_size(shm) == out.symmetricSize;
    for (uint32_t r = 0; same && r < o.worldSize; r++) same = all[r] == delta;
    if (!same) {
        smem_shm_destroy(shm, 0);
        return MF_FAIL(Z_ERROR, "zbal_heap_expand: segment %u does not line up with the first one on every rank", id);
    }
    const uint64_t local = base + (uint64_t)o.rankId * out.symmetricSize;
    rc = zbal_sma_add_segment(local, o.deviceMemorySize);
    if (rc != Z_OK) {
        smem_shm_destroy(shm, 0);
        return rc;
    }
    {
        std::lock_guard<std::mutex> g(st.mu);
        st.extraShm.push_back(shm);
        st.extraLocal.push_back(local);
    }
    if (segmentBase != nullptr) *segmentBase = local;
    if (segmentBytes != nullptr) *segmentBytes = o.deviceMemorySize;
    MF_INFO("zbal heap: segment %u of %lu MiB added", id, (unsigned long)(o.deviceMemorySize >> 20));
    return Z_OK;
}

static int GrowHook(uint64_t need, void *)
{
    if (need > S().opts.deviceMemorySize) return -1;  // one more segment would still not hold it
    return zbal_heap_expand(nullptr, nullptr) == Z_OK ? 0 : -1;
}

int32_t zbal_unbootstrap(uint32_t flags)
{
    State &st = S();
    smem_shm_t shm = nullptr;
    std::vector<smem_shm_t> extra;
    bool ownSma = false;
    {
        std::lock_guard<std::mutex> g(st.mu);
        if (!st.up) return Z_NOT_INITIALIZED;
        st.up = false;
        shm = st.shm;
        st.shm = nullptr;
        extra.swap(st.extraShm);
        st.extraLocal.clear();
        ownSma = st.ownSma;
        st.comms.clear();
        st.world.reset();
    }
    zbal_sma_set_grow_hook(nullptr, nullptr);
    if (ownSma) zbal_sma_uninit(0);
    auto *be = mf::hybm::CurrentBackend();
    if (be != nullptr) be->StreamSync(nullptr);
    if (shm != nullptr) {
        // nobody unmaps its slice while a peer may still be writing flags into it
        smem_shm_control_barrier(shm);
        for (smem_shm_t e : extra) smem_shm_destroy(e, flags);
        smem_shm_destroy(shm, flags);
    }
    smem_shm_uninit(flags);
    smem_uninit();
    return Z_OK;
}

}  // extern "C"
