// smem_bm_* C entry points: parameter checks, process-wide init (store role, auto-ranking, retries),
// handle registry, dispatch to BmEntry.
// Parity: src/smem/csrc/smem_bm/smem_bm.cpp:28-570, smem_bm_entry_manager.cpp:46-155.
#include "../util/mf_trace.h"
#include "../include/hybm.h"
#include "mf_smem_bm.h"

using namespace mf;
using namespace mf::smem;

namespace {
std::mutex g_mu;
BmGlobals g_bm;
// leaked on purpose: tearing pools down from static destructors would call into a CUDA driver that
// is already shutting down
HandleTable<BmEntry> &g_handles = *new HandleTable<BmEntry>();
constexpr uint32_t kInitTries = 5;

BmEntryPtr H(smem_bm_t h)
{
    if (h == nullptr) {
        MF_FAIL(SMEM_INVALID_PARAM, "handle is NULL");
        return nullptr;
    }
    auto e = g_handles.Find(h);
    if (!e) MF_FAIL(SMEM_INVALID_PARAM, "handle %p is not a live Big Memory object", h);
    return e;
}
}  // namespace

extern "C" {

int32_t smem_bm_config_init(smem_bm_config_t *config)
{
    if (config == nullptr) return MF_FAIL(SMEM_INVALID_PARAM, "config is NULL");
    memset(config, 0, sizeof(*config));
    config->initTimeout = kDefaultTimeoutSec;
    config->createTimeout = kDefaultTimeoutSec;
    config->controlOperationTimeout = kDefaultTimeoutSec;
    config->startConfigStoreServer = true;
    config->startConfigStoreOnly = false;
    config->dynamicWorldSize = false;
    config->unifiedAddressSpace = true;
    config->autoRanking = true;   // the reference's default (smem_bm.cpp:38-39): ranks come from the store ...
    config->rankId = UINT16_MAX;  // ... unless the caller names one (see smem_bm_init)
    config->flags = 0;
    return SMEM_OK;
}

int32_t smem_bm_init(const char *storeURL, uint32_t worldSize, uint16_t deviceId, const smem_bm_config_t *config)
{
    if (storeURL == nullptr || *storeURL == 0) return MF_FAIL(SMEM_INVALID_PARAM, "store url is empty");
    if (config == nullptr) return MF_FAIL(SMEM_INVALID_PARAM, "config is NULL");
    if (worldSize == 0 || worldSize > SMEM_WORLD_SIZE_MAX) return MF_FAIL(SMEM_INVALID_PARAM, "world size %u out of (0, %u]", worldSize, SMEM_WORLD_SIZE_MAX);
    if (config->initTimeout == 0 || config->createTimeout == 0 || config->controlOperationTimeout == 0)
        return MF_FAIL(SMEM_INVALID_PARAM, "timeouts must be at least 1 second");
    if (!config->unifiedAddressSpace) return MF_FAIL(SMEM_INVALID_PARAM, "unifiedAddressSpace must be true");
    // autoRanking is on by default. A caller that also names a valid rank wants that rank (the reference's own
    // examples set rank_id and leave auto_ranking alone, then address slices by that rank): the store assigns
    // ranks only when none was named.
    const bool autoRank = config->autoRanking && config->rankId >= worldSize;
    if (!autoRank && !config->startConfigStoreOnly && config->rankId >= worldSize)
        return MF_FAIL(SMEM_INVALID_PARAM, "rank id %u outside world %u (or enable autoRanking)", config->rankId, worldSize);
    if (!SmemInited()) return MF_FAIL(SMEM_NOT_INIT, "smem_init has not been called");
    std::lock_guard<std::mutex> g(g_mu);
    if (g_bm.inited) return MF_FAIL(SMEM_REPEAT_INVOKE, "smem_bm_init called twice");
    FaultPoints::RegisterBuiltins();

    if (config->storeTlsConfig.tlsEnable) {
        // the path fields of the config select TLS for this process's store links (same effect as smem_set_conf_store_tls)
        const smem_tls_config &t = config->storeTlsConfig;
        auto str = [](const char *a, size_t n) { return std::string(a, strnlen(a, n)); };
        net::TlsSettings ts;
        ts.enable = true;
        ts.caPath = str(t.caPath, sizeof(t.caPath));
        ts.crlPath = str(t.crlPath, sizeof(t.crlPath));
        if (!ts.crlPath.empty()) ts.crlFiles.push_back(ts.crlPath);  // the config names one CRL file
        ts.certPath = str(t.certPath, sizeof(t.certPath));
        ts.keyPath = str(t.keyPath, sizeof(t.keyPath));
        ts.keyPassPath = str(t.keyPassPath, sizeof(t.keyPassPath));
        ts.packagePath = str(t.packagePath, sizeof(t.packagePath));
        ts.decrypterLibPath = str(t.decrypterLibPath, sizeof(t.decrypterLibPath));
        int rc = store::StoreFactory::SetTlsConfig(ts);
        if (rc != OK) return Pub(rc);
    }

    if (config->startConfigStoreOnly) {
        int rc = store::StoreFactory::CreateServerOnly(storeURL, worldSize, 0);
        if (rc != OK) return Pub(rc);
        g_bm = BmGlobals();
        g_bm.storeUrl = storeURL;
        g_bm.inited = true;
        return SMEM_OK;
    }
    // Who serves the store: with fixed ranks, rank 0 when allowed to; with auto-ranking every process
    // that is allowed to races for the port and the losers become clients.
    // Behind an etcd:// or reg:// URL the store is highly available: every process that is allowed to serve stands for
    // election, whatever its rank, so that one of them can take over when the leader's process dies.
    store::StoreUrl parsed;
    const bool ha = store::StoreUrl::Parse(storeURL, parsed) && parsed.scheme != store::StoreUrl::TCP;
    bool serve = config->startConfigStoreServer && (autoRank || config->rankId == 0 || ha);
    uint32_t linkRank = autoRank ? store::kAutoRank : config->rankId;
    store::StorePtr base;
    int err = OK;
    for (uint32_t attempt = 0; attempt < kInitTries && !base; attempt++) {
        uint32_t perTry = std::max<uint32_t>(1000, 1000u * config->initTimeout / kInitTries);
        base = store::StoreFactory::CreateStore(storeURL, serve, worldSize, linkRank, perTry, 0, &err);
        if (!base && err != ERR_RECONNECT && err != ERR_NOT_CONNECTED && err != ERR_TIMEOUT) break;
    }
    if (!base) return MF_FAIL(Pub(err), "cannot reach the config store at %s (%d)", storeURL, err);
    uint32_t rank = config->rankId;
    if (autoRank) {
        int rc = base->AutoRank(rank);
        if (rc != OK) {
            store::StoreFactory::DestroyStore(storeURL);
            return Pub(rc);
        }
    }
    int rc = hybm::HybmInit(deviceId, 0);
    if (rc != OK) {
        store::StoreFactory::DestroyStore(storeURL);
        return Pub(rc);
    }
    g_bm = BmGlobals();
    g_bm.storeUrl = storeURL;
    g_bm.worldSize = worldSize;
    g_bm.deviceId = deviceId;
    g_bm.config = *config;
    g_bm.store = store::StoreFactory::Prefixed(base, "BM_");
    g_bm.rank = rank;
    g_bm.inited = true;
    g_bm.hybmInited = true;
    MF_INFO("big memory initialised: rank %u of %u, store %s", rank, worldSize, storeURL);
    return SMEM_OK;
}

void smem_bm_uninit(uint32_t)
{
    std::lock_guard<std::mutex> g(g_mu);
    if (!g_bm.inited) return;
    for (auto &e : g_handles.TakeAll()) e.reset();
    bool serverOnly = !g_bm.store;
    g_bm.store.reset();
    if (serverOnly) store::StoreFactory::DestroyServer(g_bm.storeUrl);
    else store::StoreFactory::DestroyStore(g_bm.storeUrl);
    if (g_bm.hybmInited) hybm::HybmUninit();
    FaultPoints::UnregisterBuiltins();
    g_bm = BmGlobals();
}

uint32_t smem_bm_get_rank_id(void)
{
    std::lock_guard<std::mutex> g(g_mu);
    return g_bm.inited ? g_bm.rank : UINT32_MAX;
}

smem_bm_t smem_bm_create2(uint32_t id, const smem_bm_create_option_t *option)
{
    if (option == nullptr) {
        MF_FAIL(SMEM_INVALID_PARAM, "option is NULL");
        return nullptr;
    }
    if (id > kIdMax) {
        MF_FAIL(SMEM_INVALID_PARAM, "id %u above %u", id, kIdMax);
        return nullptr;
    }
    if (option->localDRAMSize == 0 && option->localHBMSize == 0 && option->maxDramSize == 0 && option->maxHbmSize == 0) {
        MF_FAIL(SMEM_INVALID_PARAM, "pool %u: all sizes are zero", id);
        return nullptr;
    }
    if (option->localDRAMSize > option->maxDramSize || option->localHBMSize > option->maxHbmSize) {
        MF_FAIL(SMEM_INVALID_PARAM, "pool %u: local size exceeds the per-rank maximum", id);
        return nullptr;
    }
    if (option->maxHbmSize > kHbmMax || option->maxDramSize > kDramMax) {
        MF_FAIL(SMEM_INVALID_PARAM, "pool %u: per-rank maximum too large", id);
        return nullptr;
    }
    BmGlobals snap;
    {
        std::lock_guard<std::mutex> g(g_mu);
        if (!g_bm.inited || !g_bm.store) {
            MF_FAIL(SMEM_NOT_INIT, "smem_bm_init has not been called");
            return nullptr;
        }
        snap = g_bm;
    }
    auto e = std::make_shared<BmEntry>(id, *option, snap);
    int rc = e->Initialize();
    if (rc != OK) {
        if (LastError::Code() == 0) LastError::Set(Pub(rc), "pool %u: create failed with %d", id, rc);
        return nullptr;
    }
    return g_handles.Add(e);
}

smem_bm_t smem_bm_create(uint32_t id, uint32_t memberSize, smem_bm_data_op_type_t dataOpType, uint64_t localDRAMSize,
                         uint64_t localHBMSize, uint32_t flags)
{
    (void)memberSize;
    smem_bm_create_option_t o{};
    o.maxDramSize = localDRAMSize;
    o.maxHbmSize = localHBMSize;
    o.localDRAMSize = localDRAMSize;
    o.localHBMSize = localHBMSize;
    o.dataOpType = dataOpType;
    o.flags = flags;
    o.dramShmFd = -1;
    return smem_bm_create2(id, &o);
}

void smem_bm_destroy(smem_bm_t handle)
{
    auto e = g_handles.Take(handle);
    if (!e) return;
    if (e->Joined()) e->Leave(0);
    e.reset();
}

int32_t smem_bm_join(smem_bm_t handle, uint32_t flags)
{
    auto e = H(handle);
    return e ? Pub(e->Join(flags)) : SMEM_INVALID_PARAM;
}

int32_t smem_bm_leave(smem_bm_t handle, uint32_t flags)
{
    auto e = H(handle);
    return e ? Pub(e->Leave(flags)) : SMEM_INVALID_PARAM;
}

int32_t smem_bm_extend_local_mem(smem_bm_t handle, smem_bm_mem_type_t memType, uint64_t size)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    if (size == 0 || memType >= SMEM_MEM_TYPE_BUTT) return MF_FAIL(SMEM_INVALID_PARAM, "extend: zero size or bad memory type");
    return Pub(e->ExtendLocal(memType, size));
}

int32_t smem_bm_set_group_event_handler(smem_bm_t handle, smem_bm_group_event_cb cb, void *context)
{
    auto e = H(handle);
    return e ? Pub(e->SetEventHandler(cb, context)) : SMEM_INVALID_PARAM;
}

uint64_t smem_bm_get_local_mem_size_by_mem_type(smem_bm_t handle, smem_bm_mem_type_t memType)
{
    auto e = H(handle);
    return e ? e->LocalSize(memType) : 0;
}

void *smem_bm_ptr_by_mem_type(smem_bm_t handle, smem_bm_mem_type_t memType, uint16_t peerRankId)
{
    auto e = H(handle);
    return e ? e->PtrOf(memType, peerRankId) : nullptr;
}

int32_t smem_bm_gva_to_va(smem_bm_t handle, void *gva, smem_bm_mem_type_t vaMemType, void **va)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    if (gva == nullptr || va == nullptr) return MF_FAIL(SMEM_INVALID_PARAM, "gva or va is NULL");
    if (vaMemType != SMEM_MEM_TYPE_LOCAL_DEVICE && vaMemType != SMEM_MEM_TYPE_LOCAL_HOST)
        return MF_FAIL(SMEM_INVALID_PARAM, "memory type must be LOCAL_DEVICE or LOCAL_HOST");
    if (e->RankOfGva(gva) == UINT32_MAX) return MF_FAIL(SMEM_ERROR, "%p is not inside this pool", gva);
    // the pool is mapped at its global address in every member; a window of 56-bit addresses is mapped elsewhere (compact)
    uint64_t local = 0;
    if (hybm_gva_to_va(reinterpret_cast<uint64_t>(gva), HYBM_MEM_TYPE_HOST, &local) != 0)
        return MF_FAIL(SMEM_ERROR, "%p is not mapped in this process", gva);
    *va = reinterpret_cast<void *>(local);
    return SMEM_OK;
}

int32_t smem_bm_copy(smem_bm_t handle, smem_copy_params_t *params, smem_bm_copy_type_t t, uint32_t flags)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    if (params == nullptr || params->src == nullptr || params->dest == nullptr || params->dataSize == 0 || t >= SMEMB_COPY_BUTT)
        return MF_FAIL(SMEM_INVALID_PARAM, "copy: null address, zero size or bad copy type");
    return Pub(e->Copy(*params, t, flags));
}

static int32_t BatchCheck(const smem_batch_copy_params_t *p, smem_bm_copy_type_t t)
{
    if (p == nullptr || p->sources == nullptr || p->destinations == nullptr || p->dataSizes == nullptr || p->batchSize == 0 ||
        t >= SMEMB_COPY_BUTT)
        return MF_FAIL(SMEM_INVALID_PARAM, "batch copy: null array, empty batch or bad copy type");
    return SMEM_OK;
}

int32_t smem_bm_copy_batch(smem_bm_t handle, smem_batch_copy_params_t *params, smem_bm_copy_type_t t, uint32_t flags)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    int32_t rc = BatchCheck(params, t);
    return rc != SMEM_OK ? rc : Pub(e->CopyBatch(*params, t, flags, nullptr));
}

int32_t smem_bm_copy_batch_partial_succeed(smem_bm_t handle, smem_batch_copy_params_t *params, smem_bm_copy_type_t t,
                                           uint32_t flags, smem_batch_copy_result *result)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    int32_t rc = BatchCheck(params, t);
    if (rc != SMEM_OK) return rc;
    if (result == nullptr || result->results == nullptr || result->batchSize < params->batchSize)
        return MF_FAIL(SMEM_INVALID_PARAM, "batch copy: result array missing or shorter than the batch");
    for (uint32_t i = 0; i < params->batchSize; i++) result->results[i] = SMEM_OK;
    rc = e->CopyBatch(*params, t, flags & ~ASYNC_COPY_FLAG, result->results);
    uint32_t bad = 0;
    for (uint32_t i = 0; i < params->batchSize; i++) {
        result->results[i] = Pub(result->results[i]);
        bad += result->results[i] != SMEM_OK;
    }
    if (bad == 0) return Pub(rc);
    return bad == params->batchSize ? Pub(rc != OK ? rc : (int)ERR) : SMEM_PARTIAL_FAILED;
}

int32_t smem_bm_wait(smem_bm_t handle)
{
    auto e = H(handle);
    return e ? Pub(e->Wait()) : SMEM_INVALID_PARAM;
}

int32_t smem_bm_register_user_mem(smem_bm_t handle, uint64_t addr, uint64_t size)
{
    auto e = H(handle);
    if (!e) return SMEM_INVALID_PARAM;
    if (addr == 0 || size == 0) return MF_FAIL(SMEM_INVALID_PARAM, "register: null address or zero size");
    return Pub(e->RegisterUser(addr, size));
}

int32_t smem_bm_unregister_user_mem(smem_bm_t handle, uint64_t addr)
{
    auto e = H(handle);
    return e ? Pub(e->UnregisterUser(addr)) : SMEM_INVALID_PARAM;
}

uint32_t smem_bm_get_rank_id_by_gva(smem_bm_t handle, void *gva)
{
    auto e = H(handle);
    return e ? e->RankOfGva(gva) : UINT32_MAX;
}

// Extension (not in the reference ABI): quantise-while-copy on a pool object (the reference reaches this kernel only
// through smem_trans_batch_quant_write). Sources are bf16 / fp16 device buffers, destinations and factor arrays device
// addresses of this rank or of a peer's slice; params->flags & HYBM_QUANT_FP8_E4M3 selects fp8 e4m3 with 1 x 128 factors.
int32_t mf_bm_quant_copy(smem_bm_t handle, hybm_quant_copy_params *params)
{
    auto e = H(handle);
    if (!e || params == nullptr) return SMEM_INVALID_PARAM;
    return Pub(e->Entity()->QuantCopy(*params, (params->flags & HYBM_QUANT_FP8_E4M3) ? 1 : 0));
}

// Extension (not in the reference ABI): counters of what the copy paths did since creation, in the order
// kernel launches, kernel work chunks, copy-engine copies, host memcpys, process-VM copies, coalesced items.
int32_t mf_bm_copy_stats(smem_bm_t handle, uint64_t out[6])
{
    auto e = H(handle);
    if (!e || out == nullptr) return SMEM_INVALID_PARAM;
    auto s = e->Entity()->CopyStats();
    out[0] = s.kernelLaunches;
    out[1] = s.kernelItems;
    out[2] = s.engineCopies;
    out[3] = s.hostCopies;
    out[4] = s.vmCopies;
    out[5] = s.coalesced;
    return SMEM_OK;
}

// Extension: prepared batches (see include/mf_bm_ext.h).
struct mf_bm_batch {
    std::shared_ptr<mf::smem::BmEntry> entry;
    mf::hybm::PreparedBatch batch;
};

int32_t mf_bm_batch_create(smem_bm_t handle, const smem_batch_copy_params_t *params, smem_bm_copy_type_t t, mf_bm_batch **out)
{
    auto e = H(handle);
    if (!e || out == nullptr) return SMEM_INVALID_PARAM;
    int32_t rc = BatchCheck(params, t);
    if (rc != SMEM_OK) return rc;
    auto b = std::make_unique<mf_bm_batch>();
    b->entry = e;
    rc = Pub(e->PrepareBatch(*params, t, b->batch));
    if (rc != SMEM_OK) return rc;
    *out = b.release();
    return SMEM_OK;
}

int32_t mf_bm_batch_launch(mf_bm_batch *b, void *stream)
{
    if (b == nullptr || !b->entry) return SMEM_INVALID_PARAM;
    return Pub(b->entry->Entity()->LaunchPrepared(b->batch, stream));
}

uint64_t mf_bm_batch_bytes(mf_bm_batch *b) { return b != nullptr ? b->batch.bytes : 0; }

int32_t mf_bm_batch_destroy(mf_bm_batch *b)
{
    if (b == nullptr) return SMEM_INVALID_PARAM;
    if (b->entry) b->entry->Entity()->ReleasePrepared(b->batch);
    delete b;
    return SMEM_OK;
}

// Extension: shape of the bulk-copy (TMA) variant of the xcopy kernel for the launches that follow:
// pipelines per CTA (0: register-copy kernel only), stages per pipeline (>= 4), KiB per stage.
int32_t mf_xcopy_bulk_config(int pipes, int stages, int pieceKb)
{
    auto *dev = mf::hybm::CurrentBackend();
    if (dev == nullptr) return SMEM_NOT_INIT;
    dev->BindThread();
    return dev->ConfigureBulkCopy(pipes, stages, pieceKb) == 0 ? SMEM_OK : SMEM_INVALID_PARAM;
}

}  // extern "C"
