// zbal MoE entry points: a zbal_moe_t carves its receive areas out of the symmetric heap (allocator calls in
// lockstep on every member give the same offsets) and drives the kernels of csrc/kernels/mf_moe.cu and
// mf_gemm_fp8.cu through launchers resolved at run time. Epochs (call numbers of the flags) are kept here, so
// callers only pass tensors.
// Parity of role: app/zbal/src/csrc/operators/zbal_operations.cpp (dispatch / combine / fused entry points) and
// app/zbal/src/csrc/adaptor/deepep/zbal_deepep.cpp:210-700 (buffer ownership, call sequencing) of the reference.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <memory>
#include <mutex>
#include <set>

#include "../hybm/mf_device.h"
#include "../include/zbal_moe.h"
#include "../util/mf_util.h"
#include "zbal_state.h"

namespace zbal {
namespace {

// argument blocks shared with kernels/mf_moe.cu
struct MoeShape {
    int T, K, E, H, max_recv;
};
struct MoeHeap {
    uint64_t counts, recv_x, recv_scale, recv_info, comb, flags;
};
struct DispatchArgs {
    MfTeam team;
    MoeHeap hp;
    MoeShape sh;
    const void *x;
    const int *topk_idx;
    const float *topk_w;
    const int *send_idx;
    const int *put_off;
    uint32_t *done_count;
    uint32_t epoch, seq;
    int *status;
    int raw_bf16;
    const float *smooth;
};

struct MoeLaunchers {
    int (*layout)(const int *, int, int, int, int, int *, int *, int *, uint8_t *, void *) = nullptr;
    int (*notify)(const MfTeam *, const MoeHeap *, int, const int *, int *, int *, int *, int *, uint32_t, void *) = nullptr;
    int (*dispatch)(const DispatchArgs *, int, void *) = nullptr;
    int (*waitAll)(const MfTeam *, const MoeHeap *, int, uint32_t, int *, void *) = nullptr;
    int (*signalAll)(const MfTeam *, const MoeHeap *, int, uint32_t, void *) = nullptr;
    int (*combineReduce)(const MfTeam *, const MoeHeap *, const MoeShape *, const int *, void *, int, void *) = nullptr;
    int (*combinePush)(const MfTeam *, const MoeHeap *, const void *, int64_t, const int *, int, int, int, int, void *) = nullptr;
    int (*llDispatch)(const DispatchArgs *, int *, int *, int *, int *, uint32_t *, int, void *) = nullptr;
    int (*llCombine)(const MfTeam *, const MoeHeap *, const MoeShape *, const void *, int64_t, const int *, int, const int *, const float *,
                     void *, uint32_t, const uint32_t *, int *, int, void *) = nullptr;
    int (*quantRows)(const void *, int64_t, const int *, int, void *, float *, int, void *) = nullptr;
    int (*groupedGemm)(const void *, const float *, int, const void *, const float *, const int *, int, int, int, void *, int64_t, int,
                       const MfTeam *, const void *, uint64_t, int, int *, int, void *) = nullptr;
    int (*groupedGemmMx)(const void *, const float *, int, const void *, const float *, const int *, int, int, int, void *, int64_t, float *, int,
                         const MfTeam *, const void *, uint64_t, int, int *, int, void *) = nullptr;
    int (*mxSupported)(int, int, int, int) = nullptr;
    int (*smCount)() = nullptr;
    bool ok = false;
};

const MoeLaunchers *Moe()
{
    static MoeLaunchers l;
    static std::once_flag once;
    std::call_once(once, [] {
        using mf::hybm::CudaSymbol;
#define SYM(field, name) l.field = reinterpret_cast<decltype(l.field)>(CudaSymbol(name))
        SYM(layout, "mf_moe_layout");
        SYM(notify, "mf_moe_notify");
        SYM(dispatch, "mf_moe_dispatch");
        SYM(waitAll, "mf_moe_wait_all");
        SYM(signalAll, "mf_moe_signal_all");
        SYM(combineReduce, "mf_moe_combine_reduce");
        SYM(combinePush, "mf_moe_combine_push");
        SYM(llDispatch, "mf_moe_ll_dispatch");
        SYM(llCombine, "mf_moe_ll_combine");
        SYM(quantRows, "mf_quant_rows_fp8");
        SYM(groupedGemm, "mf_grouped_gemm_fp8");
        SYM(groupedGemmMx, "mf_grouped_gemm_fp8_mx");
        SYM(mxSupported, "mf_grouped_gemm_fp8_mx_supported");
        SYM(smCount, "mf_cuda_sm_count");
#undef SYM
        l.ok = l.layout && l.notify && l.dispatch && l.waitAll && l.signalAll && l.combineReduce && l.combinePush && l.llDispatch &&
               l.llCombine && l.quantRows && l.groupedGemm && l.smCount;
    });
    if (!l.ok) {
        mf::LastError::Set(Z_NOT_SUPPORTED, "the CUDA kernel library is missing");
        return nullptr;
    }
    return &l;
}

struct MoeCtx {
    std::shared_ptr<Comm> comm;
    zbal_moe_options_t opt{};
    MoeShape sh{};
    MoeHeap hp{}, hpLL{};
    uint32_t El = 0;
    std::vector<void *> allocs;       // blocks from the symmetric allocator
    uint64_t slotBase = 0;            // address of this rank's communicator slot: heap offsets are relative to it
    uint32_t *doneNormal = nullptr, *doneLL = nullptr, *epochLL = nullptr;
    int *status = nullptr;
    uint32_t epoch = 0, dispatches = 0;
    int grid = 148, llGrid = 128;
    bool rawBf16 = false;
    const float *smooth = nullptr;    // smooth-quant factors applied by the dispatch kernels (device, [hidden]); caller-owned
    std::mutex mu;
};

std::mutex g_mu;
std::set<MoeCtx *> g_live;

MoeCtx *Find(zbal_moe_t h)
{
    std::lock_guard<std::mutex> g(g_mu);
    auto *c = static_cast<MoeCtx *>(h);
    if (g_live.count(c) == 0) {
        mf::LastError::Set(Z_INVALID_PARAM, "unknown MoE handle %p", h);
        return nullptr;
    }
    return c;
}

int Launched(int rc, const char *what)
{
    if (rc == 0) return Z_OK;
    return MF_FAIL(Z_LAUNCH_FAILED, "%s: kernel launch failed (%d)", what, rc);
}

// a block of the symmetric heap; returns its offset relative to the communicator slot
bool HeapAlloc(MoeCtx &c, uint64_t bytes, uint64_t align, uint64_t &off, void **ptr = nullptr)
{
    void *p = zbal_pluggable_malloc(bytes + align, 0, nullptr);
    if (p == nullptr) return false;
    c.allocs.push_back(p);
    const uint64_t a = mf::AlignUp(reinterpret_cast<uint64_t>(p), align);
    off = a - c.slotBase;
    if (ptr != nullptr) *ptr = reinterpret_cast<void *>(a);
    return true;
}

}  // namespace
}  // namespace zbal

using namespace zbal;

extern "C" {

int32_t zbal_moe_create(zbal_comm_t comm, const zbal_moe_options_t *o, zbal_moe_t *moe)
{
    if (o == nullptr || moe == nullptr) return MF_FAIL(Z_INVALID_PARAM, "options or moe is NULL");
    auto cm = FindComm(comm);
    if (!cm) return Z_INVALID_PARAM;
    const MoeLaunchers *L = Moe();
    if (L == nullptr) return Z_NOT_SUPPORTED;
    if (o->hidden == 0 || o->hidden % 128 != 0 || o->hidden / 16 > 448) return MF_FAIL(Z_INVALID_PARAM, "hidden must be a multiple of 128, at most 7168");
    if (o->experts == 0 || o->experts > 1024 || o->experts % cm->size != 0) return MF_FAIL(Z_INVALID_PARAM, "experts must divide by the group size, at most 1024");
    if (o->topk == 0 || o->topk > 16 || o->maxTokens == 0) return MF_FAIL(Z_INVALID_PARAM, "topk 1..16 and maxTokens > 0");
    auto c = std::make_unique<MoeCtx>();
    c->comm = cm;
    c->opt = *o;
    c->El = o->experts / cm->size;
    c->rawBf16 = o->rawBf16 != 0;
    const uint32_t maxRecv = o->maxRecv ? o->maxRecv : o->maxTokens * cm->size * std::min<uint32_t>(o->topk, c->El);
    c->sh = MoeShape{(int)o->maxTokens, (int)o->topk, (int)o->experts, (int)o->hidden, (int)maxRecv};
    c->slotBase = cm->team.heap_base + (uint64_t)cm->groupRank * cm->team.stride;
    const uint64_t H = o->hidden;
    void *flagsPtr = nullptr, *countsPtr = nullptr;
    bool ok = HeapAlloc(*c, (uint64_t)cm->size * o->experts * 4, 256, c->hp.counts, &countsPtr) && HeapAlloc(*c, 4 * 16 * 4, 256, c->hp.flags, &flagsPtr) &&
              HeapAlloc(*c, (uint64_t)maxRecv * H * 2, 1024, c->hp.recv_x) && HeapAlloc(*c, (uint64_t)maxRecv * (H / 128) * 4, 256, c->hp.recv_scale) &&
              HeapAlloc(*c, (uint64_t)maxRecv * 16, 256, c->hp.recv_info) && HeapAlloc(*c, (uint64_t)o->maxTokens * o->topk * H * 2, 1024, c->hp.comb);
    uint64_t scratchOff = 0;
    void *scratch = nullptr;
    ok = ok && HeapAlloc(*c, 256, 256, scratchOff, &scratch);
    if (!ok) {
        for (void *p : c->allocs) zbal_pluggable_free(p, 0, 0, nullptr);
        return MF_FAIL(Z_NO_MEMORY, "symmetric heap exhausted while creating the MoE buffers: %s", mf::LastError::Msg());
    }
    c->hpLL = c->hp;
    c->hpLL.flags += 2 * 16 * 4;  // flag rows 2 and 3 belong to the low-latency pair
    auto *words = static_cast<uint32_t *>(scratch);
    c->doneNormal = words, c->doneLL = words + 1, c->epochLL = words + 2;
    c->status = reinterpret_cast<int *>(words + 3);
    auto *be = mf::hybm::CurrentBackend();
    if (be != nullptr) {
        be->BindThread();
        be->MemsetAsync(reinterpret_cast<uint64_t>(flagsPtr), 0, 4 * 16 * 4, nullptr);
        be->MemsetAsync(reinterpret_cast<uint64_t>(countsPtr), 0, (uint64_t)cm->size * o->experts * 4, nullptr);
        be->MemsetAsync(reinterpret_cast<uint64_t>(scratch), 0, 256, nullptr);
        be->StreamSync(nullptr);
    }
    c->grid = std::max(1, L->smCount());
    c->llGrid = std::max(1, std::min<int>((int)o->maxTokens, c->grid));
    // everybody's flags are zero before anybody may signal
    int rc = zbal_barrier(comm, nullptr);
    if (rc == Z_OK && be != nullptr) be->StreamSync(nullptr);
    if (rc != Z_OK) {
        for (void *p : c->allocs) zbal_pluggable_free(p, 0, 0, nullptr);
        return rc;
    }
    MoeCtx *raw = c.release();
    {
        std::lock_guard<std::mutex> g(g_mu);
        g_live.insert(raw);
    }
    *moe = raw;
    return Z_OK;
}

int32_t zbal_moe_destroy(zbal_moe_t moe)
{
    MoeCtx *c = Find(moe);
    if (c == nullptr) return Z_INVALID_PARAM;
    {
        std::lock_guard<std::mutex> g(g_mu);
        g_live.erase(c);
    }
    auto *be = mf::hybm::CurrentBackend();
    if (be != nullptr) be->StreamSync(nullptr);
    for (void *p : c->allocs) zbal_pluggable_free(p, 0, 0, nullptr);
    delete c;
    return Z_OK;
}

int32_t zbal_moe_get_buffers(zbal_moe_t moe, zbal_moe_buffers_t *b)
{
    MoeCtx *c = Find(moe);
    if (c == nullptr || b == nullptr) return Z_INVALID_PARAM;
    b->recvTokens = reinterpret_cast<void *>(c->slotBase + c->hp.recv_x);
    b->recvScales = reinterpret_cast<float *>(c->slotBase + c->hp.recv_scale);
    b->recvInfo = reinterpret_cast<int32_t *>(c->slotBase + c->hp.recv_info);
    b->maxRecv = (uint32_t)c->sh.max_recv;
    b->localExperts = c->El;
    return Z_OK;
}

int32_t zbal_moe_get_status(zbal_moe_t moe, int32_t *status)
{
    MoeCtx *c = Find(moe);
    if (c == nullptr || status == nullptr) return Z_INVALID_PARAM;
    auto *be = mf::hybm::CurrentBackend();
    if (be == nullptr) return Z_NOT_SUPPORTED;
    int rc = be->MemcpyAsync(reinterpret_cast<uint64_t>(status), reinterpret_cast<uint64_t>(c->status), 4, mf::hybm::CPY_D2H, nullptr);
    if (rc == 0) rc = be->StreamSync(nullptr);
    return rc == 0 ? Z_OK : Z_ERROR;
}

int32_t zbal_dispatch_normal_layout(zbal_moe_t moe, const int32_t *topkIndex, int64_t tokens, int32_t *tokensPerRank, int32_t *tokensPerExpert,
                                    int32_t *sendTokensIndex, uint8_t *isTokenInRank, zbal_stream_t stream)
{
    MoeCtx *c = Find(moe);
    if (c == nullptr) return Z_INVALID_PARAM;
    if (!topkIndex || !tokensPerRank || !tokensPerExpert || !sendTokensIndex || !isTokenInRank || tokens <= 0 || tokens > c->sh.T)
        return MF_FAIL(Z_INVALID_PARAM, "layout: NULL tensor or %ld tokens outside 1..%d", (long)tokens, c->sh.T);
    return Launched(Moe()->layout(topkIndex, (int)tokens, c->sh.K, c->sh.E, (int)c->comm->size, tokensPerExpert, tokensPerRank, sendTokensIndex,
                                  isTokenInRank, stream), "dispatch layout");
}

int32_t zbal_dispatch_normal_notify(zbal_moe_t moe, const int32_t *tokensPerExpert, int32_t *recvTokensPerExpert, int32_t *rowOffsets,
                                    int32_t *pushTargetOffset, int32_t *srcOffsets, zbal_stream_t stream)
{
    MoeCtx *c = Find(moe);
    if (c == nullptr) return Z_INVALID_PARAM;
    if (!tokensPerExpert || !recvTokensPerExpert || !rowOffsets || !pushTargetOffset || !srcOffsets) return MF_FAIL(Z_INVALID_PARAM, "notify: NULL tensor");
    std::lock_guard<std::mutex> g(c->mu);
    c->epoch++;
    return Launched(Moe()->notify(&c->comm->team, &c->hp, c->sh.E, tokensPerExpert, recvTokensPerExpert, rowOffsets, pushTargetOffset, srcOffsets,
                                  c->epoch, stream), "dispatch notify");
}

int32_t zbal_dispatch_normal(zbal_moe_t moe, const void *srcTokens, int64_t tokens, const int32_t *topkIndex, const float *topkWeights,
                             const int32_t *sendTokensIndex, const int32_t *pushTargetOffset, zbal_stream_t stream)
{
    MoeCtx *c = Find(moe);
    if (c == nullptr) return Z_INVALID_PARAM;
    if (!srcTokens || !topkIndex || !topkWeights || !sendTokensIndex || !pushTargetOffset || tokens <= 0 || tokens > c->sh.T)
        return MF_FAIL(Z_INVALID_PARAM, "dispatch: NULL tensor or bad token count");
    std::lock_guard<std::mutex> g(c->mu);
    if (c->epoch == 0) return MF_FAIL(Z_INVALID_PARAM, "dispatch before notify");
    DispatchArgs a{};
    a.team = c->comm->team;
    a.hp = c->hp;
    a.sh = c->sh;
    a.sh.T = (int)tokens;
    a.x = srcTokens, a.topk_idx = topkIndex, a.topk_w = topkWeights, a.send_idx = sendTokensIndex, a.put_off = pushTargetOffset;
    a.done_count = c->doneNormal;
    a.epoch = c->epoch;
    a.seq = ++c->dispatches;
    a.status = c->status;
    a.raw_bf16 = c->rawBf16 ? 1 : 0;
    a.smooth = c->smooth;
    int rc = Launched(Moe()->dispatch(&a, c->grid, stream), "dispatch");
    if (rc != Z_OK) return rc;
    return Launched(Moe()->waitAll(&c->comm->team, &c->hp, 0, c->epoch, c->status, stream), "dispatch wait");
}

int32_t zbal_combine_normal(zbal_moe_t moe, const void *srcTokens, int64_t ld, const int32_t *rowsDev, int32_t weighted, const int32_t *topkIndex,
                            int64_t tokens, void *destTokens, zbal_stream_t stream)
{
    MoeCtx *c = Find(moe);
    if (c == nullptr) return Z_INVALID_PARAM;
    if (!srcTokens || !rowsDev || !topkIndex || !destTokens || tokens <= 0 || tokens > c->sh.T) return MF_FAIL(Z_INVALID_PARAM, "combine: NULL tensor or bad token count");
    std::lock_guard<std::mutex> g(c->mu);
    const MoeLaunchers *L = Moe();
    int rc = Launched(L->combinePush(&c->comm->team, &c->hp, srcTokens, ld, rowsDev, c->sh.H, c->sh.K, weighted, c->grid * 2, stream), "combine push");
    if (rc == Z_OK) rc = Launched(L->signalAll(&c->comm->team, &c->hp, 1, c->epoch, stream), "combine signal");
    if (rc == Z_OK) rc = Launched(L->waitAll(&c->comm->team, &c->hp, 1, c->epoch, c->status, stream), "combine wait");
    if (rc != Z_OK) return rc;
    MoeShape sh = c->sh;
    sh.T = (int)tokens;
    return Launched(L->combineReduce(&c->comm->team, &c->hp, &sh, topkIndex, destTokens, (int)std::min<int64_t>(tokens, c->grid * 4), stream), "combine reduce");
}

int32_t zbal_dispatch_low_latency(zbal_moe_t moe, const void *x, int64_t tokens, const int32_t *topkIndex, const float *topkWeights,
                                  int32_t *sendTokensIndex, int32_t *tokensPerExpert, int32_t *recvTokensPerExpert, int32_t *rowOffsets,
                                  int32_t *pushTargetOffset, int32_t *srcOffsets, zbal_stream_t stream)
{
    MoeCtx *c = Find(moe);
    if (c == nullptr) return Z_INVALID_PARAM;
    if (!x || !topkIndex || !topkWeights || !sendTokensIndex || !tokensPerExpert || !recvTokensPerExpert || !rowOffsets || !pushTargetOffset || !srcOffsets ||
        tokens <= 0 || tokens > c->sh.T)
        return MF_FAIL(Z_INVALID_PARAM, "low-latency dispatch: NULL tensor or bad token count");
    DispatchArgs a{};
    a.team = c->comm->team;
    a.hp = c->hpLL;
    a.sh = c->sh;
    a.sh.T = (int)tokens;
    a.x = x, a.topk_idx = topkIndex, a.topk_w = topkWeights, a.send_idx = sendTokensIndex, a.put_off = pushTargetOffset;
    a.done_count = c->doneLL;
    a.epoch = 0, a.seq = 0;  // the kernel numbers its calls in device memory
    a.status = c->status;
    a.raw_bf16 = c->rawBf16 ? 1 : 0;
    a.smooth = c->smooth;
    return Launched(Moe()->llDispatch(&a, tokensPerExpert, recvTokensPerExpert, rowOffsets, srcOffsets, c->epochLL, c->llGrid, stream), "low-latency dispatch");
}

int32_t zbal_combine_low_latency(zbal_moe_t moe, const void *expandX, int64_t ld, const int32_t *rowsDev, int32_t weighted, const int32_t *topkIndex,
                                 const float *homeWeights, int64_t tokens, void *xOut, zbal_stream_t stream)
{
    MoeCtx *c = Find(moe);
    if (c == nullptr) return Z_INVALID_PARAM;
    if (!expandX || !rowsDev || !topkIndex || !xOut || tokens <= 0 || tokens > c->sh.T) return MF_FAIL(Z_INVALID_PARAM, "low-latency combine: NULL tensor or bad token count");
    MoeShape sh = c->sh;
    sh.T = (int)tokens;
    return Launched(Moe()->llCombine(&c->comm->team, &c->hpLL, &sh, expandX, ld, rowsDev, weighted, topkIndex, homeWeights, xOut, 0, c->epochLL, c->status,
                                     c->llGrid, stream), "low-latency combine");
}

uint64_t zbal_fused_deep_moe_workspace(zbal_moe_t moe, uint32_t inter)
{
    MoeCtx *c = Find(moe);
    if (c == nullptr || inter == 0 || inter % 128 != 0) return 0;
    const uint64_t R = (uint64_t)c->sh.max_recv, T = (uint64_t)c->sh.T;
    // layout scratch (per call) + SwiGLU output bf16 + its fp8 requantisation + scales
    return mf::AlignUp(T * c->sh.K * 4 + (uint64_t)c->sh.E * 8 + c->comm->size * 4 + T * c->comm->size + (uint64_t)c->El * (8 + 4 * c->comm->size) + 64, 256) + 1024 +
           R * inter * 2 + R * inter + R * (inter / 128) * 4 + 3 * 256;
}

int32_t zbal_fused_deep_moe_gate_up_tile(zbal_moe_t moe, uint32_t inter)
{
    MoeCtx *c = Find(moe);
    const MoeLaunchers *L = Moe();
    if (c == nullptr || L == nullptr || inter == 0 || inter % 128 != 0) return 0;
    const bool mx = L->groupedGemmMx != nullptr && L->mxSupported != nullptr && L->mxSupported((int)c->El, (int)(2 * inter), c->sh.H, 3) != 0 &&
                    L->mxSupported((int)c->El, c->sh.H, (int)inter, 2) != 0;
    return mx ? 128 : 64;
}

int32_t zbal_fused_deep_moe(zbal_moe_t moe, const void *x, int64_t tokens, const int32_t *topkIndex, const float *topkWeights, const void *gmm1Weight,
                            const float *gmm1Scale, const void *gmm2Weight, const float *gmm2Scale, uint32_t inter, void *workspace, void *xOut,
                            zbal_stream_t stream)
{
    MoeCtx *c = Find(moe);
    if (c == nullptr) return Z_INVALID_PARAM;
    if (c->rawBf16) return MF_FAIL(Z_NOT_SUPPORTED, "the fused path runs on fp8 rows");
    if (!x || !topkIndex || !topkWeights || !gmm1Weight || !gmm1Scale || !gmm2Weight || !gmm2Scale || !workspace || !xOut || inter == 0 || inter % 128 != 0 ||
        tokens <= 0 || tokens > c->sh.T)
        return MF_FAIL(Z_INVALID_PARAM, "fused MoE: NULL tensor, bad token count or intermediate size not a multiple of 128");
    // carve the workspace
    auto p = mf::AlignUp(reinterpret_cast<uint64_t>(workspace), 256);
    auto take = [&](uint64_t bytes) {
        const uint64_t a = p;
        p = mf::AlignUp(p + bytes, 256);
        return a;
    };
    const uint32_t W = c->comm->size, E = (uint32_t)c->sh.E, El = c->El;
    const uint64_t R = (uint64_t)c->sh.max_recv;
    auto *sendIdx = reinterpret_cast<int32_t *>(take((uint64_t)tokens * c->sh.K * 4));
    auto *tpe = reinterpret_cast<int32_t *>(take(E * 4));
    auto *tpr = reinterpret_cast<int32_t *>(take(W * 4));
    auto *inRank = reinterpret_cast<uint8_t *>(take((uint64_t)tokens * W));
    auto *rpe = reinterpret_cast<int32_t *>(take(El * 4));
    auto *rowOff = reinterpret_cast<int32_t *>(take((El + 1) * 4));
    auto *putOff = reinterpret_cast<int32_t *>(take(E * 4));
    auto *srcOff = reinterpret_cast<int32_t *>(take((uint64_t)El * W * 4));
    auto *h = reinterpret_cast<void *>(take(R * inter * 2));
    auto *hq = reinterpret_cast<void *>(take(R * inter));
    auto *hs = reinterpret_cast<float *>(take(R * (inter / 128) * 4));
    int rc = zbal_dispatch_normal_layout(moe, topkIndex, tokens, tpr, tpe, sendIdx, inRank, stream);
    if (rc == Z_OK) rc = zbal_dispatch_normal_notify(moe, tpe, rpe, rowOff, putOff, srcOff, stream);
    if (rc == Z_OK) rc = zbal_dispatch_normal(moe, x, tokens, topkIndex, topkWeights, sendIdx, putOff, stream);
    if (rc != Z_OK) return rc;
    std::lock_guard<std::mutex> g(c->mu);
    const MoeLaunchers *L = Moe();
    const void *recvX = reinterpret_cast<const void *>(c->slotBase + c->hp.recv_x);
    const float *recvS = reinterpret_cast<const float *>(c->slotBase + c->hp.recv_scale);
    const void *recvInfo = reinterpret_cast<const void *>(c->slotBase + c->hp.recv_info);
    if (zbal_fused_deep_moe_gate_up_tile(moe, inter) == 128) {
        // block-scaled tensor-core path: SwiGLU and the re-quantisation to fp8 are the first GEMM's epilogue
        rc = Launched(L->groupedGemmMx(recvX, recvS, (int)R, gmm1Weight, gmm1Scale, rowOff, (int)El, (int)(2 * inter), c->sh.H, hq, inter, hs, 3, nullptr,
                                       nullptr, 0, c->sh.K, c->status, c->grid, stream), "grouped GEMM (gate/up + requantisation)");
        if (rc == Z_OK)
            rc = Launched(L->groupedGemmMx(hq, hs, (int)R, gmm2Weight, gmm2Scale, rowOff, (int)El, c->sh.H, (int)inter, nullptr, 0, nullptr, 2, &c->comm->team,
                                           recvInfo, c->hp.comb, c->sh.K, c->status, c->grid, stream), "grouped GEMM (down + combine)");
    } else {
        rc = Launched(L->groupedGemm(recvX, recvS, (int)R, gmm1Weight, gmm1Scale, rowOff, (int)El, (int)(2 * inter), c->sh.H, h, inter, 1, nullptr, nullptr, 0,
                                     c->sh.K, c->status, c->grid, stream), "grouped GEMM (gate/up)");
        if (rc == Z_OK) rc = Launched(L->quantRows(h, inter, rowOff + El, (int)inter, hq, hs, c->grid * 4, stream), "requantisation");
        if (rc == Z_OK)
            rc = Launched(L->groupedGemm(hq, hs, (int)R, gmm2Weight, gmm2Scale, rowOff, (int)El, c->sh.H, (int)inter, nullptr, 0, 2, &c->comm->team, recvInfo,
                                         c->hp.comb, c->sh.K, c->status, c->grid, stream), "grouped GEMM (down + combine)");
    }
    if (rc == Z_OK) rc = Launched(L->signalAll(&c->comm->team, &c->hp, 1, c->epoch, stream), "combine signal");
    if (rc == Z_OK) rc = Launched(L->waitAll(&c->comm->team, &c->hp, 1, c->epoch, c->status, stream), "combine wait");
    if (rc != Z_OK) return rc;
    MoeShape sh = c->sh;
    sh.T = (int)tokens;
    return Launched(L->combineReduce(&c->comm->team, &c->hp, &sh, topkIndex, xOut, (int)std::min<int64_t>(tokens, c->grid * 4), stream), "combine reduce");
}

}  // extern "C"

// ---- load-balance matrix -----------------------------------------------------------------------------
// The plan the reference's notify kernel derives from the gathered send counts
// (ops/dispatch_combine_normal/zbal_kernel_notify_dispatch.h:421-498): row = helper rank, column pair
// (2c, 2c + 1) = [start, end) of rank c's tokens that the helper pushes on c's behalf, -1 = none. Every rank
// computes the same matrix from the same counts. tokens[r] = sum(counts[r]) / topk; avg = total / ranks; a rank
// above the average may handle ceil(avg * factorHigh) tokens, the others ceil(avg * factorLow); when
// avg <= minTokens every rank handles only itself; otherwise each rank first takes min(tokens, capacity) of its
// own and the overflow of overloaded ranks goes, in rank order, to ranks with spare capacity.
// The dispatch kernels of this library do not use the plan (on NVSwitch a token routed through a helper crosses
// NVLink twice); the function exists for schedulers that want the same numbers the reference would produce.
extern "C" int32_t zbal_moe_set_smooth_scales(zbal_moe_t moe, const float *scales)
{
    MoeCtx *c = Find(moe);
    if (c == nullptr) return Z_INVALID_PARAM;
    if (scales != nullptr && c->rawBf16) return MF_FAIL(Z_INVALID_PARAM, "smooth-quant factors apply to fp8 rows; this object sends raw bf16");
    std::lock_guard<std::mutex> g(c->mu);
    c->smooth = scales;
    return Z_OK;
}

extern "C" int32_t zbal_moe_balance_matrix(const int32_t *counts, uint32_t ranks, uint32_t experts, uint32_t topk, float factorHigh, float factorLow,
                                           uint32_t minTokens, int32_t *matrix)
{
    if (counts == nullptr || matrix == nullptr || ranks == 0 || experts == 0 || topk == 0) return MF_FAIL(Z_INVALID_PARAM, "balance matrix: bad argument");
    std::vector<int64_t> tokens(ranks, 0), cap(ranks, 0), taken(ranks, 0);
    int64_t total = 0;
    for (uint32_t r = 0; r < ranks; r++) {
        int64_t s = 0;
        for (uint32_t e = 0; e < experts; e++) s += counts[(size_t)r * experts + e];
        tokens[r] = s / topk;
        total += tokens[r];
    }
    for (size_t i = 0; i < (size_t)ranks * ranks * 2; i++) matrix[i] = -1;
    const double avg = (double)total / ranks;
    auto put = [&](uint32_t helper, uint32_t owner, int64_t b, int64_t e) {
        matrix[((size_t)helper * ranks + owner) * 2] = (int32_t)b;
        matrix[((size_t)helper * ranks + owner) * 2 + 1] = (int32_t)e;
    };
    if (avg <= (double)minTokens) {
        for (uint32_t r = 0; r < ranks; r++)
            if (tokens[r] > 0) put(r, r, 0, tokens[r]);
        return Z_OK;
    }
    for (uint32_t r = 0; r < ranks; r++) {
        const double f = (double)tokens[r] > avg ? factorHigh : factorLow;
        cap[r] = (int64_t)std::ceil(avg * f - 1e-3);  // the factors arrive as floats: 1.2f is a hair above 1.2
        taken[r] = std::min(tokens[r], cap[r]);
        if (taken[r] > 0) put(r, r, 0, taken[r]);
    }
    uint32_t helper = 0;
    for (uint32_t owner = 0; owner < ranks; owner++) {
        int64_t next = taken[owner];
        while (next < tokens[owner]) {
            while (helper < ranks && (helper == owner || taken[helper] >= cap[helper])) helper++;
            if (helper >= ranks) {
                // nobody has room left: the owner keeps the rest itself
                put(owner, owner, 0, tokens[owner]);
                next = tokens[owner];
                break;
            }
            const int64_t n = std::min(tokens[owner] - next, cap[helper] - taken[helper]);
            put(helper, owner, next, next + n);
            taken[helper] += n;
            next += n;
        }
    }
    return Z_OK;
}
