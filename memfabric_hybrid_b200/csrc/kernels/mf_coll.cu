// Collectives on the symmetric heap: each kernel reads and writes peers' slots directly over NVLink
// (plain loads/stores on mapped peer memory) and fuses the x scale and the output cast into the same
// pass. One launch per collective; CTA b of every rank works on the same element ranges as CTA b of
// every other rank and synchronises only with those (lane flags), so no grid-wide barrier is needed.
//   allreduce  one-shot : stage -> sync -> every rank reads all W copies, reduces, writes its output
//   allreduce  two-shot : stage -> sync -> reduce own 1/W -> push result to all -> sync -> unstage
//   reduce_scatter      : stage -> sync -> reduce own 1/W straight into the output
//   allgather           : push own shard into every peer's gather buffer -> sync -> unstage
//   broadcast, all-to-all-v, send / recv
// Staging buffers A (inputs) and B (results) live in the slot; the host alternates between two sets
// per call so that no trailing synchronisation is needed (a rank can only start call k+2 after every
// peer entered call k+1, i.e. finished reading the buffers of call k).
// Parity of role: app/zbal/src/csrc/operators/npu/aicore/ops/classic/zbal_kernel_{allreduce,
// reducescatter,allgather,alltoallv,broadcast,send,recv,barrier}.* of the reference.
#include <cooperative_groups.h>

#include "mf_coll.cuh"
#include "mf_devtrace.cuh"

namespace mfk {

struct CollArgs {
    Team team;
    uint64_t in;               // local input (rank 0's when emulating)
    uint64_t out;              // local output
    uint64_t in_rank_stride;   // emulation only: distance between consecutive ranks' local buffers
    uint64_t out_rank_stride;
    uint64_t n;                // elements: allreduce/broadcast total; reduce_scatter total input; allgather per-rank input
    uint64_t stage_a;          // slot offset of staging A
    uint64_t stage_b;          // slot offset of staging B
    float scale;
    int op;
    uint32_t epoch;
    uint32_t zero_copy;        // 1: input already sits at stage_a of every slot; 2: direct mode (buffers inside the slices);
                               // 3: direct mode through the multicast alias (team.mc_base)
    uint32_t root;
    uint32_t algo;             // allreduce: 0 one-shot, 1 two-shot; rooted copy: 0 broadcast, 1 scatter
    uint64_t part_stride;      // elements between consecutive members' parts in the user buffer (0: packed):
                               // reduce_scatter input rows, allgather output rows, scatter source parts
};

struct Range {
    uint64_t beg, end;
};

template <int VN> __device__ __forceinline__ Range cta_range(uint64_t count)
{
    uint64_t per = (count + gridDim.x - 1) / gridDim.x;
    per = (per + VN - 1) / VN * VN;
    Range r;
    r.beg = min(count, (uint64_t)blockIdx.x * per);
    r.end = min(count, r.beg + per);
    return r;
}

__device__ __forceinline__ bool aligned16(const void *p) { return (reinterpret_cast<uint64_t>(p) & 15) == 0; }

// dst[i] = (TD)(src[i] * scale) for i in [beg, end): 16-byte vectors where both ends allow it
template <typename TS, typename TD>
__device__ __forceinline__ void cta_convert_copy(const TS *__restrict__ src, TD *__restrict__ dst, uint64_t beg, uint64_t end, float scale)
{
    constexpr int G = 8;  // elements per step: one 16-byte vector of the narrower type
    uint64_t vend = beg;
    if (aligned16(src + beg) && aligned16(dst + beg)) {
        vend = beg + (end - beg) / G * G;
#pragma unroll 4
        for (uint64_t i = beg + (uint64_t)threadIdx.x * G; i < vend; i += (uint64_t)blockDim.x * G) {
            float f[G];
            if (Vec<TS>::N == G) {
                float t[Vec<TS>::N];
                Vec<TS>::load(src + i, t);
#pragma unroll
                for (int k = 0; k < Vec<TS>::N; k++) f[k] = t[k];
            } else {
#pragma unroll
                for (int h = 0; h < G / Vec<TS>::N; h++) {
                    float t[Vec<TS>::N];
                    Vec<TS>::load(src + i + h * Vec<TS>::N, t);
#pragma unroll
                    for (int k = 0; k < Vec<TS>::N; k++) f[h * Vec<TS>::N + k] = t[k];
                }
            }
            if (scale != 1.f) {
#pragma unroll
                for (int k = 0; k < G; k++) f[k] *= scale;
            }
#pragma unroll
            for (int h = 0; h < G / Vec<TD>::N; h++) {
                float t[Vec<TD>::N];
#pragma unroll
                for (int k = 0; k < Vec<TD>::N; k++) t[k] = f[h * Vec<TD>::N + k];
                Vec<TD>::store(dst + i + h * Vec<TD>::N, t);
            }
        }
    }
    for (uint64_t i = vend + threadIdx.x; i < end; i += blockDim.x) {
        const float v = Vec<TS>::to_f(src[i]);
        dst[i] = Vec<TD>::from_f(scale != 1.f ? v * scale : v);
    }
}

// Raw copy of [beg, end) elements of T (no conversion).
template <typename T> __device__ __forceinline__ void cta_raw_copy(const T *src, T *dst, uint64_t beg, uint64_t end)
{
    constexpr int VN = 16 / sizeof(T);
    uint64_t vend = beg;
    if (aligned16(src + beg) && aligned16(dst + beg)) {
        vend = beg + (end - beg) / VN * VN;
        const uint64_t step = (uint64_t)blockDim.x * VN;
        uint64_t i = beg + (uint64_t)threadIdx.x * VN;
        // four independent 16-byte loads in flight per thread before the first store (NVLink latency)
        for (; i + 3 * step < vend; i += 4 * step) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u] = __ldcg(reinterpret_cast<const uint4 *>(src + i + u * step));
#pragma unroll
            for (int u = 0; u < 4; u++) *reinterpret_cast<uint4 *>(dst + i + u * step) = v[u];
        }
        for (; i < vend; i += step) *reinterpret_cast<uint4 *>(dst + i) = __ldcg(reinterpret_cast<const uint4 *>(src + i));
    }
    for (uint64_t i = vend + threadIdx.x; i < end; i += blockDim.x) dst[i] = src[i];
}

// One source range to several destinations (all-gather, broadcast): every 16-byte vector is loaded ONCE, four
// independent loads in flight per thread, and stored to each destination in turn, so that all peers fill at the same
// time and the source is not re-read per peer. Same element type on both sides, no scaling; falls back to
// element-wise copies when an address is not 16-byte aligned.
template <typename T> __device__ __forceinline__ void cta_fanout_copy(const T *src, T *const *dsts, uint32_t ndst, uint64_t beg, uint64_t end)
{
    constexpr int VN = 16 / sizeof(T);
    bool al = aligned16(src + beg);
    for (uint32_t k = 0; k < ndst; k++) al = al && aligned16(dsts[k] + beg);
    uint64_t vend = beg;
    if (al) {
        vend = beg + (end - beg) / VN * VN;
        const uint64_t step = (uint64_t)blockDim.x * VN;
        uint64_t i = beg + (uint64_t)threadIdx.x * VN;
        for (; i + 3 * step < vend; i += 4 * step) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u] = __ldcs(reinterpret_cast<const uint4 *>(src + i + u * step));
            for (uint32_t k = 0; k < ndst; k++) {
#pragma unroll
                for (int u = 0; u < 4; u++) *reinterpret_cast<uint4 *>(dsts[k] + i + u * step) = v[u];
            }
        }
        for (; i < vend; i += step) {
            const uint4 v = __ldcs(reinterpret_cast<const uint4 *>(src + i));
            for (uint32_t k = 0; k < ndst; k++) *reinterpret_cast<uint4 *>(dsts[k] + i) = v;
        }
    }
    for (uint64_t i = vend + threadIdx.x; i < end; i += blockDim.x) {
        const T v = src[i];
        for (uint32_t k = 0; k < ndst; k++) dsts[k][i] = v;
    }
}

// Reduces element range [beg, end) of staging A across all ranks (offset `base` elements into A) and
// hands each result vector to `sink(i, values, count)`. Loads are issued in an order rotated by the
// rank to spread the traffic over the peers; the accumulation order is fixed (rank 0 first) so that
// every rank computes bit-identical results.
template <typename T, bool INT, int W, typename Sink>
__device__ __forceinline__ void reduce_ranks(const Team &t, uint32_t me, uint64_t stage_a, uint64_t base, uint64_t beg, uint64_t end,
                                             int op, Sink sink)
{
    constexpr int VN = Vec<T>::N;
    const uint32_t world = W > 0 ? (uint32_t)W : t.world;
    uint64_t vend = beg;
    if (((base + beg) * sizeof(T) & 15) == 0 && (stage_a & 15) == 0) {
        vend = beg + (end - beg) / VN * VN;
        for (uint64_t i = beg + (uint64_t)threadIdx.x * VN; i < vend; i += (uint64_t)blockDim.x * VN) {
            float acc[VN];
            if (W > 0) {
                uint4 raw[W > 0 ? W : 1];
#pragma unroll
                for (int k = 0; k < W; k++) {
                    const uint32_t r = (me + k) % W;
                    const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(peer_ptr(t, r, stage_a)) + base + i));
#pragma unroll
                    for (int q = 0; q < W; q++)
                        if (q == (int)r) raw[q] = v;  // static indexing keeps raw[] in registers
                }
#pragma unroll
                for (int r = 0; r < W; r++) {
                    float f[VN];
                    Vec<T>::unpack(raw[r], f);
#pragma unroll
                    for (int k = 0; k < VN; k++) acc[k] = r == 0 ? f[k] : red_apply<INT>(acc[k], f[k], op);
                }
            } else {
                for (uint32_t r = 0; r < world; r++) {
                    float f[VN];
                    Vec<T>::load(reinterpret_cast<const T *>(peer_ptr(t, r, stage_a)) + base + i, f);
#pragma unroll
                    for (int k = 0; k < VN; k++) acc[k] = r == 0 ? f[k] : red_apply<INT>(acc[k], f[k], op);
                }
            }
            sink(i, acc, VN);
        }
    }
    for (uint64_t i = vend + threadIdx.x; i < end; i += blockDim.x) {
        float acc[VN];
        for (uint32_t r = 0; r < world; r++) {
            float f = Vec<T>::to_f(__ldcg(reinterpret_cast<const T *>(peer_ptr(t, r, stage_a)) + base + i));
            acc[0] = r == 0 ? f : red_apply<INT>(acc[0], f, op);
        }
        sink(i, acc, 1);
    }
}

// Epilogue: x scale (floating types), cast to TO, store `cnt` values at dst + i.
template <typename TO, bool INT> __device__ __forceinline__ void emit(TO *dst, uint64_t i, float *acc, int cnt, float scale)
{
    constexpr int VN = Vec<TO>::N;
    if (!INT && scale != 1.f)
        for (int k = 0; k < cnt; k++) acc[k] *= scale;
    if (cnt == VN && aligned16(dst + i)) {
        float g[VN];
#pragma unroll
        for (int k = 0; k < VN; k++) g[k] = acc[k];
        Vec<TO>::store(dst + i, g);
    } else if (sizeof(TO) == 2 && cnt == 4 && (reinterpret_cast<uint64_t>(dst + i) & 7) == 0) {
        // four 16-bit results of a 32-bit input vector: one 8-byte store
        union {
            uint2 u;
            TO h[4];
        } pk;
#pragma unroll
        for (int k = 0; k < 4; k++) pk.h[k] = Vec<TO>::from_f(acc[k]);
        *reinterpret_cast<uint2 *>(dst + i) = pk.u;
    } else {
        for (int k = 0; k < cnt; k++) dst[i + k] = Vec<TO>::from_f(acc[k]);
    }
}

// ------------------------------------------------------------------------------------------------
template <typename T, typename TO, bool INT, int W> __global__ void __launch_bounds__(512) k_allreduce(CollArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const uint32_t world = t.world;
    const T *in = reinterpret_cast<const T *>(a.in + (uint64_t)me * a.in_rank_stride);
    TO *out = reinterpret_cast<TO *>(a.out + (uint64_t)me * a.out_rank_stride);
    T *myA = reinterpret_cast<T *>(peer_ptr(t, me, a.stage_a));
    constexpr int VN = Vec<T>::N;
    if (a.algo == 0) {
        const Range rg = cta_range<8>(a.n);
        if (!a.zero_copy) cta_raw_copy<T>(in, myA, rg.beg, rg.end);
        if (!lane_sync(t, me, 0, a.epoch, 0x100)) return;
        reduce_ranks<T, INT, W>(t, me, a.stage_a, 0, rg.beg, rg.end, a.op,
                                [&](uint64_t i, float *acc, int cnt) { emit<TO, INT>(out, i, acc, cnt, a.scale); });
        return;
    }
    // two-shot: chunk c = elements [c * C, (c + 1) * C) belongs to rank c
    uint64_t C = (a.n + world - 1) / world;
    C = (C + 7) / 8 * 8;
    const Range sub = cta_range<8>(C);
    MF_PROF_START(PF_STAGE_IN);
    if (!a.zero_copy) {
        for (uint32_t c = 0; c < world; c++) {
            const uint64_t b = min(a.n, c * C + sub.beg), e = min(a.n, c * C + sub.end);
            cta_raw_copy<T>(in, myA, b, e);
        }
    }
    MF_PROF_STOP(PF_STAGE_IN);
    MF_PROF_START(PF_SYNC);
    if (!lane_sync(t, me, 0, a.epoch, 0x110)) return;
    MF_PROF_STOP(PF_SYNC);
    MF_PROF_START(PF_REDUCE);
    {
        const uint64_t b = min(a.n, me * C + sub.beg), e = min(a.n, me * C + sub.end);
        reduce_ranks<T, INT, W>(t, me, a.stage_a, 0, b, e, a.op, [&](uint64_t i, float *acc, int cnt) {
            if (!INT && a.scale != 1.f)
                for (int k = 0; k < cnt; k++) acc[k] *= a.scale;
            // push the finished values into every rank's result buffer (own included)
            for (uint32_t k = 0; k < world; k++) {
                const uint32_t r = (me + k) % world;
                TO *dst = reinterpret_cast<TO *>(peer_ptr(t, r, a.stage_b));
                float tmp[VN];
#pragma unroll
                for (int q = 0; q < VN; q++) tmp[q] = acc[q];
                emit<TO, true>(dst, i, tmp, cnt, 1.f);
            }
        });
    }
    MF_PROF_STOP(PF_REDUCE);
    MF_PROF_START(PF_SYNC);
    if (!lane_sync(t, me, 1, a.epoch, 0x111)) return;
    MF_PROF_STOP(PF_SYNC);
    MF_PROF_START(PF_COPY_OUT);
    const TO *myB = reinterpret_cast<const TO *>(peer_ptr(t, me, a.stage_b));
    for (uint32_t c = 0; c < world; c++) {
        const uint64_t b = min(a.n, c * C + sub.beg), e = min(a.n, c * C + sub.end);
        cta_raw_copy<TO>(myB, out, b, e);
    }
    MF_PROF_STOP(PF_COPY_OUT);
}

// reduce_scatter: input n = W * m elements, output m elements (rank r gets the reduction of chunk r)
template <typename T, typename TO, bool INT, int W> __global__ void __launch_bounds__(512) k_reduce_scatter(CollArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const uint32_t world = t.world;
    const T *in = reinterpret_cast<const T *>(a.in + (uint64_t)me * a.in_rank_stride);
    TO *out = reinterpret_cast<TO *>(a.out + (uint64_t)me * a.out_rank_stride);
    T *myA = reinterpret_cast<T *>(peer_ptr(t, me, a.stage_a));
    constexpr int VN = Vec<T>::N;
    const uint64_t m = a.n / world;
    const Range sub = cta_range<8>(m);
    const uint64_t ps = a.part_stride ? a.part_stride : m;
    if (!a.zero_copy)
        for (uint32_t c = 0; c < world; c++) cta_raw_copy<T>(in + c * ps, myA + c * m, sub.beg, sub.end);
    if (!lane_sync(t, me, 0, a.epoch, 0x120)) return;
    reduce_ranks<T, INT, W>(t, me, a.stage_a, (uint64_t)me * m, sub.beg, sub.end, a.op,
                            [&](uint64_t i, float *acc, int cnt) { emit<TO, INT>(out, i, acc, cnt, a.scale); });
}

// allgather: every rank contributes n elements; output W * n. Shards are pushed (one NVLink crossing).
template <typename T, typename TO> __global__ void __launch_bounds__(512) k_allgather(CollArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const uint32_t world = t.world;
    const T *in = reinterpret_cast<const T *>(a.in + (uint64_t)me * a.in_rank_stride);
    TO *out = reinterpret_cast<TO *>(a.out + (uint64_t)me * a.out_rank_stride);
    constexpr int VN = Vec<T>::N;
    const Range sub = cta_range<8>(a.n);
    for (uint32_t k = 0; k < world; k++) {
        const uint32_t r = (me + k) % world;
        TO *dst = reinterpret_cast<TO *>(peer_ptr(t, r, a.stage_b)) + (uint64_t)me * a.n;
        cta_convert_copy<T, TO>(in, dst, sub.beg, sub.end, a.scale);
    }
    if (!lane_sync(t, me, 0, a.epoch, 0x130)) return;
    const TO *myB = reinterpret_cast<const TO *>(peer_ptr(t, me, a.stage_b));
    const uint64_t ps = a.part_stride ? a.part_stride : a.n;
    for (uint32_t c = 0; c < world; c++) cta_raw_copy<TO>(myB + (uint64_t)c * a.n, out + (uint64_t)c * ps, sub.beg, sub.end);
}

// broadcast of n elements from a.root
template <typename T> __global__ void __launch_bounds__(512) k_broadcast(CollArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const uint32_t world = t.world;
    const T *in = reinterpret_cast<const T *>(a.in + (uint64_t)me * a.in_rank_stride);
    T *out = reinterpret_cast<T *>(a.out + (uint64_t)me * a.out_rank_stride);
    const Range sub = cta_range<8>(a.n);
    if (me == a.root) {
        for (uint32_t k = 0; k < world; k++) {
            const uint32_t r = (me + k) % world;
            // scatter mode: member r gets part r of the root's buffer
            const T *src = a.algo == 1 ? in + (uint64_t)r * (a.part_stride ? a.part_stride : a.n) : in;
            cta_raw_copy<T>(src, reinterpret_cast<T *>(peer_ptr(t, r, a.stage_b)), sub.beg, sub.end);
        }
    }
    if (!lane_sync(t, me, 0, a.epoch, 0x140)) return;
    cta_raw_copy<T>(reinterpret_cast<const T *>(peer_ptr(t, me, a.stage_b)), out, sub.beg, sub.end);
}

// ------------------------------------------------------------------------------------------------
// Direct ("zero-copy") variants for buffers that live inside the ranks' own slices of the symmetric
// heap (tensors from the symmetric allocator): no staging copy on either side. The ranks swap the slot
// offsets of their buffers in the opening handshake, so the buffers need not sit at the same offset on
// every rank. A closing handshake keeps every input intact until all peers have read it and tells each
// rank that the peers' stores into its output have landed.
template <typename T, bool INT, int W, typename Sink>
__device__ __forceinline__ void reduce_direct(const Team &t, uint32_t me, const uint64_t *src_off, uint64_t base, uint64_t beg, uint64_t end,
                                              int op, Sink sink)
{
    constexpr int VN = Vec<T>::N;
    const uint32_t world = W > 0 ? (uint32_t)W : t.world;
    bool vec_ok = true;
    for (uint32_t r = 0; r < world; r++) vec_ok = vec_ok && (((src_off[r] + (base + beg) * sizeof(T)) & 15) == 0);
    uint64_t vend = beg;
    if (vec_ok) {
        vend = beg + (end - beg) / VN * VN;
        for (uint64_t i = beg + (uint64_t)threadIdx.x * VN; i < vend; i += (uint64_t)blockDim.x * VN) {
            float acc[VN];
            if (W > 0) {
                uint4 raw[W > 0 ? W : 1];
#pragma unroll
                for (int k = 0; k < W; k++) {
                    const uint32_t r = (me + k) % W;
                    const uint4 v = __ldcg(reinterpret_cast<const uint4 *>(reinterpret_cast<const T *>(peer_ptr(t, r, src_off[r])) + base + i));
#pragma unroll
                    for (int q = 0; q < W; q++)
                        if (q == (int)r) raw[q] = v;
                }
#pragma unroll
                for (int r = 0; r < W; r++) {
                    float f[VN];
                    Vec<T>::unpack(raw[r], f);
#pragma unroll
                    for (int k = 0; k < VN; k++) acc[k] = r == 0 ? f[k] : red_apply<INT>(acc[k], f[k], op);
                }
            } else {
                for (uint32_t r = 0; r < world; r++) {
                    float f[VN];
                    Vec<T>::load(reinterpret_cast<const T *>(peer_ptr(t, r, src_off[r])) + base + i, f);
#pragma unroll
                    for (int k = 0; k < VN; k++) acc[k] = r == 0 ? f[k] : red_apply<INT>(acc[k], f[k], op);
                }
            }
            sink(i, acc, VN);
        }
    }
    for (uint64_t i = vend + threadIdx.x; i < end; i += blockDim.x) {
        float acc[VN];
        for (uint32_t r = 0; r < world; r++) {
            float f = Vec<T>::to_f(__ldcg(reinterpret_cast<const T *>(peer_ptr(t, r, src_off[r])) + base + i));
            acc[0] = r == 0 ? f : red_apply<INT>(acc[0], f, op);
        }
        sink(i, acc, 1);
    }
}

// all-reduce: rank r reduces chunk r straight from every rank's input and stores the result straight
// into every rank's output. In place (out == in) is fine: chunk r is read and written by rank r only.
template <typename T, typename TO, bool INT, int W>
__device__ __forceinline__ void allreduce_direct_body(const CollArgs &a, const Team &t, uint32_t me, const uint64_t *p_in, const uint64_t *p_out)
{
    const uint32_t world = t.world;
    constexpr int VN = Vec<T>::N;
    uint64_t C = (a.n + world - 1) / world;
    C = (C + 7) / 8 * 8;
    const Range sub = cta_range<8>(C);
    const uint64_t b = min(a.n, me * C + sub.beg), e = min(a.n, me * C + sub.end);
    reduce_direct<T, INT, W>(t, me, p_in, 0, b, e, a.op, [&](uint64_t i, float *acc, int cnt) {
        if (!INT && a.scale != 1.f)
            for (int k = 0; k < cnt; k++) acc[k] *= a.scale;
        for (uint32_t k = 0; k < world; k++) {
            const uint32_t r = (me + k) % world;
            TO *dst = reinterpret_cast<TO *>(peer_ptr(t, r, p_out[r]));
            float tmp[VN];
#pragma unroll
            for (int q = 0; q < VN; q++) tmp[q] = acc[q];
            emit<TO, true>(dst, i, tmp, cnt, 1.f);
        }
    });
}

template <typename T, typename TO, bool INT, int W> __global__ void __launch_bounds__(512) k_allreduce_zc(CollArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    __shared__ uint64_t p_in[kMaxRanks], p_out[kMaxRanks];
    const uint64_t slot = t.heap_base + (uint64_t)me * t.stride;
    MF_PROF_START(PF_SYNC);
    if (!lane_sync_xchg(t, me, 0, a.epoch, 0x180, a.in - slot, a.out - slot, p_in, p_out)) return;
    MF_PROF_STOP(PF_SYNC);
    MF_PROF_START(PF_REDUCE);
    allreduce_direct_body<T, TO, INT, W>(a, t, me, p_in, p_out);
    MF_PROF_STOP(PF_REDUCE);
    MF_PROF_START(PF_SYNC);
    lane_sync(t, me, 1, a.epoch, 0x181);
    MF_PROF_STOP(PF_SYNC);
}

// NVLink multicast ("NVLS") all-reduce (sum of bf16 / fp16 / fp32): rank r reduces chunk r with ONE
// multimem.ld_reduce per 16 bytes (the switch adds the values of all ranks, fp32 accumulation) and writes the
// result into every rank's output with ONE multimem.st. Per GPU that is n bytes on the wire in each direction
// instead of 1.75 n with peer loads and stores (8 ranks). Needs team.mc_base (the multicast alias of the
// team's slot) and input / output at the SAME slot offset on every rank, 16-byte aligned; the ranks swap
// their offsets first and fall back to peer loads and stores, all together, when they differ.
template <typename T> struct MultiMem;
template <> struct MultiMem<__nv_bfloat16> {
    __device__ static uint4 ld_add(uint64_t p)
    {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
        return v;
    }
    __device__ static void st(uint64_t p, const uint4 &v)
    {
        asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    }
};
template <> struct MultiMem<__half> {
    __device__ static uint4 ld_add(uint64_t p)
    {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
        return v;
    }
    __device__ static void st(uint64_t p, const uint4 &v)
    {
        asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
    }
};
template <> struct MultiMem<float> {
    __device__ static uint4 ld_add(uint64_t p)
    {
        float4 f;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(f.x), "=f"(f.y), "=f"(f.z), "=f"(f.w) : "l"(p) : "memory");
        return make_uint4(__float_as_uint(f.x), __float_as_uint(f.y), __float_as_uint(f.z), __float_as_uint(f.w));
    }
    __device__ static void st(uint64_t p, const uint4 &v)
    {
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)),
                     "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
    }
};

template <typename T, int W> __global__ void __launch_bounds__(512) k_allreduce_mc(CollArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const uint32_t world = t.world;
    __shared__ uint64_t p_in[kMaxRanks], p_out[kMaxRanks];
    const uint64_t slot = t.heap_base + (uint64_t)me * t.stride;
    MF_PROF_START(PF_SYNC);
    if (!lane_sync_xchg(t, me, 0, a.epoch, 0x188, a.in - slot, a.out - slot, p_in, p_out)) return;
    MF_PROF_STOP(PF_SYNC);
    constexpr int VN = Vec<T>::N;
    // every rank sees the same table, so every rank takes the same branch
    bool same = t.mc_base != 0 && a.op == OP_SUM && (a.n % VN) == 0 && ((p_in[0] | p_out[0]) & 15) == 0;
    for (uint32_t r = 1; r < world; r++) same = same && p_in[r] == p_in[0] && p_out[r] == p_out[0];
    MF_PROF_START(PF_REDUCE);
    if (same) {
        uint64_t C = (a.n + world - 1) / world;
        C = (C + 7) / 8 * 8;
        const Range sub = cta_range<8>(C);
        const uint64_t b = min(a.n, me * C + sub.beg), e = min(a.n, me * C + sub.end);
        const uint64_t src = t.mc_base + p_in[0], dst = t.mc_base + p_out[0];
        const uint64_t step = (uint64_t)blockDim.x * VN;
        uint64_t i = b + (uint64_t)threadIdx.x * VN;
        // four independent load-reduces in flight per thread: a multimem load is a round trip through the switch
        auto scaled = [&](uint4 &v) {
            if (a.scale != 1.f) {
                float f[VN];
                Vec<T>::unpack(v, f);
#pragma unroll
                for (int k = 0; k < VN; k++) f[k] *= a.scale;
                Vec<T>::store(reinterpret_cast<T *>(&v), f);
            }
        };
        for (; i + 3 * step < e; i += 4 * step) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u] = MultiMem<T>::ld_add(src + (i + u * step) * sizeof(T));
#pragma unroll
            for (int u = 0; u < 4; u++) {
                scaled(v[u]);
                MultiMem<T>::st(dst + (i + u * step) * sizeof(T), v[u]);
            }
        }
        for (; i < e; i += step) {
            uint4 v0 = MultiMem<T>::ld_add(src + i * sizeof(T));
            if (a.scale != 1.f) {
                float f[VN];
                Vec<T>::unpack(v0, f);
#pragma unroll
                for (int k = 0; k < VN; k++) f[k] *= a.scale;
                Vec<T>::store(reinterpret_cast<T *>(&v0), f);
            }
            MultiMem<T>::st(dst + i * sizeof(T), v0);
        }
    } else {
        allreduce_direct_body<T, T, false, W>(a, t, me, p_in, p_out);
    }
    MF_PROF_STOP(PF_REDUCE);
    MF_PROF_START(PF_SYNC);
    lane_sync(t, me, 1, a.epoch, 0x189);
    MF_PROF_STOP(PF_SYNC);
}

// reduce-scatter: rank r reduces part r of every rank's input into its local output.
template <typename T, typename TO, bool INT, int W> __global__ void __launch_bounds__(512) k_reduce_scatter_zc(CollArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    __shared__ uint64_t p_in[kMaxRanks], p_unused[kMaxRanks];
    const uint64_t slot = t.heap_base + (uint64_t)me * t.stride;
    if (!lane_sync_xchg(t, me, 0, a.epoch, 0x182, a.in - slot, 0, p_in, p_unused)) return;
    TO *out = reinterpret_cast<TO *>(a.out);
    const uint64_t m = a.n / t.world;
    const uint64_t ps = a.part_stride ? a.part_stride : m;
    const Range sub = cta_range<8>(m);
    reduce_direct<T, INT, W>(t, me, p_in, (uint64_t)me * ps, sub.beg, sub.end, a.op,
                             [&](uint64_t i, float *acc, int cnt) { emit<TO, INT>(out, i, acc, cnt, a.scale); });
    lane_sync(t, me, 1, a.epoch, 0x183);
}

// reduce-scatter through the multicast alias: rank r pulls part r with ONE multimem.ld_reduce per 16 bytes (the
// switch adds all ranks' values), so each GPU receives n/W bytes instead of (W-1) n/W. Needs the input at the
// same slot offset on every rank and 16-byte aligned parts; otherwise, all together, the ranks fall back to
// peer loads.
template <typename T, typename TO, int W> __global__ void __launch_bounds__(512) k_reduce_scatter_mc(CollArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const uint32_t world = t.world;
    __shared__ uint64_t p_in[kMaxRanks], p_unused[kMaxRanks];
    const uint64_t slot = t.heap_base + (uint64_t)me * t.stride;
    if (!lane_sync_xchg(t, me, 0, a.epoch, 0x18e, a.in - slot, 0, p_in, p_unused)) return;
    TO *out = reinterpret_cast<TO *>(a.out);
    const uint64_t m = a.n / world;
    const uint64_t ps = a.part_stride ? a.part_stride : m;
    constexpr int VN = Vec<T>::N;
    bool same = t.mc_base != 0 && a.op == OP_SUM && (m % VN) == 0 && (ps % VN) == 0 && (p_in[0] & 15) == 0;
    for (uint32_t r = 1; r < world; r++) same = same && p_in[r] == p_in[0];
    const Range sub = cta_range<8>(m);
    if (same) {
        const uint64_t src = t.mc_base + p_in[0] + (uint64_t)me * ps * sizeof(T);
        const uint64_t step = (uint64_t)blockDim.x * VN;
        uint64_t i = sub.beg + (uint64_t)threadIdx.x * VN;
        for (; i + 3 * step < sub.end; i += 4 * step) {
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u] = MultiMem<T>::ld_add(src + (i + u * step) * sizeof(T));
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float f[VN];
                Vec<T>::unpack(v[u], f);
                emit<TO, false>(out, i + u * step, f, VN, a.scale);
            }
        }
        for (; i < sub.end; i += step) {
            uint4 v0 = MultiMem<T>::ld_add(src + i * sizeof(T));
            float f[VN];
            Vec<T>::unpack(v0, f);
            emit<TO, false>(out, i, f, VN, a.scale);
        }
    } else {
        reduce_direct<T, false, W>(t, me, p_in, (uint64_t)me * ps, sub.beg, sub.end, a.op,
                                   [&](uint64_t i, float *acc, int cnt) { emit<TO, false>(out, i, acc, cnt, a.scale); });
    }
    lane_sync(t, me, 1, a.epoch, 0x18f);
}

// all-gather: every rank stores its shard straight into every rank's output.
template <typename T, typename TO> __global__ void __launch_bounds__(512) k_allgather_zc(CollArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const uint32_t world = t.world;
    __shared__ uint64_t p_out[kMaxRanks], p_unused[kMaxRanks];
    const uint64_t slot = t.heap_base + (uint64_t)me * t.stride;
    if (!lane_sync_xchg(t, me, 0, a.epoch, 0x184, a.out - slot, 0, p_out, p_unused)) return;
    const T *in = reinterpret_cast<const T *>(a.in);
    const uint64_t ps = a.part_stride ? a.part_stride : a.n;
    const Range sub = cta_range<8>(a.n);
    if (sizeof(T) == sizeof(TO) && a.scale == 1.f) {
        // same type, no scaling: the shard is read once and fanned out to every rank's output
        __shared__ TO *dsts[kMaxRanks];
        if (threadIdx.x < world) {
            const uint32_t r = (me + threadIdx.x) % world;
            dsts[threadIdx.x] = reinterpret_cast<TO *>(peer_ptr(t, r, p_out[r])) + (uint64_t)me * ps;
        }
        __syncthreads();
        cta_fanout_copy<TO>(reinterpret_cast<const TO *>(in), dsts, world, sub.beg, sub.end);
    } else {
        for (uint32_t k = 0; k < world; k++) {
            const uint32_t r = (me + k) % world;
            TO *dst = reinterpret_cast<TO *>(peer_ptr(t, r, p_out[r])) + (uint64_t)me * ps;
            cta_convert_copy<T, TO>(in, dst, sub.beg, sub.end, a.scale);
        }
    }
    lane_sync(t, me, 1, a.epoch, 0x185);
}

// rooted copy: the root stores straight into every rank's output (scatter mode: part r to rank r).
template <typename T> __global__ void __launch_bounds__(512) k_broadcast_zc(CollArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const uint32_t world = t.world;
    __shared__ uint64_t p_out[kMaxRanks], p_unused[kMaxRanks];
    const uint64_t slot = t.heap_base + (uint64_t)me * t.stride;
    if (!lane_sync_xchg(t, me, 0, a.epoch, 0x186, a.out - slot, 0, p_out, p_unused)) return;
    if (me == a.root) {
        const T *in = reinterpret_cast<const T *>(a.in);
        const Range sub = cta_range<8>(a.n);
        for (uint32_t k = 0; k < world; k++) {
            const uint32_t r = (me + k) % world;
            const T *src = a.algo == 1 ? in + (uint64_t)r * (a.part_stride ? a.part_stride : a.n) : in;
            T *dst = reinterpret_cast<T *>(peer_ptr(t, r, p_out[r]));
            if (src != dst) cta_raw_copy<T>(src, dst, sub.beg, sub.end);
        }
    }
    lane_sync(t, me, 1, a.epoch, 0x187);
}

// Raw 16-byte multimem store (any element type: the bits travel unchanged).
__device__ __forceinline__ void multimem_st16(uint64_t p, const uint4 &v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)),
                 "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w)) : "memory");
}

// all-gather through the multicast alias: every rank writes its shard ONCE and the switch delivers it to all
// ranks' outputs (send traffic n per rank instead of (W-1) n). Needs the output at the same slot offset on every
// rank; otherwise, all together, the ranks fall back to one peer store per destination.
template <typename T, typename TO> __global__ void __launch_bounds__(512) k_allgather_mc(CollArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const uint32_t world = t.world;
    __shared__ uint64_t p_out[kMaxRanks], p_unused[kMaxRanks];
    const uint64_t slot = t.heap_base + (uint64_t)me * t.stride;
    if (!lane_sync_xchg(t, me, 0, a.epoch, 0x18a, a.out - slot, 0, p_out, p_unused)) return;
    const T *in = reinterpret_cast<const T *>(a.in);
    const uint64_t ps = a.part_stride ? a.part_stride : a.n;
    constexpr int G = 16 / sizeof(TO);  // output elements per 16-byte store
    bool same = t.mc_base != 0 && (a.n % G) == 0 && (ps % G) == 0 && (p_out[0] & 15) == 0 && (reinterpret_cast<uint64_t>(in) & 15) == 0;
    for (uint32_t r = 1; r < world; r++) same = same && p_out[r] == p_out[0];
    const Range sub = cta_range<8>(a.n);
    if (same) {
        const uint64_t dst = t.mc_base + p_out[0] + (uint64_t)me * ps * sizeof(TO);
        for (uint64_t i = sub.beg + (uint64_t)threadIdx.x * G; i < sub.end; i += (uint64_t)blockDim.x * G) {
            float f[G];
#pragma unroll
            for (int h = 0; h < G / Vec<T>::N; h++) {
                float tmp[Vec<T>::N];
                Vec<T>::load(in + i + h * Vec<T>::N, tmp);
#pragma unroll
                for (int k = 0; k < Vec<T>::N; k++) f[h * Vec<T>::N + k] = a.scale != 1.f ? tmp[k] * a.scale : tmp[k];
            }
            uint4 v;
            {
                float g[Vec<TO>::N];
#pragma unroll
                for (int k = 0; k < Vec<TO>::N; k++) g[k] = f[k];
                Vec<TO>::store(reinterpret_cast<TO *>(&v), g);
            }
            multimem_st16(dst + i * sizeof(TO), v);
        }
    } else {
        for (uint32_t k = 0; k < world; k++) {
            const uint32_t r = (me + k) % world;
            TO *dst = reinterpret_cast<TO *>(peer_ptr(t, r, p_out[r])) + (uint64_t)me * ps;
            cta_convert_copy<T, TO>(in, dst, sub.beg, sub.end, a.scale);
        }
    }
    lane_sync(t, me, 1, a.epoch, 0x18b);
}

// rooted copy through the multicast alias: the root writes once, the switch fans out.
template <typename T> __global__ void __launch_bounds__(512) k_broadcast_mc(CollArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const uint32_t world = t.world;
    __shared__ uint64_t p_out[kMaxRanks], p_unused[kMaxRanks];
    const uint64_t slot = t.heap_base + (uint64_t)me * t.stride;
    if (!lane_sync_xchg(t, me, 0, a.epoch, 0x18c, a.out - slot, 0, p_out, p_unused)) return;
    constexpr int G = 16 / sizeof(T);
    const T *in = reinterpret_cast<const T *>(a.in);
    bool same = t.mc_base != 0 && a.algo == 0 && (a.n % G) == 0 && (p_out[0] & 15) == 0;
    for (uint32_t r = 1; r < world; r++) same = same && p_out[r] == p_out[0];
    if (me == a.root) {
        const Range sub = cta_range<8>(a.n);
        if (same && (reinterpret_cast<uint64_t>(in) & 15) == 0) {
            const uint64_t dst = t.mc_base + p_out[0];
            const uint64_t step = (uint64_t)blockDim.x * G;
            uint64_t i = sub.beg + (uint64_t)threadIdx.x * G;
            for (; i + 3 * step < sub.end; i += 4 * step) {
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; u++) v[u] = __ldcg(reinterpret_cast<const uint4 *>(in + i + u * step));
#pragma unroll
                for (int u = 0; u < 4; u++) multimem_st16(dst + (i + u * step) * sizeof(T), v[u]);
            }
            for (; i < sub.end; i += step) multimem_st16(dst + i * sizeof(T), __ldcg(reinterpret_cast<const uint4 *>(in + i)));
        } else {
            for (uint32_t k = 0; k < world; k++) {
                const uint32_t r = (me + k) % world;
                const T *src = a.algo == 1 ? in + (uint64_t)r * (a.part_stride ? a.part_stride : a.n) : in;
                T *dst = reinterpret_cast<T *>(peer_ptr(t, r, p_out[r]));
                if (src != dst) cta_raw_copy<T>(src, dst, sub.beg, sub.end);
            }
        }
    }
    lane_sync(t, me, 1, a.epoch, 0x18d);
}

// all-to-all-v (bytes). Each rank stages its whole send buffer plus its (offset, count) table; after the
// handshake every rank pulls its pieces from the peers' staging.
//   table in staging A header: W x {u64 send_off, u64 send_cnt} toward each destination, bytes
struct A2AArgs {
    Team team;
    uint64_t in, out, in_rank_stride, out_rank_stride;
    uint64_t meta;       // device array [W][4] u64 per emulated rank: send_off, send_cnt, recv_off, recv_cnt (bytes)
    uint64_t meta_rank_stride;
    uint64_t in_bytes;   // total bytes of the send buffer
    uint64_t stage_a;
    uint32_t epoch;
};
constexpr uint64_t kA2AHeader = 4096;

// Push model: (1) every receiver tells every sender where in the RECEIVER's staging area its piece goes and how many bytes
// it expects (two 8-byte words per pair, written into the sender's header); (2) a rank stores its piece for rank me + k,
// k = 1 .. W - 1, straight into that rank's staging area over NVLink; (3) it then copies the pieces that arrived in its own
// staging area to `out`. CTA b of the sender and CTA b of the receiver work on the same byte range of a piece, so with two
// ranks one flag per lane and sender is all the ordering the copy needs; with more ranks one handshake follows all pushes
// (see per_piece below). The piece for the rank itself goes from `in` to `out` directly. The data crosses memory once on the
// sending side (no local staging copy), once over NVLink, once more locally on the receiving side.
__global__ void __launch_bounds__(512) k_alltoallv(A2AArgs a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const uint32_t world = t.world;
    const uint8_t *in = reinterpret_cast<const uint8_t *>(a.in + (uint64_t)me * a.in_rank_stride);
    uint8_t *out = reinterpret_cast<uint8_t *>(a.out + (uint64_t)me * a.out_rank_stride);
    const uint64_t *meta = reinterpret_cast<const uint64_t *>(a.meta + (uint64_t)me * a.meta_rank_stride);
    uint8_t *myA = peer_ptr(t, me, a.stage_a);
    cooperative_groups::grid_group grid = cooperative_groups::this_grid();
    __shared__ int arrived_sh;
    // (1) header of sender p, slot `me`: {offset of p's piece in my staging area, bytes I expect from p}
    if (blockIdx.x == 0 && threadIdx.x < world) {
        const uint32_t p = threadIdx.x;
        uint64_t *hdr = reinterpret_cast<uint64_t *>(peer_ptr(t, p, a.stage_a));
        hdr[2 * me] = meta[4 * p + 2];
        hdr[2 * me + 1] = meta[4 * p + 3];
    }
    // Lane 0's handshake carries the header stores (its CTA wrote them); the grid-wide sync of this cooperative launch hands
    // what lane 0 acquired to the other CTAs. A lane that timed out still joins the grid sync (leaving would hang the others).
    const bool ok = lane_sync(t, me, 0, a.epoch, 0x150);
    grid.sync();
    if (!ok) return;
    const uint64_t *hdr = reinterpret_cast<const uint64_t *>(myA);
    const uint64_t flag_off = kLaneOff + (((uint64_t)1 * kMaxCtas + blockIdx.x) * kMaxRanks) * sizeof(uint32_t);  // phase 1 flags of this lane
    // How the receiver learns that a piece is complete. Two ranks: one flag per piece (measured 43 / 170 us for 16 / 128 MiB
    // against 45 / 178 us). More ranks: every release has to wait until the CTA's earlier stores are performed at the
    // peer, and one such drain per piece cost more than it saved (8 GPUs: 94 / 280 us against 66 / 272 us), so there the
    // pieces are all pushed first and ONE handshake per lane plus a grid-wide sync follows.
    const bool per_piece = world <= 2;
    // (2) all pieces leave first, nearest rank last (rank me + 1 copies my piece first: see the order of (3)). The byte range
    // of this CTA is cut from the RECEIVER's count, so that the receiver's CTA of the same index finds exactly its range
    // complete when the flag is up.
    for (uint32_t k = 0; k < world; k++) {
        const uint32_t r = (me + k) % world;
        const uint64_t soff = meta[4 * r], scnt = meta[4 * r + 1];
        const uint64_t roff = __ldcg(hdr + 2 * r), rcnt = __ldcg(hdr + 2 * r + 1);
        const Range pr = cta_range<16>(rcnt);
        const uint64_t end = min(pr.end, min(scnt, rcnt));
        uint8_t *dst = r == me ? out + roff : peer_ptr(t, r, a.stage_a) + kA2AHeader + roff;
        if (pr.beg < end) cta_raw_copy<uint8_t>(in + soff, dst, pr.beg, end);
        if (k == 0 || !per_piece) continue;
        __syncthreads();  // every thread's stores of the piece are ordered before the signalling thread's release
        if (threadIdx.x == 0) st_release_sys(reinterpret_cast<uint32_t *>(peer_ptr(t, r, flag_off)) + me, a.epoch);
    }
    if (!per_piece) {
        // Lane b passing this handshake means lane b of every peer finished pushing; the grid sync extends that to all lanes
        // (a lane that timed out still joins it).
        const bool landed = lane_sync(t, me, 1, a.epoch, 0x151);
        grid.sync();
        if (!landed) return;
    }
    // (3) the pieces pushed to me, in the order in which their senders sent them: rank me - 1 pushed to me first
    for (uint32_t k = 1; k < world; k++) {
        const uint32_t p = (me + world - k) % world;
        if (threadIdx.x == 0) {
            arrived_sh = 1;
            if (per_piece) {
                const uint32_t *f = reinterpret_cast<const uint32_t *>(peer_ptr(t, me, flag_off)) + p;
                arrived_sh = wait_flag(f, a.epoch, t.spin_limit) ? 1 : 0;
                if (!arrived_sh) report_timeout(t, me, 0x151, a.epoch);
            }
        }
        __syncthreads();
        if (arrived_sh) {
            const uint64_t poff = meta[4 * p + 2], pcnt = meta[4 * p + 3];
            const Range cr = cta_range<16>(pcnt);
            cta_raw_copy<uint8_t>(myA + kA2AHeader + poff, out + poff, cr.beg, cr.end);
        }
        __syncthreads();  // arrived_sh is rewritten in the next step
    }
}

// Point-to-point: the sender writes into the receiver's slot and raises a channel flag; the receiver
// waits, copies out and acknowledges, which frees the landing area for the next message of that pair.
struct P2PArgs {
    Team team;
    uint64_t buf;       // local send or receive buffer
    uint64_t bytes;
    uint64_t stage_off; // landing area in the RECEIVER's slot
    uint32_t peer;
    uint32_t epoch;     // per-pair message number, starts at 1
    uint32_t channel;   // flag channel of this ordered pair
};

__global__ void __launch_bounds__(512) k_send(P2PArgs a)
{
    const Team &t = a.team;
    const uint32_t me = t.rank;
    __shared__ int ok;
    cooperative_groups::grid_group grid = cooperative_groups::this_grid();
    // CTA 0 waits until the receiver consumed the previous message of this pair (ack flag in OUR slot)
    // and publishes the verdict through the slot so that every CTA takes the same branch.
    uint32_t *verdict = reinterpret_cast<uint32_t *>(peer_ptr(t, me, kBarrierOff + (uint64_t)a.channel * 256)) + 16;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        int good = 1;
        if (a.epoch > 1) {
            const uint32_t *ack = reinterpret_cast<const uint32_t *>(peer_ptr(t, me, kBarrierOff + (uint64_t)a.channel * 256)) + 32 + a.peer;  // one ack word per receiver
            if (!wait_flag(ack, a.epoch - 1, t.spin_limit)) {
                good = 0;
                report_timeout(t, me, 0x160, a.epoch);
            }
        }
        *verdict = good;
        __threadfence();
    }
    grid.sync();
    if (threadIdx.x == 0) ok = (int)__ldcg(verdict);
    __syncthreads();
    if (ok) {
        const Range sub = cta_range<16>(a.bytes);
        cta_raw_copy<uint8_t>(reinterpret_cast<const uint8_t *>(a.buf), peer_ptr(t, a.peer, a.stage_off), sub.beg, sub.end);
        __threadfence_system();
    }
    grid.sync();
    if (ok && blockIdx.x == 0 && threadIdx.x == 0)
        st_release_sys(reinterpret_cast<uint32_t *>(peer_ptr(t, a.peer, kBarrierOff + (uint64_t)a.channel * 256)), a.epoch);
}

__global__ void __launch_bounds__(512) k_recv(P2PArgs a)
{
    const Team &t = a.team;
    const uint32_t me = t.rank;
    __shared__ int ok;
    cooperative_groups::grid_group grid = cooperative_groups::this_grid();
    uint32_t *verdict = reinterpret_cast<uint32_t *>(peer_ptr(t, me, kBarrierOff + (uint64_t)a.channel * 256)) + 17;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        const uint32_t *flag = reinterpret_cast<const uint32_t *>(peer_ptr(t, me, kBarrierOff + (uint64_t)a.channel * 256));
        int good = wait_flag(flag, a.epoch, t.spin_limit) ? 1 : 0;
        if (!good) report_timeout(t, me, 0x161, a.epoch);
        *verdict = good;
        __threadfence();
    }
    grid.sync();
    if (threadIdx.x == 0) ok = (int)__ldcg(verdict);
    __syncthreads();
    if (ok) {
        const Range sub = cta_range<16>(a.bytes);
        cta_raw_copy<uint8_t>(peer_ptr(t, me, a.stage_off), reinterpret_cast<uint8_t *>(a.buf), sub.beg, sub.end);
    }
    grid.sync();
    if (ok && blockIdx.x == 0 && threadIdx.x == 0)
        st_release_sys(reinterpret_cast<uint32_t *>(peer_ptr(t, a.peer, kBarrierOff + (uint64_t)a.channel * 256)) + 32 + me, a.epoch);
}

__global__ void k_barrier(Team t, uint32_t channel, uint32_t epoch)
{
    team_barrier(t, team_rank(t), channel, epoch);
}

// Waits on a flag of the caller's own slot that the caller names; used to show that a wait which
// nothing satisfies ends with a status, not a hang.
__global__ void k_wait_flag(Team t, uint64_t flag_off, uint32_t epoch)
{
    const uint32_t me = team_rank(t);
    if (threadIdx.x == 0 && !wait_flag(reinterpret_cast<const uint32_t *>(peer_ptr(t, me, flag_off)), epoch, t.spin_limit))
        report_timeout(t, me, 0x1ff, epoch);
}

}  // namespace mfk

// ------------------------------------------------------------------------------------------------
using namespace mfk;

namespace {
template <typename K, typename A> int launch(K kernel, const A &args, int ctas, int threads, cudaStream_t s, bool coop)
{
    dim3 grid((unsigned)ctas, args.team.emu ? args.team.world : 1);
    if (coop || args.team.emu) {
        void *params[] = {const_cast<A *>(&args)};
        cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(kernel), grid, dim3(threads), params, 0, s);
        return e == cudaSuccess ? 0 : (int)e;
    }
    kernel<<<grid, threads, 0, s>>>(args);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

template <typename T, typename TO, bool INT> int launch_allreduce(const CollArgs &a, int ctas, int threads, cudaStream_t s)
{
    switch (a.team.world) {
        case 2: return launch(k_allreduce<T, TO, INT, 2>, a, ctas, threads, s, false);
        case 4: return launch(k_allreduce<T, TO, INT, 4>, a, ctas, threads, s, false);
        case 8: return launch(k_allreduce<T, TO, INT, 8>, a, ctas, threads, s, false);
        default: return launch(k_allreduce<T, TO, INT, 0>, a, ctas, threads, s, false);
    }
}
template <typename T, typename TO, bool INT> int launch_allreduce_zc(const CollArgs &a, int ctas, int threads, cudaStream_t s)
{
    switch (a.team.world) {
        case 2: return launch(k_allreduce_zc<T, TO, INT, 2>, a, ctas, threads, s, false);
        case 4: return launch(k_allreduce_zc<T, TO, INT, 4>, a, ctas, threads, s, false);
        case 8: return launch(k_allreduce_zc<T, TO, INT, 8>, a, ctas, threads, s, false);
        default: return launch(k_allreduce_zc<T, TO, INT, 0>, a, ctas, threads, s, false);
    }
}
template <typename T> int launch_allreduce_mc(const CollArgs &a, int ctas, int threads, cudaStream_t s)
{
    switch (a.team.world) {
        case 2: return launch(k_allreduce_mc<T, 2>, a, ctas, threads, s, false);
        case 4: return launch(k_allreduce_mc<T, 4>, a, ctas, threads, s, false);
        case 8: return launch(k_allreduce_mc<T, 8>, a, ctas, threads, s, false);
        default: return launch(k_allreduce_mc<T, 0>, a, ctas, threads, s, false);
    }
}
template <typename T, typename TO, bool INT> int launch_rs_zc(const CollArgs &a, int ctas, int threads, cudaStream_t s)
{
    switch (a.team.world) {
        case 2: return launch(k_reduce_scatter_zc<T, TO, INT, 2>, a, ctas, threads, s, false);
        case 4: return launch(k_reduce_scatter_zc<T, TO, INT, 4>, a, ctas, threads, s, false);
        case 8: return launch(k_reduce_scatter_zc<T, TO, INT, 8>, a, ctas, threads, s, false);
        default: return launch(k_reduce_scatter_zc<T, TO, INT, 0>, a, ctas, threads, s, false);
    }
}
template <typename T, typename TO> int launch_rs_mc(const CollArgs &a, int ctas, int threads, cudaStream_t s)
{
    switch (a.team.world) {
        case 2: return launch(k_reduce_scatter_mc<T, TO, 2>, a, ctas, threads, s, false);
        case 4: return launch(k_reduce_scatter_mc<T, TO, 4>, a, ctas, threads, s, false);
        case 8: return launch(k_reduce_scatter_mc<T, TO, 8>, a, ctas, threads, s, false);
        default: return launch(k_reduce_scatter_mc<T, TO, 0>, a, ctas, threads, s, false);
    }
}
template <typename T, typename TO, bool INT> int launch_rs(const CollArgs &a, int ctas, int threads, cudaStream_t s)
{
    switch (a.team.world) {
        case 2: return launch(k_reduce_scatter<T, TO, INT, 2>, a, ctas, threads, s, false);
        case 4: return launch(k_reduce_scatter<T, TO, INT, 4>, a, ctas, threads, s, false);
        case 8: return launch(k_reduce_scatter<T, TO, INT, 8>, a, ctas, threads, s, false);
        default: return launch(k_reduce_scatter<T, TO, INT, 0>, a, ctas, threads, s, false);
    }
}
}  // namespace

extern "C" {

// kind: 0 allreduce, 1 reduce_scatter, 2 allgather, 3 broadcast. dtypes as mfk::DType. Returns 0 or a CUDA error.
int mf_coll_launch(int kind, int in_dtype, int out_dtype, const CollArgs *args, int ctas, int threads, void *stream)
{
    if (args == nullptr || ctas <= 0 || ctas > kMaxCtas || threads <= 0 || threads > 512 || args->team.world == 0 ||
        args->team.world > kMaxRanks || (int)args->team.world > threads)
        return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const CollArgs &a = *args;
    const bool same = in_dtype == out_dtype;
    const bool to_bf16 = out_dtype == DT_BF16;
    if (!same && !to_bf16) return -2;
    if (a.zero_copy == 3) {
        // direct mode through the NVLink multicast alias: all-reduce (sum, same type in and out), reduce-scatter (sum), all-gather, rooted copy
        if (a.team.emu || a.team.mc_base == 0) return -4;
        if (kind == 0) {
            if (!same) return -4;
            if (in_dtype == DT_BF16) return launch_allreduce_mc<__nv_bfloat16>(a, ctas, threads, s);
            if (in_dtype == DT_F16) return launch_allreduce_mc<__half>(a, ctas, threads, s);
            if (in_dtype == DT_F32) return launch_allreduce_mc<float>(a, ctas, threads, s);
            return -2;
        }
        if (kind == 1) {
            if (in_dtype == DT_BF16) return launch_rs_mc<__nv_bfloat16, __nv_bfloat16>(a, ctas, threads, s);
            if (in_dtype == DT_F16) return same ? launch_rs_mc<__half, __half>(a, ctas, threads, s) : -2;
            if (in_dtype == DT_F32)
                return same ? launch_rs_mc<float, float>(a, ctas, threads, s) : launch_rs_mc<float, __nv_bfloat16>(a, ctas, threads, s);
            return -2;
        }
        if (kind == 2) {
            if (in_dtype == DT_BF16) return launch(k_allgather_mc<__nv_bfloat16, __nv_bfloat16>, a, ctas, threads, s, false);
            if (in_dtype == DT_F16) return same ? launch(k_allgather_mc<__half, __half>, a, ctas, threads, s, false) : -2;
            if (in_dtype == DT_F32)
                return same ? launch(k_allgather_mc<float, float>, a, ctas, threads, s, false)
                            : launch(k_allgather_mc<float, __nv_bfloat16>, a, ctas, threads, s, false);
            if (in_dtype == DT_I32) return same ? launch(k_allgather_mc<int, int>, a, ctas, threads, s, false) : -2;
            return -2;
        }
        if (kind == 3) {
            if (in_dtype == DT_F32 || in_dtype == DT_I32) return launch(k_broadcast_mc<float>, a, ctas, threads, s, false);
            return launch(k_broadcast_mc<__nv_bfloat16>, a, ctas, threads, s, false);
        }
        return -4;
    }
    if (a.zero_copy == 2) {
        // direct mode: the buffers named by the operation live inside the callers' own slices; emulation
        // keeps its per-rank buffers outside the emulated slots, so it has no direct mode
        if (a.team.emu) return -4;
        switch (kind) {
            case 0:
                if (in_dtype == DT_BF16) return launch_allreduce_zc<__nv_bfloat16, __nv_bfloat16, false>(a, ctas, threads, s);
                if (in_dtype == DT_F16) return same ? launch_allreduce_zc<__half, __half, false>(a, ctas, threads, s) : -2;
                if (in_dtype == DT_F32)
                    return same ? launch_allreduce_zc<float, float, false>(a, ctas, threads, s)
                                : launch_allreduce_zc<float, __nv_bfloat16, false>(a, ctas, threads, s);
                if (in_dtype == DT_I32) return same ? launch_allreduce_zc<int, int, true>(a, ctas, threads, s) : -2;
                return -2;
            case 1:
                if (in_dtype == DT_BF16) return launch_rs_zc<__nv_bfloat16, __nv_bfloat16, false>(a, ctas, threads, s);
                if (in_dtype == DT_F16) return same ? launch_rs_zc<__half, __half, false>(a, ctas, threads, s) : -2;
                if (in_dtype == DT_F32)
                    return same ? launch_rs_zc<float, float, false>(a, ctas, threads, s)
                                : launch_rs_zc<float, __nv_bfloat16, false>(a, ctas, threads, s);
                if (in_dtype == DT_I32) return same ? launch_rs_zc<int, int, true>(a, ctas, threads, s) : -2;
                return -2;
            case 2:
                if (in_dtype == DT_BF16) return launch(k_allgather_zc<__nv_bfloat16, __nv_bfloat16>, a, ctas, threads, s, false);
                if (in_dtype == DT_F16) return same ? launch(k_allgather_zc<__half, __half>, a, ctas, threads, s, false) : -2;
                if (in_dtype == DT_F32)
                    return same ? launch(k_allgather_zc<float, float>, a, ctas, threads, s, false)
                                : launch(k_allgather_zc<float, __nv_bfloat16>, a, ctas, threads, s, false);
                if (in_dtype == DT_I32) return same ? launch(k_allgather_zc<int, int>, a, ctas, threads, s, false) : -2;
                return -2;
            case 3:
                if (in_dtype == DT_F32 || in_dtype == DT_I32) return launch(k_broadcast_zc<float>, a, ctas, threads, s, false);
                return launch(k_broadcast_zc<__nv_bfloat16>, a, ctas, threads, s, false);
            default:
                return -3;
        }
    }
    switch (kind) {
        case 0:
            if (in_dtype == DT_BF16) return launch_allreduce<__nv_bfloat16, __nv_bfloat16, false>(a, ctas, threads, s);
            if (in_dtype == DT_F16) return same ? launch_allreduce<__half, __half, false>(a, ctas, threads, s) : -2;
            if (in_dtype == DT_F32)
                return same ? launch_allreduce<float, float, false>(a, ctas, threads, s)
                            : launch_allreduce<float, __nv_bfloat16, false>(a, ctas, threads, s);
            if (in_dtype == DT_I32) return same ? launch_allreduce<int, int, true>(a, ctas, threads, s) : -2;
            return -2;
        case 1:
            if (in_dtype == DT_BF16) return launch_rs<__nv_bfloat16, __nv_bfloat16, false>(a, ctas, threads, s);
            if (in_dtype == DT_F16) return same ? launch_rs<__half, __half, false>(a, ctas, threads, s) : -2;
            if (in_dtype == DT_F32)
                return same ? launch_rs<float, float, false>(a, ctas, threads, s) : launch_rs<float, __nv_bfloat16, false>(a, ctas, threads, s);
            if (in_dtype == DT_I32) return same ? launch_rs<int, int, true>(a, ctas, threads, s) : -2;
            return -2;
        case 2:
            if (in_dtype == DT_BF16) return launch(k_allgather<__nv_bfloat16, __nv_bfloat16>, a, ctas, threads, s, false);
            if (in_dtype == DT_F16) return same ? launch(k_allgather<__half, __half>, a, ctas, threads, s, false) : -2;
            if (in_dtype == DT_F32)
                return same ? launch(k_allgather<float, float>, a, ctas, threads, s, false)
                            : launch(k_allgather<float, __nv_bfloat16>, a, ctas, threads, s, false);
            if (in_dtype == DT_I32) return same ? launch(k_allgather<int, int>, a, ctas, threads, s, false) : -2;
            return -2;
        case 3:
            // broadcast moves bytes: n is in units of the element size chosen by the caller
            if (in_dtype == DT_F32 || in_dtype == DT_I32) return launch(k_broadcast<float>, a, ctas, threads, s, false);
            return launch(k_broadcast<__nv_bfloat16>, a, ctas, threads, s, false);
        default:
            return -3;
    }
}

int mf_coll_alltoallv(const A2AArgs *args, int ctas, int threads, void *stream)
{
    if (args == nullptr || ctas <= 0 || ctas > kMaxCtas || threads < (int)args->team.world || threads > 512) return -1;
    // lanes of one rank wait on a shared counter: the grid must be co-resident
    return launch(k_alltoallv, *args, ctas, threads, (cudaStream_t)stream, true);
}

int mf_coll_send(const P2PArgs *args, int ctas, void *stream) { return args ? launch(k_send, *args, ctas, 512, (cudaStream_t)stream, true) : -1; }
int mf_coll_recv(const P2PArgs *args, int ctas, void *stream) { return args ? launch(k_recv, *args, ctas, 512, (cudaStream_t)stream, true) : -1; }

int mf_coll_barrier(const Team *team, uint32_t channel, uint32_t epoch, void *stream)
{
    if (team == nullptr || channel >= 64) return -1;
    dim3 grid(1, team->emu ? team->world : 1);
    if (team->emu) {
        void *params[] = {const_cast<Team *>(team), &channel, &epoch};
        cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(k_barrier), grid, dim3(32), params, 0, (cudaStream_t)stream);
        return e == cudaSuccess ? 0 : (int)e;
    }
    k_barrier<<<grid, 32, 0, (cudaStream_t)stream>>>(*team, channel, epoch);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

int mf_coll_wait_flag(const Team *team, uint64_t flag_off, uint32_t epoch, void *stream)
{
    if (team == nullptr) return -1;
    k_wait_flag<<<1, 32, 0, (cudaStream_t)stream>>>(*team, flag_off, epoch);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

}  // extern "C"
MF_DEVTRACE_DEFINE_SETTER(mf_coll_set_devtrace)
extern "C" {
unsigned mf_coll_signal_bytes(void) { return kSignalBytes; }
unsigned mf_coll_max_ctas(void) { return kMaxCtas; }
unsigned mf_coll_args_size(void) { return (unsigned)sizeof(CollArgs); }

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// All-reduce without allocation (declared in include/mf_noalloc.h; no counterpart in the reference).
// The staging buffers and flags of the emulated group live in this file-scope array instead of a heap
// that somebody had to allocate. In host code the array's name is only a handle: the device address
// comes from cudaGetSymbolAddress, once per device, with that device current.
#include <mutex>

#include "../include/mf_noalloc.h"

namespace {
constexpr uint64_t kNaSlot = (uint64_t)kSignalBytes + 2ull * MF_NOALLOC_MAX_BYTES;  // flags | staging A | staging B
static __device__ __align__(256) unsigned char g_noalloc_scratch[MF_NOALLOC_MAX_WORLD * kNaSlot];

struct NaDevice {
    void *base = nullptr;  // device address of g_noalloc_scratch on that device
    uint32_t epoch = 0;
};
std::mutex g_na_mu;
NaDevice g_na_dev[64];
}  // namespace

extern "C" {

const char *mf_noalloc_strerror(int code)
{
    switch (code) {
        case MF_NOALLOC_OK: return "ok";
        case MF_NOALLOC_E_ARG: return "bad argument: null pointer, or dtype / op / world out of range";
        case MF_NOALLOC_E_TOO_LARGE: return "vector larger than MF_NOALLOC_MAX_BYTES (1 MiB): the built-in scratch cannot stage it";
        case MF_NOALLOC_E_SETUP: return "could not obtain the device address of the built-in scratch array";
        case MF_NOALLOC_E_LAUNCH: return "kernel launch refused";
        case MF_NOALLOC_E_TIMEOUT: return "a bounded wait inside an earlier call ran out: that call did not write its output";
        default: return "unknown code";
    }
}

int mf_allreduce_stacked_noalloc(const void *in, void *out, int world, uint64_t n, int dtype, int op, float scale, void *stream)
{
    if (in == nullptr || out == nullptr || world < 1 || world > MF_NOALLOC_MAX_WORLD || n == 0 || dtype < 0 || dtype > 3 || op < 0 || op > 3)
        return MF_NOALLOC_E_ARG;
    const uint64_t es = (dtype == DT_F32 || dtype == DT_I32) ? 4 : 2;
    if (n > MF_NOALLOC_MAX_BYTES / es) return MF_NOALLOC_E_TOO_LARGE;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MF_NOALLOC_E_SETUP;
    uint32_t epoch;
    void *base;
    {
        std::lock_guard<std::mutex> lock(g_na_mu);
        NaDevice &d = g_na_dev[dev];
        if (d.base == nullptr) {
            // first call on this device: resolve the symbol here (its host-side name is not a device
            // pointer). A file-scope __device__ array is zero when the module is loaded, so the status
            // words and flags need no clearing, and nothing is queued on any stream but the caller's.
            void *p = nullptr;
            if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) {
                (void)cudaGetLastError();
                return MF_NOALLOC_E_SETUP;
            }
            d.base = p;
        }
        base = d.base;
        epoch = ++d.epoch;
    }
    CollArgs a{};
    a.team.heap_base = reinterpret_cast<uint64_t>(base);
    a.team.stride = kNaSlot;
    a.team.mc_base = 0;
    a.team.rank = 0;
    a.team.world = (uint32_t)world;
    a.team.emu = 1;
    a.team.spin_limit = 1u << 22;
    a.in = reinterpret_cast<uint64_t>(in);
    a.out = reinterpret_cast<uint64_t>(out);
    a.in_rank_stride = n * es;
    a.out_rank_stride = n * es;
    a.n = n;
    a.stage_a = kSignalBytes;
    a.stage_b = kSignalBytes + MF_NOALLOC_MAX_BYTES;
    a.scale = scale;
    a.op = op;
    a.epoch = epoch;
    a.zero_copy = 0;
    a.root = 0;
    a.algo = 0;  // one-shot: a single set of staging buffers is enough because calls are serialised
    const int ctas = n * es <= (32u << 10) ? 1 : (n * es <= (256u << 10) ? 4 : 8);
    int rc = mf_coll_launch(0, dtype, dtype, &a, ctas, 512, stream);
    return rc == 0 ? MF_NOALLOC_OK : MF_NOALLOC_E_LAUNCH;
}

int mf_noalloc_status(uint32_t out[4], int clear)
{
    if (out == nullptr) return MF_NOALLOC_E_ARG;
    out[0] = out[1] = out[2] = out[3] = 0;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MF_NOALLOC_E_SETUP;
    void *base;
    {
        std::lock_guard<std::mutex> lock(g_na_mu);
        base = g_na_dev[dev].base;
    }
    if (base == nullptr) return MF_NOALLOC_OK;  // no call on this device yet: nothing can have gone wrong
    for (int r = 0; r < MF_NOALLOC_MAX_WORLD; r++) {
        uint32_t w[4] = {0, 0, 0, 0};
        unsigned char *st = static_cast<unsigned char *>(base) + r * kNaSlot + kStatusOff;
        if (cudaMemcpy(w, st, sizeof(w), cudaMemcpyDeviceToHost) != cudaSuccess) {
            (void)cudaGetLastError();
            return MF_NOALLOC_E_SETUP;
        }
        if (w[0] != 0) {
            if (out[0] == 0) {
                out[0] = w[0];
                out[1] = w[1];
                out[2] = w[2];
            }
            out[3] += w[3];
            if (clear && cudaMemset(st, 0, sizeof(w)) != cudaSuccess) {
                (void)cudaGetLastError();
                return MF_NOALLOC_E_SETUP;
            }
        }
    }
    return out[0] == 0 ? MF_NOALLOC_OK : MF_NOALLOC_E_TIMEOUT;
}

}  // extern "C"
