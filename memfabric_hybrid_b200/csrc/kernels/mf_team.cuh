// Device-side view of the symmetric heap and the cross-GPU signalling primitives every multi-GPU
// kernel here is built from.
//
// Addressing: each rank owns one slot of `stride` bytes in a range mapped at the same address by all
// ranks; an object at offset `off` of rank r lives at heap_base + r * stride + off. One multiply-add,
// no table (the rule the reference's kernels use: zbal_kernel_base.h:35-42).
//
// Signals: 32-bit epoch-numbered flags written with st.release.sys into the peer's slot and polled with
// ld.acquire.sys. Every wait is bounded: when the budget runs out the waiter records where it gave up
// in the status words of its own slot and the kernel returns normally (no trap, no endless spin), so a
// peer that never arrives costs a time-out, not a hung GPU. Epochs only grow, so a flag left over from
// an earlier call can never satisfy a later wait (the reference's `waitSymbol`,
// zbal_comm_host_device_struct.h:235).
//
// Emulation: with team.emu != 0 the rank is taken from blockIdx.y, so ONE cooperative launch runs all
// ranks of a protocol on one GPU (ranks must never be separate launches on one device: nothing would
// guarantee they run at the same time).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mfk {

constexpr int kMaxRanks = 16;           // NVSwitch domain of one box (8) with head-room
constexpr int kMaxCtas = 256;           // CTAs of one collective launch that own private flag lanes
constexpr uint32_t kSignalBytes = 1u << 20;  // signal area at the start of every slot

// Layout of the signal area (all offsets relative to the slot start):
//   [0, 64)                      status words: [0] error code, [1] where, [2] epoch, [3] count
//   [4 KiB, 4 KiB + 64 KiB)      barrier flags   [channel 0..63][rank 0..15] x u32 (padded to 256 B rows)
//   [128 KiB, ...)               lane flags      [phase 0..3][cta 0..255][rank 0..15] x u32
constexpr uint32_t kStatusOff = 0;
constexpr uint32_t kBarrierOff = 4096;
constexpr uint32_t kLaneOff = 128 * 1024;
constexpr int kPhases = 4;
//   [256 KiB, 256 KiB + 128 KiB) address exchange [cta 0..255][rank 0..15] x 4 words {epoch, 32 bits of payload}
constexpr uint32_t kXchgOff = 256 * 1024;

enum MfStatus : uint32_t { ST_OK = 0, ST_TIMEOUT = 1, ST_BAD_ARG = 2 };

struct Team {
    uint64_t heap_base;   // address of rank 0's slot
    uint64_t stride;      // bytes between consecutive ranks' slots
    uint64_t mc_base;     // multicast alias of the heap (0 when NVLS is not bound)
    uint32_t rank;
    uint32_t world;
    uint32_t emu;         // 1: rank = blockIdx.y (single-GPU emulation of all ranks)
    uint32_t spin_limit;  // polls before a wait gives up
};

__device__ __forceinline__ uint32_t team_rank(const Team &t) { return t.emu ? blockIdx.y : t.rank; }

__device__ __forceinline__ uint8_t *peer_ptr(const Team &t, uint32_t r, uint64_t off)
{
    return reinterpret_cast<uint8_t *>(t.heap_base + (uint64_t)r * t.stride + off);
}

__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t *p)
{
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void report_timeout(const Team &t, uint32_t me, uint32_t where, uint32_t epoch)
{
    uint32_t *st = reinterpret_cast<uint32_t *>(peer_ptr(t, me, kStatusOff));
    if (atomicCAS(st, ST_OK, ST_TIMEOUT) == ST_OK) {
        st[1] = where;
        st[2] = epoch;
    }
    atomicAdd(st + 3, 1u);
}

// Polls until *flag >= epoch (wrap-safe). Returns false when the budget ran out.
__device__ __forceinline__ bool wait_flag(const uint32_t *flag, uint32_t epoch, uint32_t limit)
{
    for (uint32_t i = 0; i < limit; i++) {
        if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
        if (i > 64) __nanosleep(i > 4096 ? 256 : 32);
    }
    return false;
}

// CTA-lane handshake: CTA b of every rank tells CTA b of every other rank that its stores of `phase`
// are visible, then waits for the same from all of them. All threads of the CTA must call it.
// Returns false on time-out (uniform across the CTA).
__device__ __forceinline__ bool lane_sync(const Team &t, uint32_t me, int phase, uint32_t epoch, uint32_t where)
{
    __shared__ int ok_sh;
    // The CTA barrier orders every thread's earlier stores (possibly to peers) before the signalling threads, whose
    // system-scope release store then publishes all of them (release is cumulative). Only the few signalling threads
    // pay for system-scope ordering: a fence in every thread of a 512-thread CTA cost several microseconds per
    // handshake, and a separate fence in front of the release store about three more.
    __syncthreads();
    const uint32_t lane = blockIdx.x;
    const uint64_t off = kLaneOff + (((uint64_t)phase * kMaxCtas + lane) * kMaxRanks) * sizeof(uint32_t);
    if (threadIdx.x == 0) ok_sh = 1;
    __syncthreads();
    if (threadIdx.x < t.world) {
        const uint32_t r = threadIdx.x;
        st_release_sys(reinterpret_cast<uint32_t *>(peer_ptr(t, r, off)) + me, epoch);
        const uint32_t *mine = reinterpret_cast<const uint32_t *>(peer_ptr(t, me, off)) + r;
        if (!wait_flag(mine, epoch, t.spin_limit)) {
            ok_sh = 0;
            report_timeout(t, me, where, epoch);
        }
    }
    __syncthreads();
    return ok_sh != 0;
}

// Swaps two 64-bit values (buffer offsets inside the senders' slots) between the CTAs of one lane, and with that tells
// every peer that this rank has entered the call. Nothing here needs release ordering (no data written by this call
// has to be visible yet), so it is done with flag-carrying words: each value travels as two 8-byte words
// {epoch, 32 bits of payload} written with relaxed system-scope stores (an aligned 8-byte store arrives whole), and the
// receiver polls its own row until all four words of a peer carry this call's epoch. One NVLink crossing, no fence.
// peer_a / peer_b are shared-memory arrays of kMaxRanks entries, valid for every thread on return. A row is rewritten
// by the next call only: callers end with a lane_sync, which a peer passes after it has read its row.
__device__ __forceinline__ void st_relaxed_sys_u64(uint64_t *p, uint64_t v)
{
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_relaxed_sys_u64(const uint64_t *p)
{
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ bool lane_sync_xchg(const Team &t, uint32_t me, int phase, uint32_t epoch, uint32_t where, uint64_t my_a,
                                               uint64_t my_b, uint64_t *peer_a, uint64_t *peer_b)
{
    (void)phase;
    __shared__ int ok_sh;
    const uint32_t lane = blockIdx.x;
    const uint64_t xoff = kXchgOff + ((uint64_t)lane * kMaxRanks) * 32;  // 4 words of 8 bytes per (lane, sender)
    if (threadIdx.x == 0) ok_sh = 1;
    __syncthreads();
    if (threadIdx.x < t.world) {
        const uint32_t r = threadIdx.x;
        const uint64_t tag = (uint64_t)epoch << 32;
        uint64_t *to = reinterpret_cast<uint64_t *>(peer_ptr(t, r, xoff)) + (uint64_t)me * 4;
        st_relaxed_sys_u64(to + 0, tag | (uint32_t)my_a);
        st_relaxed_sys_u64(to + 1, tag | (uint32_t)(my_a >> 32));
        st_relaxed_sys_u64(to + 2, tag | (uint32_t)my_b);
        st_relaxed_sys_u64(to + 3, tag | (uint32_t)(my_b >> 32));
        const uint64_t *row = reinterpret_cast<const uint64_t *>(peer_ptr(t, me, xoff)) + (uint64_t)r * 4;
        uint64_t w[4] = {0, 0, 0, 0};
        bool got = false;
        for (uint32_t i = 0; i < t.spin_limit && !got; i++) {
#pragma unroll
            for (int k = 0; k < 4; k++) w[k] = ld_relaxed_sys_u64(row + k);
            got = (uint32_t)(w[0] >> 32) == epoch && (uint32_t)(w[1] >> 32) == epoch && (uint32_t)(w[2] >> 32) == epoch &&
                  (uint32_t)(w[3] >> 32) == epoch;
            if (!got && i > 64) __nanosleep(i > 4096 ? 256 : 32);
        }
        if (!got) {
            ok_sh = 0;
            report_timeout(t, me, where, epoch);
            peer_a[r] = 0;
            peer_b[r] = 0;
        } else {
            peer_a[r] = (w[0] & 0xFFFFFFFFull) | (w[1] << 32);
            peer_b[r] = (w[2] & 0xFFFFFFFFull) | (w[3] << 32);
        }
    }
    __syncthreads();
    return ok_sh != 0;
}

// Whole-rank barrier on a numbered channel; call from ONE CTA (all its threads).
__device__ __forceinline__ bool team_barrier(const Team &t, uint32_t me, uint32_t channel, uint32_t epoch)
{
    __shared__ int ok_sh;
    __syncthreads();  // see lane_sync: the signalling threads fence for the whole CTA
    const uint64_t off = kBarrierOff + (uint64_t)channel * 256;
    if (threadIdx.x == 0) ok_sh = 1;
    __syncthreads();
    if (threadIdx.x < t.world) {
        const uint32_t r = threadIdx.x;
        st_release_sys(reinterpret_cast<uint32_t *>(peer_ptr(t, r, off)) + me, epoch);
        const uint32_t *mine = reinterpret_cast<const uint32_t *>(peer_ptr(t, me, off)) + r;
        if (!wait_flag(mine, epoch, t.spin_limit)) {
            ok_sh = 0;
            report_timeout(t, me, 0x1000 | channel, epoch);
        }
    }
    __syncthreads();
    return ok_sh != 0;
}

}  // namespace mfk
