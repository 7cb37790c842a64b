/*
 * Device-side API of the symmetric shared memory (SHM): what a user kernel needs to reach its peers'
 * slices and to synchronise with them.
 *
 *   __global__ void k(smem_shm_device_ctx_t ctx, float *mine, ...)   // ctx comes from smem_shm_get_device_context()
 *   {
 *       float *theirs = smem_shm_peer_ptr(ctx, mine, peer);          // same object in the peer's slice
 *       ...
 *       if (!smem_shm_barrier(ctx, epoch)) return;                   // bounded: false = a peer did not arrive
 *   }
 *
 * Addressing rule: an object at address p of this rank's slice lives at p + (peer - my_rank) * symmetric_size
 * on the peer (the rule of the reference's device API, src/smem/include/device/ of the reference, and of
 * examples/hbm_share_memory there). Loads and stores to that address travel over NVLink.
 * Synchronisation: the first 1 MiB of every slice is reserved for flags (status words, barrier rows);
 * user data starts at SMEM_SHM_USER_OFFSET. Flags carry call numbers ("epochs") that the caller
 * increases by one per call, so nothing has to be cleared between calls. Every wait gives up after
 * ctx.spin_limit polls, writes a status code into the slice's status words (read them with
 * smem_shm_device_status on the host) and returns false; nothing traps and nothing spins forever.
 */
#ifndef MF_B200_SMEM_SHM_DEVICE_CUH
#define MF_B200_SMEM_SHM_DEVICE_CUH

#include <stdint.h>

#define SMEM_SHM_USER_OFFSET (1u << 20)
/* The extra context that the host set with smem_shm_set_extra_context lives inside the flag area of the rank's own
 * slice: a 32-bit size at this offset, the bytes (at most 64 KiB) 64 bytes further on. */
#define SMEM_SHM_EXTRA_CTX_OFFSET (896u << 10)
#define SMEM_SHM_EXTRA_CTX_MAX 65536u

typedef struct {
    uint64_t base;           /* address of rank 0's slice */
    uint64_t symmetric_size; /* bytes between consecutive ranks' slices */
    uint64_t mc_base;        /* multicast alias, 0 when not bound */
    uint32_t rank;
    uint32_t rank_size;
    uint32_t reserved;       /* must be 0 */
    uint32_t spin_limit;     /* polls before a wait gives up (about 0.5 us each once it backs off) */
} smem_shm_device_ctx_t;

#ifdef __CUDACC__
#include "../kernels/mf_team.cuh"

__device__ __forceinline__ uint32_t smem_shm_get_global_rank(const smem_shm_device_ctx_t &c) { return c.rank; }
__device__ __forceinline__ uint32_t smem_shm_get_global_rank_size(const smem_shm_device_ctx_t &c) { return c.rank_size; }
__device__ __forceinline__ uint64_t smem_shm_get_symmetric_size(const smem_shm_device_ctx_t &c) { return c.symmetric_size; }

/* The peer's copy of an object of this rank's slice. */
template <typename T> __device__ __forceinline__ T *smem_shm_peer_ptr(const smem_shm_device_ctx_t &c, T *local, uint32_t peer)
{
    return reinterpret_cast<T *>(reinterpret_cast<uint64_t>(local) + ((int64_t)peer - (int64_t)c.rank) * (int64_t)c.symmetric_size);
}
/* Address of byte `offset` of a rank's slice. */
__device__ __forceinline__ void *smem_shm_slice_ptr(const smem_shm_device_ctx_t &c, uint32_t rank, uint64_t offset)
{
    return reinterpret_cast<void *>(c.base + (uint64_t)rank * c.symmetric_size + offset);
}

/* The user's extra context of THIS rank (set on the host with smem_shm_set_extra_context; every rank sets its own) and
 * its size in bytes, 0 when none was set. Parity: smem_shm_get_extra_context_addr / _size of the reference's device API
 * (src/smem/include/device/smem_shm_aicore_base_api.h:44-53). */
__device__ __forceinline__ const void *smem_shm_get_extra_context_addr(const smem_shm_device_ctx_t &c)
{
    return smem_shm_slice_ptr(c, c.rank, SMEM_SHM_EXTRA_CTX_OFFSET + 64);
}
__device__ __forceinline__ uint32_t smem_shm_get_extra_context_size(const smem_shm_device_ctx_t &c)
{
    return *reinterpret_cast<const volatile uint32_t *>(smem_shm_slice_ptr(c, c.rank, SMEM_SHM_EXTRA_CTX_OFFSET));
}

__device__ __forceinline__ mfk::Team smem_shm_team(const smem_shm_device_ctx_t &c)
{
    mfk::Team t;
    t.heap_base = c.base, t.stride = c.symmetric_size, t.mc_base = c.mc_base;
    t.rank = c.rank, t.world = c.rank_size, t.emu = 0, t.spin_limit = c.spin_limit;
    return t;
}

/* All ranks meet; call from ONE block with all its threads (blockDim.x >= rank_size). channel 32..63 is
 * free for user kernels. Orders this rank's earlier stores (to any slice) before the peers' later loads. */
__device__ __forceinline__ bool smem_shm_barrier(const smem_shm_device_ctx_t &c, uint32_t epoch, uint32_t channel = 32)
{
    return mfk::team_barrier(smem_shm_team(c), c.rank, channel, epoch);
}

/* One-way signal: raise flag word `index` (0..15) of `channel` in the peer's slice to `epoch`. */
__device__ __forceinline__ void smem_shm_signal(const smem_shm_device_ctx_t &c, uint32_t peer, uint32_t channel, uint32_t index, uint32_t epoch)
{
    __threadfence_system();
    uint32_t *f = reinterpret_cast<uint32_t *>(smem_shm_slice_ptr(c, peer, mfk::kBarrierOff + (uint64_t)channel * 256)) + 16 + (index & 15);
    mfk::st_release_sys(f, epoch);
}
/* Waits until flag word `index` of `channel` in the own slice reaches `epoch`; false on time-out. */
__device__ __forceinline__ bool smem_shm_wait(const smem_shm_device_ctx_t &c, uint32_t channel, uint32_t index, uint32_t epoch)
{
    const uint32_t *f = reinterpret_cast<const uint32_t *>(smem_shm_slice_ptr(c, c.rank, mfk::kBarrierOff + (uint64_t)channel * 256)) + 16 + (index & 15);
    if (mfk::wait_flag(f, epoch, c.spin_limit)) return true;
    mfk::report_timeout(smem_shm_team(c), c.rank, 0x2000 | channel, epoch);
    return false;
}

/* ---- data movement helpers (the reference's smem_shm_copy_ub2gm / gm2ub and smem_shm_roce_write / read) -------------
 * "ub" is the on-chip buffer of the calling block: shared memory here. The global side may be any address of any rank's
 * slice (smem_shm_peer_ptr / smem_shm_slice_ptr): stores and loads to a peer travel over NVLink. All threads of the CTA
 * call these together; 16-byte vectors when both addresses allow it, bytes otherwise. The calls return when the calling
 * thread's part is issued: put a __syncthreads() (and, before telling a peer, smem_shm_signal, whose release covers the
 * CTA's stores after a barrier) behind them as with any other store. */
template <typename T> __device__ __forceinline__ void smem_shm_copy_ub2gm(T *dst_gva, const T *src_smem, uint32_t bytes)
{
    const uint8_t *s = reinterpret_cast<const uint8_t *>(src_smem);
    uint8_t *d = reinterpret_cast<uint8_t *>(dst_gva);
    uint32_t done = 0;
    if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 15) == 0) {
        const uint32_t vecs = bytes / 16;
        for (uint32_t i = threadIdx.x; i < vecs; i += blockDim.x) reinterpret_cast<uint4 *>(d)[i] = reinterpret_cast<const uint4 *>(s)[i];
        done = vecs * 16;
    }
    for (uint32_t i = done + threadIdx.x; i < bytes; i += blockDim.x) d[i] = s[i];
}
template <typename T> __device__ __forceinline__ void smem_shm_copy_gm2ub(T *dst_smem, const T *src_gva, uint32_t bytes)
{
    const uint8_t *s = reinterpret_cast<const uint8_t *>(src_gva);
    uint8_t *d = reinterpret_cast<uint8_t *>(dst_smem);
    uint32_t done = 0;
    if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 15) == 0) {
        const uint32_t vecs = bytes / 16;
        for (uint32_t i = threadIdx.x; i < vecs; i += blockDim.x)
            reinterpret_cast<uint4 *>(d)[i] = __ldcg(reinterpret_cast<const uint4 *>(s) + i);  // a peer may have just written it: not through L1
        done = vecs * 16;
    }
    for (uint32_t i = done + threadIdx.x; i < bytes; i += blockDim.x) d[i] = *reinterpret_cast<const volatile uint8_t *>(s + i);
}
/* Remote write / read between this rank's memory and rank `peer`'s slice: `remote` is the address the object has in THIS
 * rank's slice (the symmetric address), as with smem_shm_peer_ptr. The whole grid shares the range: CTA b moves its part.
 * No queue pairs and no work requests on this hardware: the SMs store (load) through NVLink directly. */
template <typename T> __device__ __forceinline__ void smem_shm_roce_write(const smem_shm_device_ctx_t &c, const T *local_src, T *remote, uint32_t peer,
                                                                         uint64_t bytes)
{
    const uint8_t *s = reinterpret_cast<const uint8_t *>(local_src);
    uint8_t *d = reinterpret_cast<uint8_t *>(smem_shm_peer_ptr(c, remote, peer));
    const uint64_t per = ((bytes + gridDim.x - 1) / gridDim.x + 15) / 16 * 16;
    const uint64_t beg = min(bytes, (uint64_t)blockIdx.x * per), end = min(bytes, beg + per);
    uint64_t i = beg;
    if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 15) == 0) {
        const uint64_t vend = beg + (end - beg) / 16 * 16;
        for (i = beg + (uint64_t)threadIdx.x * 16; i < vend; i += (uint64_t)blockDim.x * 16)
            *reinterpret_cast<uint4 *>(d + i) = __ldg(reinterpret_cast<const uint4 *>(s + i));
        i = vend;
    }
    for (i += threadIdx.x; i < end; i += blockDim.x) d[i] = s[i];
}
template <typename T> __device__ __forceinline__ void smem_shm_roce_read(const smem_shm_device_ctx_t &c, const T *remote, T *local_dst, uint32_t peer,
                                                                        uint64_t bytes)
{
    const uint8_t *s = reinterpret_cast<const uint8_t *>(smem_shm_peer_ptr(c, const_cast<T *>(remote), peer));
    uint8_t *d = reinterpret_cast<uint8_t *>(local_dst);
    const uint64_t per = ((bytes + gridDim.x - 1) / gridDim.x + 15) / 16 * 16;
    const uint64_t beg = min(bytes, (uint64_t)blockIdx.x * per), end = min(bytes, beg + per);
    uint64_t i = beg;
    if (((reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(d)) & 15) == 0) {
        const uint64_t vend = beg + (end - beg) / 16 * 16;
        for (i = beg + (uint64_t)threadIdx.x * 16; i < vend; i += (uint64_t)blockDim.x * 16)
            *reinterpret_cast<uint4 *>(d + i) = __ldcg(reinterpret_cast<const uint4 *>(s + i));
        i = vend;
    }
    for (i += threadIdx.x; i < end; i += blockDim.x) d[i] = *reinterpret_cast<const volatile uint8_t *>(s + i);
}
/* Completion of remote writes (the reference's smem_shm_roce_quiet / smem_shm_roce_poll_cq, which drain a queue pair's
 * completion queue). There is no queue here: a store to a peer is complete for every observer once a system-scope fence
 * issued after it has returned. quiet() is that fence for the calling thread; all threads that wrote call it (or a
 * __syncthreads() follows and one thread fences, as smem_shm_signal does). poll_cq() reports how many work requests are
 * still in flight after a fence: always 0. */
__device__ __forceinline__ void smem_shm_roce_quiet(const smem_shm_device_ctx_t &c, uint32_t peer)
{
    (void)c;
    (void)peer;
    __threadfence_system();
}
__device__ __forceinline__ uint32_t smem_shm_roce_poll_cq(const smem_shm_device_ctx_t &c, uint32_t peer)
{
    smem_shm_roce_quiet(c, peer);
    return 0;
}
#endif /* __CUDACC__ */
#endif
