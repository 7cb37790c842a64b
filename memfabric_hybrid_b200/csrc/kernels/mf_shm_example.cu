// Example user kernel on the public device API of the symmetric shared memory: an all-reduce (sum) of
// fp32 vectors that live in the ranks' slices. Every rank reads all peers' inputs over NVLink after a
// barrier and writes its own output; a closing barrier keeps the inputs intact until all have read.
// The counterpart of the reference's examples/hbm_share_memory/AllReduce; k_example_shift below is the
// counterpart of examples/hbm_share_memory/ShiftPutGet (neighbour put with a one-way signal, neighbour get
// between barriers). The tuned collectives are
// in mf_coll.cu; this file shows what a few lines of user code on smem_shm_device.cuh look like.
#include <cooperative_groups.h>

#include "../include/smem_shm_device.cuh"

namespace {

__global__ void __launch_bounds__(256) k_example_allreduce(smem_shm_device_ctx_t ctx, const float *in, float *out, uint64_t n, uint32_t epoch,
                                                            int *status)
{
    cooperative_groups::grid_group grid = cooperative_groups::this_grid();
    __shared__ int ok;
    if (blockIdx.x == 0) {
        const bool good = smem_shm_barrier(ctx, 2 * epoch - 1);   // everybody's input is in place
        if (threadIdx.x == 0) {
            ok = good;
            if (!good) atomicExch(status, 1);
        }
    }
    grid.sync();
    if (*reinterpret_cast<volatile int *>(status) == 0) {
        for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
            float acc = 0.f;
            for (uint32_t r = 0; r < ctx.rank_size; r++) acc += __ldcg(smem_shm_peer_ptr(ctx, in, r) + i);
            out[i] = acc;
        }
    }
    grid.sync();
    if (blockIdx.x == 0) smem_shm_barrier(ctx, 2 * epoch);        // nobody overwrites its input before all have read it
}

// Shift: rank r hands its vector to rank r + 1 (mod size).
//   put (mode 0): stores `src` into the NEXT rank's `box` over NVLink, then raises a flag there; waits for the flag
//                 that the previous rank raises here. No barrier: a one-way signal per neighbour is enough.
//   get (mode 1): after a barrier (every rank's `src` is in place) loads the PREVIOUS rank's `src` into the own `box`;
//                 a closing barrier keeps `src` intact until the reader is done.
__global__ void __launch_bounds__(256) k_example_shift(smem_shm_device_ctx_t ctx, const float *src, float *box, uint64_t n, int mode,
                                                        uint32_t epoch, int *status)
{
    cooperative_groups::grid_group grid = cooperative_groups::this_grid();
    const uint32_t next = (ctx.rank + 1) % ctx.rank_size, prev = (ctx.rank + ctx.rank_size - 1) % ctx.rank_size;
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, step = (uint64_t)gridDim.x * blockDim.x;
    if (mode == 0) {
        float *remote = smem_shm_peer_ptr(ctx, box, next);
        for (uint64_t i = tid; i < n; i += step) remote[i] = src[i];
        grid.sync();                                              // all stores of this grid are issued ...
        if (blockIdx.x == 0 && threadIdx.x == 0) {
            smem_shm_signal(ctx, next, 33, 0, epoch);             // ... and made visible before the flag (fence inside)
            if (!smem_shm_wait(ctx, 33, 0, epoch)) atomicExch(status, 1);
        }
    } else {
        if (blockIdx.x == 0 && !smem_shm_barrier(ctx, 2 * epoch - 1, 34) && threadIdx.x == 0) atomicExch(status, 1);
        grid.sync();
        if (*reinterpret_cast<volatile int *>(status) == 0) {
            const float *remote = smem_shm_peer_ptr(ctx, src, prev);
            for (uint64_t i = tid; i < n; i += step) box[i] = __ldcg(remote + i);
        }
        grid.sync();
        if (blockIdx.x == 0) smem_shm_barrier(ctx, 2 * epoch, 34);
    }
}

}  // namespace

// src, box: inside this rank's slice, at the same offsets on every rank. mode 0 = put to the next rank, 1 = get from the
// previous rank. epoch: 1, 2, 3, ... per mode, the same on every rank. status: device int, 0 on entry; 1 = a wait ran out.
extern "C" int mf_example_shm_shift(const smem_shm_device_ctx_t *ctx, const float *src, float *box, uint64_t n, int mode, uint32_t epoch,
                                    int *status, void *stream)
{
    if (ctx == nullptr || ctx->rank_size == 0 || ctx->rank_size > 16 || (mode != 0 && mode != 1)) return -1;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    smem_shm_device_ctx_t c = *ctx;
    void *params[] = {&c, &src, &box, &n, &mode, &epoch, &status};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(k_example_shift), dim3(sms > 0 ? sms : 64), dim3(256), params,
                                                0, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : (int)e;
}

// in: inside this rank's slice (at the same offset on every rank); out: anywhere on this device.
// epoch: 1, 2, 3, ... one per call, the same on every rank. status: device int, 0 on entry; 1 = a peer did not arrive.
extern "C" int mf_example_shm_allreduce(const smem_shm_device_ctx_t *ctx, const float *in, float *out, uint64_t n, uint32_t epoch, int *status,
                                        void *stream)
{
    if (ctx == nullptr || ctx->rank_size == 0 || ctx->rank_size > 16) return -1;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    smem_shm_device_ctx_t c = *ctx;
    void *params[] = {&c, &in, &out, &n, &epoch, &status};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(k_example_allreduce), dim3(sms > 0 ? sms : 64), dim3(256),
                                                params, 0, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : (int)e;
}

namespace {
__global__ void k_example_read_context(smem_shm_device_ctx_t ctx, uint8_t *out, uint32_t cap, uint32_t *size_out)
{
    const uint32_t n = smem_shm_get_extra_context_size(ctx);
    const uint8_t *p = static_cast<const uint8_t *>(smem_shm_get_extra_context_addr(ctx));
    if (threadIdx.x == 0) *size_out = n;
    for (uint32_t i = threadIdx.x; i < n && i < cap; i += blockDim.x) out[i] = p[i];
}
}  // namespace

namespace {
// A round trip through every data-movement helper of the device header: `src` goes to rank `peer`'s copy of `box` with
// smem_shm_roce_write, comes back into `back` with smem_shm_roce_read, and CTA 0 takes the first `tile` bytes of the peer's
// box through shared memory (gm2ub, then ub2gm into `via_smem`). A barrier between the steps makes the peer's box complete.
__global__ void k_example_copy_helpers(smem_shm_device_ctx_t ctx, const uint8_t *src, uint8_t *box, uint8_t *back, uint8_t *via_smem, uint64_t bytes,
                                       uint32_t tile, uint32_t peer, int *ok)
{
    extern __shared__ __align__(16) uint8_t ub[];
    cooperative_groups::grid_group grid = cooperative_groups::this_grid();
    smem_shm_roce_write(ctx, src, box, peer, bytes);
    smem_shm_roce_quiet(ctx, peer);   // this thread's writes are complete at the peer
    grid.sync();
    smem_shm_roce_read(ctx, box, back, peer, bytes);
    if (blockIdx.x == 0) {
        smem_shm_copy_gm2ub(ub, smem_shm_peer_ptr(ctx, box, peer), tile);
        __syncthreads();
        smem_shm_copy_ub2gm(via_smem, ub, tile);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) *ok = 1;
}
}  // namespace

// Runs the helper round trip above on one rank (peer may be the rank itself). Cooperative launch of `ctas` blocks.
extern "C" int mf_example_shm_copy_helpers(const smem_shm_device_ctx_t *ctx, const void *src, void *box, void *back, void *via_smem, uint64_t bytes,
                                           uint32_t tile, uint32_t peer, int *ok, int ctas, void *stream)
{
    if (ctx == nullptr || src == nullptr || box == nullptr || back == nullptr || via_smem == nullptr || tile > 48 * 1024 || peer >= ctx->rank_size) return -1;
    smem_shm_device_ctx_t c = *ctx;
    const uint8_t *s = static_cast<const uint8_t *>(src);
    uint8_t *b = static_cast<uint8_t *>(box), *k = static_cast<uint8_t *>(back), *v = static_cast<uint8_t *>(via_smem);
    void *params[] = {&c, &s, &b, &k, &v, &bytes, &tile, &peer, &ok};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(k_example_copy_helpers), dim3((unsigned)ctas), dim3(256), params, tile,
                                                (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : (int)e;
}

// Copies this rank's extra context (smem_shm_set_extra_context) as a kernel sees it into out[0 .. cap) and its size into
// *size_out (both device memory).
extern "C" int mf_example_shm_read_context(const smem_shm_device_ctx_t *ctx, void *out, uint32_t cap, uint32_t *size_out, void *stream)
{
    if (ctx == nullptr || out == nullptr || size_out == nullptr) return -1;
    k_example_read_context<<<1, 256, 0, (cudaStream_t)stream>>>(*ctx, static_cast<uint8_t *>(out), cap, size_out);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
