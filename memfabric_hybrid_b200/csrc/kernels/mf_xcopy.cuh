// sm_100a copy kernels of the data-operation layer ("xcopy"): every byte that moves between two
// device-visible addresses (local HBM, a peer's HBM mapped over NVLink, pinned pooled DRAM) goes
// through these, issued from inside the kernel as 16-byte vector loads and stores.
//   mf_xcopy_batch_kernel : list of (src, dst, len) work chunks in a pinned, device-visible ring
//   mf_xcopy_quant_kernel : bf16/fp16 -> int8 (per-unit scale) or fp8 e4m3 (1x128 scale) while pushing
// Parity of role: src/hybm/csrc/copy_extend/hybm_copy_kernel.cpp:53-90 (contiguous), :114-136 (batch),
// :163-235 (quantising batch).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace mfk {

struct CopyItem {
    uint64_t src;
    uint64_t dst;
    uint64_t len;
};

struct QuantItem {
    uint64_t src;
    uint64_t dst;
    uint64_t scale;
    uint64_t elems;
};

// Debug aid (MF_XCOPY_DEBUG=1): the pool's address window as the copy kernels check it. An address inside the window must
// lie, with its whole length, in the part of a rank's slot that is mapped here; addresses outside the window are the
// caller's own buffers and are taken as given. A descriptor that fails is skipped (nothing is read or written) and
// reported through the status word. The host validates every item before it builds descriptors; this second check
// sits in front of the first access of the kernel itself, where a sanitizer would otherwise be the only witness.
struct CopyWindow {
    uint64_t base;        // 0: no window, nothing is checked
    uint64_t slot;        // bytes between consecutive ranks' slots
    uint32_t ranks;
    uint32_t pad;
    uint64_t mapped[64];  // bytes mapped of every rank's slot
};
constexpr uint32_t kCopyBadDescriptor = 0x7D1u;

__device__ __forceinline__ bool xc_in_window(const CopyWindow *w, uint64_t a, uint64_t len)
{
    if (w == nullptr || w->base == 0 || a < w->base || a >= w->base + w->slot * w->ranks) return true;
    const uint64_t rel = a - w->base;
    const uint32_t r = (uint32_t)(rel / w->slot);
    const uint64_t off = rel - (uint64_t)r * w->slot;
    const uint64_t m = r < 64 ? w->mapped[r] : 0;
    return len <= m && off <= m - len;
}
__device__ __forceinline__ bool xc_check(const CopyWindow *w, const uint64_t src, const uint64_t dst, const uint64_t len, uint32_t *status)
{
    if (xc_in_window(w, src, len) && xc_in_window(w, dst, len)) return true;
    *reinterpret_cast<volatile uint32_t *>(status) = kCopyBadDescriptor;
    __threadfence_system();
    return false;
}

constexpr int kCopyThreads = 512;
constexpr int kCopyUnroll = 4;

// Copies `len` bytes with all threads of the CTA. Fast path: both ends 16-byte aligned relative to
// each other; the unaligned head and tail go byte-wise.
__device__ __forceinline__ void cta_copy(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst, uint64_t len)
{
    const int tid = threadIdx.x;
    const int nt = blockDim.x;
    if (((reinterpret_cast<uint64_t>(src) ^ reinterpret_cast<uint64_t>(dst)) & 15) != 0) {
        // Mutually misaligned: 4-byte words when possible, else bytes. Rare (KV segments are aligned).
        if ((((reinterpret_cast<uint64_t>(src) | reinterpret_cast<uint64_t>(dst)) | len) & 3) == 0) {
            const uint32_t *s = reinterpret_cast<const uint32_t *>(src);
            uint32_t *d = reinterpret_cast<uint32_t *>(dst);
            for (uint64_t i = tid; i < len / 4; i += nt) d[i] = s[i];
        } else {
            for (uint64_t i = tid; i < len; i += nt) dst[i] = src[i];
        }
        return;
    }
    uint64_t head = (16 - (reinterpret_cast<uint64_t>(src) & 15)) & 15;
    if (head > len) head = len;
    if (tid < head) dst[tid] = src[tid];
    const uint64_t body = (len - head) & ~15ULL;
    const uint4 *s = reinterpret_cast<const uint4 *>(src + head);
    uint4 *d = reinterpret_cast<uint4 *>(dst + head);
    const uint64_t n16 = body >> 4;
    uint64_t i = tid;
    // main loop: kCopyUnroll independent 16-byte loads in flight per thread before the first store
    for (; i + (uint64_t)(kCopyUnroll - 1) * nt < n16; i += (uint64_t)kCopyUnroll * nt) {
        uint4 v[kCopyUnroll];
#pragma unroll
        for (int u = 0; u < kCopyUnroll; u++) v[u] = __ldcs(s + i + (uint64_t)u * nt);
#pragma unroll
        for (int u = 0; u < kCopyUnroll; u++) __stcs(d + i + (uint64_t)u * nt, v[u]);
    }
    for (; i < n16; i += nt) __stcs(d + i, __ldcs(s + i));
    const uint64_t tail = len - head - body;
    if (tid < tail) dst[head + body + tid] = src[head + body + tid];
}

__global__ void __launch_bounds__(kCopyThreads) mf_xcopy_batch_kernel(const CopyItem *__restrict__ items, uint32_t count,
                                                                      const CopyWindow *__restrict__ window, uint32_t *status)
{
    __shared__ CopyItem sh[2];
    uint32_t i = blockIdx.x;
    if (i >= count) return;
    if (threadIdx.x == 0) sh[0] = items[i];
    __syncthreads();
    int buf = 0;
    for (; i < count; i += gridDim.x) {
        const CopyItem it = sh[buf];
        // descriptor of the next chunk is fetched (from pinned host memory) while this one is copied
        if (threadIdx.x == 0 && i + gridDim.x < count) sh[buf ^ 1] = items[i + gridDim.x];
        if (window == nullptr || xc_check(window, it.src, it.dst, it.len, status))
            cta_copy(reinterpret_cast<const uint8_t *>(it.src), reinterpret_cast<uint8_t *>(it.dst), it.len);
        __syncthreads();
        buf ^= 1;
    }
}

// ---- bulk-copy engine variant ---------------------------------------------------------------------
// The same descriptor list, moved by the TMA unit instead of by registers: one lane per pipeline issues
// `cp.async.bulk` loads of `piece` bytes from the source into a ring of shared-memory stages and, as each
// lands (mbarrier), a `cp.async.bulk` store from that stage to the destination. No multicast; source and
// destination may be local HBM or a peer's mapped HBM. A pipeline keeps (stages - 2) loads and up to two
// stores in flight and runs on across chunk boundaries, so neither a CTA barrier nor a drain separates
// two items. Needs every chunk's source, destination and length to be multiples of 16 bytes (the host
// checks that and otherwise launches mf_xcopy_batch_kernel).
// A wait that runs out stores its code into *status (pinned host memory) and the pipeline stops after
// the copies it has in flight.
constexpr uint64_t kBulkWaitNs = 2000000000ull;  // a load that has not landed after 2 s is given up
constexpr int kBulkMaxStages = 8;

__device__ __forceinline__ uint32_t xc_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__global__ void __launch_bounds__(128) mf_xcopy_bulk_kernel(const CopyItem *__restrict__ items, uint32_t count, uint32_t stages,
                                                            uint32_t piece, uint32_t *status, const CopyWindow *__restrict__ window)
{
    extern __shared__ __align__(128) uint8_t xc_smem[];
    __shared__ __align__(8) uint64_t full[4][kBulkMaxStages];
    __shared__ uint64_t st_dst[4][kBulkMaxStages];
    __shared__ uint32_t st_len[4][kBulkMaxStages];
    if ((threadIdx.x & 31) != 0) return;
    const uint32_t w = threadIdx.x >> 5, W = blockDim.x >> 5;
    const uint32_t pipe = blockIdx.x * W + w, pipes = gridDim.x * W;
    if (pipe >= count) return;
    uint8_t *ring = xc_smem + (size_t)w * stages * piece;
    for (uint32_t s = 0; s < stages; s++)
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(xc_smem_u32(&full[w][s])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the initialised barriers as the copy unit sees them

    const uint32_t look = stages - 2;  // loads issued ahead of the store front
    uint32_t ci = pipe;                // chunk whose pieces are being loaded
    CopyItem cur = items[ci];
    CopyItem nxt = ci + pipes < count ? items[ci + pipes] : CopyItem{0, 0, 0};
    uint64_t off = 0;
    bool more = true, fine = true;
    // debug window: a chunk that fails the check is emptied (its pieces are never issued)
    if (window != nullptr && !xc_check(window, cur.src, cur.dst, cur.len, status)) off = cur.len;
    if (off >= cur.len) {
        // walk on to the first chunk of this pipeline that has bytes to move
        while (more && off >= cur.len) {
            ci += pipes;
            if (ci < count) {
                cur = nxt;
                off = (window != nullptr && !xc_check(window, cur.src, cur.dst, cur.len, status)) ? cur.len : 0;
                if (ci + pipes < count) nxt = items[ci + pipes];
            } else {
                more = false;
            }
        }
    }
    uint32_t loaded = 0, stored = 0;
    while (fine && (more || stored < loaded)) {
        if (more) {
            const uint32_t s = loaded % stages;
            // the store that last read this stage is at least two store groups back
            asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            const uint64_t left = cur.len - off;
            const uint32_t n = left < piece ? (uint32_t)left : piece;
            const uint32_t bar = xc_smem_u32(&full[w][s]);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(n) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                             xc_smem_u32(ring + (size_t)s * piece)),
                         "l"(cur.src + off), "r"(n), "r"(bar)
                         : "memory");
            st_dst[w][s] = cur.dst + off;
            st_len[w][s] = n;
            loaded++;
            off += n;
            while (more && off >= cur.len) {
                ci += pipes;
                if (ci < count) {
                    cur = nxt;
                    off = (window != nullptr && !xc_check(window, cur.src, cur.dst, cur.len, status)) ? cur.len : 0;
                    if (ci + pipes < count) nxt = items[ci + pipes];
                } else {
                    more = false;
                }
            }
        }
        if (loaded >= stored + look + 1 || (!more && stored < loaded)) {
            const uint32_t s = stored % stages, parity = (stored / stages) & 1;
            const uint32_t bar = xc_smem_u32(&full[w][s]);
            uint32_t ok = 0;
            uint64_t t0 = 0;
            for (uint32_t spin = 0; !ok; spin++) {
                asm volatile(
                    "{\n\t.reg .pred P;\n\t"
                    "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
                    "selp.b32 %0, 1, 0, P;\n\t}"
                    : "=r"(ok)
                    : "r"(bar), "r"(parity)
                    : "memory");
                if (!ok && (spin & 255u) == 255u) {  // time limit, not an iteration count: a try_wait may suspend for a while
                    uint64_t now;
                    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                    if (t0 == 0) t0 = now;
                    else if (now - t0 > kBulkWaitNs) break;
                }
            }
            if (!ok) {
                *reinterpret_cast<volatile uint32_t *>(status) = 0x701u;
                __threadfence_system();
                fine = false;
                break;
            }
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(st_dst[w][s]),
                         "r"(xc_smem_u32(ring + (size_t)s * piece)), "r"(st_len[w][s])
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            stored++;
        }
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// One WARP per (item, unit); a CTA of 8 warps walks the units of its item. The unit is read once when it fits in
// the lanes' registers (unit <= 512 elements with 16-byte loads), else twice (the second pass hits L1 / L2):
// absolute maximum by warp shuffles, then scale + round + 8-byte stores to the (peer) destination.
// mode 0: int8, q = rint(x * 127 / amax), dequant factor amax / 127 written to scale[unitIndex]
// mode 1: fp8 e4m3 (satfinite), q = x * 448 / amax, dequant factor amax / 448
// Vector path: source 16-byte aligned, destination 8-byte aligned, unit a multiple of 8; anything else takes
// the element-wise path of the same warp layout.
template <typename In> __device__ __forceinline__ float to_f32(In v);
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename In> __device__ __forceinline__ void unpack8(const uint4 &raw, float *f)
{
    const In *h = reinterpret_cast<const In *>(&raw);
#pragma unroll
    for (int k = 0; k < 8; k++) f[k] = to_f32<In>(h[k]);
}

template <int MODE> __device__ __forceinline__ uint8_t quant1(float x, float mul)
{
    if (MODE == 0) {
        const float q = fminf(127.f, fmaxf(-127.f, rintf(x * mul)));
        return (uint8_t)(int8_t)q;
    }
    return (uint8_t)__nv_cvt_float_to_fp8(x * mul, __NV_SATFINITE, __NV_E4M3);
}

template <int MODE> __device__ __forceinline__ uint2 quant8(const float *f, float mul)
{
    uint32_t lo = 0, hi = 0;
    if (MODE == 1) {
        // two values per conversion instruction (cvt.rn.satfinite.e4m3x2.f32)
#pragma unroll
        for (int k = 0; k < 2; k++) {
            lo |= (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(f[2 * k] * mul, f[2 * k + 1] * mul), __NV_SATFINITE, __NV_E4M3) << (16 * k);
            hi |= (uint32_t)__nv_cvt_float2_to_fp8x2(make_float2(f[4 + 2 * k] * mul, f[5 + 2 * k] * mul), __NV_SATFINITE, __NV_E4M3) << (16 * k);
        }
        return make_uint2(lo, hi);
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
        lo |= (uint32_t)quant1<MODE>(f[k], mul) << (8 * k);
        hi |= (uint32_t)quant1<MODE>(f[4 + k], mul) << (8 * k);
    }
    return make_uint2(lo, hi);
}

template <typename In, int MODE>
__global__ void __launch_bounds__(256) mf_xcopy_quant_kernel(const QuantItem *__restrict__ items, uint32_t unit)
{
    __shared__ QuantItem it;
    if (threadIdx.x == 0) it = items[blockIdx.y];
    __syncthreads();
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint64_t units = (it.elems + unit - 1) / unit;
    const In *src = reinterpret_cast<const In *>(it.src);
    uint8_t *dst = reinterpret_cast<uint8_t *>(it.dst);
    float *scales = reinterpret_cast<float *>(it.scale);
    const float qmax = MODE == 0 ? 127.f : 448.f;
    const bool vec = (unit % 8) == 0 && (it.src & 15) == 0 && (it.dst & 7) == 0;
    // Lanes per unit: a unit of up to 128 elements is 16 vectors, so two units share a warp. Each group of lanes
    // works on J units per step, all loads issued before the first reduction (latency hiding).
    const uint32_t W = (vec && unit <= 128) ? 16u : 32u;
    const uint32_t upw = 32u / W, sub = lane / W, sl = lane % W;
    constexpr int J = 2;
    const uint64_t per_cta = 8ull * upw * J;
    for (uint64_t base = (uint64_t)blockIdx.x * per_cta + (uint64_t)warp * upw * J; base < units; base += (uint64_t)gridDim.x * per_cta) {
        uint64_t ub[J], ue[J], nv[J];
        uint4 keep[J][2];
        float amax[J], f[8];
#pragma unroll
        for (int j = 0; j < J; j++) {
            const uint64_t u = base + (uint64_t)j * upw + sub;
            const bool on = u < units;
            ub[j] = on ? u * unit : 0;
            ue[j] = on ? min(it.elems, ub[j] + (uint64_t)unit) : 0;   // off: an empty range, the lanes only take part in the shuffles
            nv[j] = vec ? (ue[j] - ub[j]) / 8 : 0;                     // whole 8-element vectors of this unit
            const uint4 *src16 = reinterpret_cast<const uint4 *>(src + ub[j]);
            amax[j] = 0.f;
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const uint64_t v = sl + (uint64_t)W * i;
                if (v < nv[j]) {
                    keep[j][i] = __ldg(src16 + v);
                    unpack8<In>(keep[j][i], f);
#pragma unroll
                    for (int k = 0; k < 8; k++) amax[j] = fmaxf(amax[j], fabsf(f[k]));
                }
            }
            for (uint64_t v = sl + 2ull * W; v < nv[j]; v += W) {
                unpack8<In>(__ldg(src16 + v), f);
#pragma unroll
                for (int k = 0; k < 8; k++) amax[j] = fmaxf(amax[j], fabsf(f[k]));
            }
            for (uint64_t k = ub[j] + nv[j] * 8 + sl; k < ue[j]; k += W) amax[j] = fmaxf(amax[j], fabsf(to_f32<In>(src[k])));
        }
#pragma unroll
        for (int j = 0; j < J; j++)
            for (uint32_t o = W / 2; o > 0; o >>= 1) amax[j] = fmaxf(amax[j], __shfl_xor_sync(0xffffffffu, amax[j], o));
#pragma unroll
        for (int j = 0; j < J; j++) {
            const float mul = amax[j] > 0.f ? qmax / amax[j] : 1.f;
            if (sl == 0 && ue[j] > ub[j]) scales[ub[j] / unit] = amax[j] > 0.f ? amax[j] / qmax : 1.f;
            const uint4 *src16 = reinterpret_cast<const uint4 *>(src + ub[j]);
            uint2 *dst8 = reinterpret_cast<uint2 *>(dst + ub[j]);
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const uint64_t v = sl + (uint64_t)W * i;
                if (v < nv[j]) {
                    unpack8<In>(keep[j][i], f);
                    dst8[v] = quant8<MODE>(f, mul);
                }
            }
            for (uint64_t v = sl + 2ull * W; v < nv[j]; v += W) {
                unpack8<In>(__ldg(src16 + v), f);
                dst8[v] = quant8<MODE>(f, mul);
            }
            for (uint64_t k = ub[j] + nv[j] * 8 + sl; k < ue[j]; k += W) dst[k] = quant1<MODE>(to_f32<In>(src[k]), mul);
        }
    }
}

// Fast path of the quantising copy for the common shape: units of 128 elements, source 16-byte aligned, destination
// 8-byte aligned, element count a multiple of 128. A half-warp (16 lanes x 16 bytes = one unit per load instruction)
// takes EIGHT consecutive units per step: eight independent loads per lane are in flight before the first reduction,
// the eight maxima are reduced by interleaved shuffles, the eight factors leave as two 16-byte stores. The kernel above
// keeps two loads per lane in flight and is bound by the latency of each step, not by memory or instruction issue.
template <typename In, int MODE>
__global__ void __launch_bounds__(256) mf_xcopy_quant128_kernel(const QuantItem *__restrict__ items)
{
    __shared__ QuantItem it;
    if (threadIdx.x == 0) it = items[blockIdx.y];
    __syncthreads();
    constexpr int J = 8;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t sub = lane >> 4, sl = lane & 15;
    const uint64_t units = it.elems / 128;
    const uint4 *src = reinterpret_cast<const uint4 *>(it.src);   // 16 vectors per unit
    uint2 *dst = reinterpret_cast<uint2 *>(it.dst);               // 16 x 8 bytes per unit
    float *scales = reinterpret_cast<float *>(it.scale);
    const float qmax = MODE == 0 ? 127.f : 448.f;
    const bool s16 = (it.scale & 15) == 0;
    const uint64_t per_cta = 8ull * 2 * J;  // warps x half-warps x units
    for (uint64_t base = (uint64_t)blockIdx.x * per_cta + ((uint64_t)warp * 2 + sub) * J; base < units; base += (uint64_t)gridDim.x * per_cta) {
        uint4 raw[J];
        float amax[J];
#pragma unroll
        for (int j = 0; j < J; j++) {
            const uint64_t u = base + j;
            raw[j] = u < units ? __ldcs(src + u * 16 + sl) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int j = 0; j < J; j++) {
            float f[8];
            unpack8<In>(raw[j], f);
            float m = 0.f;
#pragma unroll
            for (int k = 0; k < 8; k++) m = fmaxf(m, fabsf(f[k]));
            amax[j] = m;
        }
#pragma unroll
        for (uint32_t o = 8; o > 0; o >>= 1) {
#pragma unroll
            for (int j = 0; j < J; j++) amax[j] = fmaxf(amax[j], __shfl_xor_sync(0xffffffffu, amax[j], o));
        }
        float fac[J];
#pragma unroll
        for (int j = 0; j < J; j++) {
            const float mul = amax[j] > 0.f ? qmax / amax[j] : 1.f;
            fac[j] = amax[j] > 0.f ? amax[j] / qmax : 1.f;
            const uint64_t u = base + j;
            if (u < units) {
                float f[8];
                unpack8<In>(raw[j], f);
                __stcs(dst + u * 16 + sl, quant8<MODE>(f, mul));
            }
        }
        // the eight factors of this half-warp are consecutive in the factor array
        if (s16 && base + J <= units) {
            if (sl < 2) reinterpret_cast<float4 *>(scales + base)[sl] = sl == 0 ? make_float4(fac[0], fac[1], fac[2], fac[3]) : make_float4(fac[4], fac[5], fac[6], fac[7]);
        } else if (sl == 0) {
#pragma unroll
            for (int j = 0; j < J; j++)
                if (base + j < units) scales[base + j] = fac[j];
        }
    }
}

}  // namespace mfk
