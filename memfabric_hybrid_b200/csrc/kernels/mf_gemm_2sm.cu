// bf16 GEMM with CTA pairs (tcgen05 cta_group::2): C[M,N] = A[M,K] . B[N,K]^T, fp32 accumulation in TMEM.
//
// Two CTAs on the two SMs of one TPC form a cluster and work on ONE 256 x 256 tile: each CTA loads its own 128 rows of A
// and its own 128 of the tile's 256 rows of B (half the B bytes per SM of the one-CTA kernel in mf_gemm.cu), the leader
// CTA's MMA thread issues tcgen05.mma.cta_group::2, which reads both CTAs' shared memory and writes 128 rows x 256 columns of
// accumulators into EACH CTA's tensor memory; each CTA's epilogue warps store their own 128 rows.
//   * TMA loads carry the cta_group::2 form and count their bytes on the LEADER's "full" barrier (every CTA fetches its
//     own tiles); the leader's producer expects the bytes of both CTAs.
//   * The leader commits every stage's MMAs to its own "empty" barrier and to the peer's (two plain commits, the second
//     on the peer's barrier address obtained with mapa), likewise the accumulator's "full" barrier.
//   * The peer's epilogue warps release the accumulator on the leader's barrier with a remote mbarrier arrive.
// Persistent: cluster c takes tiles c, c + clusters, ...; two accumulators of 256 columns alternate, six stages of 32 KiB.
// Every wait is bounded (mf_umma.cuh); a wait that runs out raises the CTA's abort flag and the kernel returns.
// EPI 1 fuses SwiGLU (B holds, per 256-row tile, 128 gate rows followed by their 128 up rows).
#include <cuda_bf16.h>
#include <stdlib.h>

#include "mf_gemm.cuh"

namespace mfk {

constexpr int P_BN = 256;        // tile columns (both CTAs together)
constexpr int P_BHALF = 128;     // rows of B each CTA loads
constexpr int P_STAGES = 6;
constexpr int kPairThreads = 192;

struct PairSmem {
    static constexpr int kABytes = BM * KSPAN;
    static constexpr int kBBytes = P_BHALF * KSPAN;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarOff = P_STAGES * kStageBytes;
    static constexpr int kOutRowBytes = 144;
    static constexpr int kOutOff = kBarOff + 1024;
    static constexpr int kOutBytes = 4 * 32 * kOutRowBytes;
    static constexpr int kTotal = kOutOff + kOutBytes;
    static constexpr int kDynBytes = kTotal + 1024;
    uint8_t *base;
    __device__ explicit PairSmem(uint8_t *raw) : base(reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023)) {}
    __device__ uint8_t *a(int s) const { return base + s * kStageBytes; }
    __device__ uint8_t *b(int s) const { return base + s * kStageBytes + kABytes; }
    __device__ uint64_t *full(int s) const { return reinterpret_cast<uint64_t *>(base + kBarOff) + s; }
    __device__ uint64_t *empty(int s) const { return reinterpret_cast<uint64_t *>(base + kBarOff) + P_STAGES + s; }
    __device__ uint64_t *tfull(int i) const { return reinterpret_cast<uint64_t *>(base + kBarOff) + 2 * P_STAGES + i; }
    __device__ uint64_t *tempty(int i) const { return reinterpret_cast<uint64_t *>(base + kBarOff) + 2 * P_STAGES + 2 + i; }
    __device__ uint32_t *tmem_slot() const { return reinterpret_cast<uint32_t *>(base + kBarOff + 512); }
    __device__ volatile int *abort_flag() const { return reinterpret_cast<volatile int *>(base + kBarOff + 520); }
    __device__ uint8_t *out_stage(int epi_warp) const { return base + kOutOff + epi_warp * 32 * kOutRowBytes; }
};
static_assert(PairSmem::kDynBytes <= 227 * 1024, "shared memory of the paired bf16 GEMM");

struct PairArgs {
    CUtensorMap a;       // [M, K] bf16, box 128 rows
    CUtensorMap b;       // [N, K] bf16, box 128 rows (each CTA's half of a tile)
    __nv_bfloat16 *C;
    int64_t ldc;
    int M, N, K;
    int band;            // pair-rows per raster band
    int *status;
};

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `local` (a shared-memory address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local, uint32_t rank)
{
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// 2-D tile load of the CTA-pair form into this CTA's shared memory; the bytes are counted on the barrier at cluster address
// `bar_cluster` (the leader's). Every CTA fetches its own tiles.
__device__ __forceinline__ void tma_load_2d_pair(void *smem_dst, const CUtensorMap *m, int x, int y, uint32_t bar_cluster)
{
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(m), "r"(x), "r"(y), "r"(bar_cluster)
                 : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t *smem_result, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the barrier at `cluster_addr` (any CTA of the pair) once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr)
{
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr) : "memory");
}

template <int EPI> __global__ void __launch_bounds__(kPairThreads, 1) k_gemm_bf16_pair(const __grid_constant__ PairArgs g)
{
    extern __shared__ uint8_t smem_raw[];
    PairSmem sm(smem_raw);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();   // 0: leader (issues the MMAs)
    const int cluster_id = blockIdx.x >> 1, clusters = gridDim.x >> 1;
    const int m_tiles = (g.M + 2 * BM - 1) / (2 * BM);
    const int n_tiles = (g.N + P_BN - 1) / P_BN;
    const int total = m_tiles * n_tiles;
    const int k_iters = (g.K * 2 + KSPAN - 1) / KSPAN;
    AbortCtl ac{sm.abort_flag(), g.status};

    if (threadIdx.x == 0) {
        *sm.abort_flag() = 0;
        for (int s = 0; s < P_STAGES; s++) {
            mbar_init(sm.full(s), 1);
            mbar_init(sm.empty(s), 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(sm.tfull(i), 1);
            mbar_init(sm.tempty(i), 8);  // four epilogue warps of each CTA (used in the leader only)
        }
        mbar_fence_init();
        tma_prefetch_desc(&g.a);
        tma_prefetch_desc(&g.b);
    }
    if (warp == 1) {
        tmem_alloc_pair(sm.tmem_slot(), 2 * P_BN);
        tmem_relinquish_pair();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers are initialised and both halves of the tensor memory are allocated
    tc_fence_after();
    const uint32_t tmem_base = *sm.tmem_slot();

    // bands of g.band pair-rows; inside a band the column varies slowest so that clusters running together share B
    auto tile_mn = [&](int t, int &mt, int &nt) {
        const int band = g.band;
        const int per_band = band * n_tiles;
        const int b = t / per_band;
        const int rows_in_band = min(band, m_tiles - b * band);
        const int r = t - b * per_band;
        nt = r / rows_in_band;
        mt = b * band + r % rows_in_band;
    };

    if (warp == 0) {
        if (elect_one()) {
            PipeState ps;
            bool fine = true;
            for (int t = cluster_id; t < total && fine; t += clusters) {
                int mt, nt;
                tile_mn(t, mt, nt);
                for (int kb = 0; kb < k_iters; kb++) {
                    fine = mbar_wait(sm.empty(ps.stage), ps.phase ^ 1, ac, 0x702);
                    if (!fine) break;
                    if (rank == 0) mbar_expect_tx(sm.full(ps.stage), 2 * PairSmem::kStageBytes);  // both CTAs' tiles land on this barrier
                    const uint32_t lead_full = mapa_u32(smem_u32(sm.full(ps.stage)), 0);
                    tma_load_2d_pair(sm.a(ps.stage), &g.a, kb * (KSPAN / 2), mt * 2 * BM + (int)rank * BM, lead_full);
                    tma_load_2d_pair(sm.b(ps.stage), &g.b, kb * (KSPAN / 2), nt * P_BN + (int)rank * P_BHALF, lead_full);
                    ps.advance<P_STAGES>();
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0 && elect_one()) {
            PipeState ps;
            int acc = 0;
            uint32_t acc_phase = 0;
            const uint32_t idesc = umma_idesc(1, 1, 2 * BM, P_BN);
            bool fine = true;
            for (int t = cluster_id; t < total && fine; t += clusters) {
                fine = mbar_wait(sm.tempty(acc), acc_phase ^ 1, ac, 0x703);
                if (!fine) break;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(acc * P_BN);
                for (int kb = 0; kb < k_iters; kb++) {
                    fine = mbar_wait(sm.full(ps.stage), ps.phase, ac, 0x704);
                    if (!fine) break;
                    tc_fence_after();
                    const uint64_t da = umma_desc_sw128(sm.a(ps.stage));
                    const uint64_t db = umma_desc_sw128(sm.b(ps.stage));
#pragma unroll
                    for (int k = 0; k < KSPAN / 32; k++)  // 32 bytes = 16 bf16 = one UMMA K step
                        umma_bf16_pair(d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb | k) != 0);
                    // the stage is free in both CTAs once these MMAs have read it
                    const uint32_t e = smem_u32(sm.empty(ps.stage));
                    umma_commit_pair(e);
                    umma_commit_pair(mapa_u32(e, 1));
                    ps.advance<P_STAGES>();
                }
                if (!fine) break;
                const uint32_t f = smem_u32(sm.tfull(acc));
                umma_commit_pair(f);
                umma_commit_pair(mapa_u32(f, 1));
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else {
        const int quad = warp & 3;  // TMEM lane quadrant this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int t = cluster_id; t < total; t += clusters) {
            int mt, nt;
            tile_mn(t, mt, nt);
            if (!__all_sync(0xffffffffu, mbar_wait(sm.tfull(acc), acc_phase, ac, 0x705))) break;
            tc_fence_after();
            const int row0 = mt * 2 * BM + (int)rank * BM + quad * 32;
            const int row = row0 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * P_BN);
            if (EPI == 1) {
                // columns [0,128) of the tile are gate, [128,256) the matching up projections
#pragma unroll 1
                for (int c = 0; c < P_BN / 64; c++) {
                    uint32_t gt[32], up[32];
                    tmem_ld32(taddr + (uint32_t)(c * 32), gt);
                    tmem_ld32(taddr + (uint32_t)(P_BN / 2 + c * 32), up);
                    tmem_ld_wait();
                    const int col = nt * (P_BN / 2) + c * 32;
                    if (row < g.M && col + 32 <= g.N / 2) {
                        __nv_bfloat16 *dst = g.C + (int64_t)row * g.ldc + col;
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            uint4 pk;
                            __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const float g0 = __uint_as_float(gt[q * 8 + 2 * e]), g1 = __uint_as_float(gt[q * 8 + 2 * e + 1]);
                                const float u0 = __uint_as_float(up[q * 8 + 2 * e]), u1 = __uint_as_float(up[q * 8 + 2 * e + 1]);
                                h[e] = __floats2bfloat162_rn(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
                            }
                            *reinterpret_cast<uint4 *>(dst + q * 8) = pk;
                        }
                    }
                }
            } else if ((g.ldc & 7) == 0 && nt * P_BN + P_BN <= g.N) {
                // full tile: 64 columns at a time through shared memory, so that every store instruction writes 4 rows x
                // 128 contiguous bytes instead of 32 rows x 16 bytes
                uint8_t *stg = sm.out_stage(warp - 2);
                __nv_bfloat16 *tile_dst = g.C + (int64_t)row0 * g.ldc;
#pragma unroll 1
                for (int c2 = 0; c2 < P_BN / 64; c2++) {
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        uint32_t v[32];
                        tmem_ld32(taddr + (uint32_t)(c2 * 64 + half * 32), v);
                        tmem_ld_wait();
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            uint4 pk;
                            __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                            for (int e = 0; e < 4; e++)
                                h[e] = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 2 * e]), __uint_as_float(v[q * 8 + 2 * e + 1]));
                            *reinterpret_cast<uint4 *>(stg + lane * PairSmem::kOutRowBytes + half * 64 + q * 16) = pk;
                        }
                    }
                    __syncwarp();
                    const int col = nt * P_BN + c2 * 64 + (lane & 7) * 8;
#pragma unroll
                    for (int it = 0; it < 8; it++) {
                        const int r = it * 4 + (lane >> 3);
                        const uint4 val = *reinterpret_cast<const uint4 *>(stg + r * PairSmem::kOutRowBytes + (lane & 7) * 16);
                        if (row0 + r < g.M) *reinterpret_cast<uint4 *>(tile_dst + (int64_t)r * g.ldc + col) = val;
                    }
                    __syncwarp();
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < P_BN / 32; c++) {
                    uint32_t v[32];
                    tmem_ld32(taddr + (uint32_t)(c * 32), v);
                    tmem_ld_wait();
                    const int col = nt * P_BN + c * 32;
                    if (row < g.M && col < g.N) {
                        __nv_bfloat16 *dst = g.C + (int64_t)row * g.ldc + col;
#pragma unroll
                        for (int e = 0; e < 32; e++)
                            if (col + e < g.N) dst[e] = __float2bfloat16_rn(__uint_as_float(v[e]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                // the accumulator of this CTA's half is out of tensor memory: tell the leader's MMA thread
                const uint32_t e = smem_u32(sm.tempty(acc));
                if (rank == 0) mbar_arrive(sm.tempty(acc));
                else mbar_arrive_cluster(mapa_u32(e, 0));
            }
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // nobody signals a barrier of a CTA that has left, and both halves are free together
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, 2 * P_BN);
    }
}

}  // namespace mfk

using namespace mfk;

namespace {
// Pair-rows (256 rows of A each) per raster band; MF_GEMM_BAND overrides.
int pair_band()
{
    static int band = [] {
        const char *e = getenv("MF_GEMM_BAND");
        int v = e != nullptr ? atoi(e) : 8;
        return v >= 1 && v <= 64 ? v : 8;
    }();
    return band;
}

template <int EPI> int launch_pair(const PairArgs &g, int grid, cudaStream_t s)
{
    auto kern = k_gemm_bf16_pair<EPI>;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::kDynBytes) != cudaSuccess) {
            (void)cudaGetLastError();
            return -2;
        }
        attr_set = true;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kPairThreads);
    cfg.dynamicSmemBytes = PairSmem::kDynBytes;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, g);
    if (e != cudaSuccess) (void)cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
}  // namespace

extern "C" {

// C = A[M,K] . B[N,K]^T (bf16, K contiguous) on CTA pairs. swiglu != 0: B is tile-interleaved (128 gate rows, 128 up rows per
// 256) and C is [M, N/2] = silu(gate) * up. status: device int, zero on entry; non-zero = a pipeline wait gave up.
// Needs K % 8 == 0, 16-byte aligned operands with row strides that are multiples of 8 elements, and an even number of SMs.
int mf_gemm_bf16_pair(const void *A, const void *B, void *C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int *status,
                      int sms, int swiglu, void *stream)
{
    if (M <= 0 || N <= 0 || K <= 0 || (K & 7) != 0 || sms < 2) return -1;
    if (swiglu && (N % P_BN) != 0) return -3;
    PairArgs g{};
    int rc = make_tmap_2d(&g.a, A, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, BM, false);
    if (rc == 0) rc = make_tmap_2d(&g.b, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, P_BHALF, false);
    if (rc != 0) return rc;
    g.C = static_cast<__nv_bfloat16 *>(C);
    g.ldc = ldc;
    g.M = M;
    g.N = N;
    g.K = K;
    g.status = status;
    g.band = pair_band();
    const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + P_BN - 1) / P_BN);
    int grid = 2 * (tiles < sms / 2 ? tiles : sms / 2);
    return swiglu ? launch_pair<1>(g, grid, (cudaStream_t)stream) : launch_pair<0>(g, grid, (cudaStream_t)stream);
}

}  // extern "C"
