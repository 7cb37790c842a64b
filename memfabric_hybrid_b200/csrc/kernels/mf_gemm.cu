// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] . B[N,K]^T, fp32 accumulation in TMEM.
// Persistent kernel, one CTA per SM, 128 x 256 tiles, 4-stage TMA ring, two TMEM accumulators so that
// the epilogue of tile i overlaps the main loop of tile i+1.
//
// The same kernel carries the two tensor-parallel fusions:
//   all-gather -> GEMM : the A operand is a gather buffer in THIS GPU's memory that peers' copy warps
//                        fill shard by shard; the producer warp waits on a per-shard ready flag before
//                        the first TMA load of a tile whose rows belong to that shard (no TMA load ever
//                        touches a peer's memory)
//   GEMM -> reduce-scatter : the epilogue sends each finished 128-row x 256-col block of partial sums to
//                        the rank that owns those rows (plain peer stores into its landing zone), and the
//                        owner adds the W partial blocks in a fixed order
#include <cuda_bf16.h>

#include "mf_gemm.cuh"
#include "mf_team.cuh"

namespace mfk {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

int make_tmap_2d(CUtensorMap *out, const void *base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                 uint32_t box_rows, bool is_fp8)
{
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return -10;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (row_stride_bytes & 15) != 0) return -11;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {(cuuint32_t)(KSPAN / elem_bytes), box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapDataType dt = is_fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    CUresult r = fn(out, dt, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -12;
}

struct GemmArgs {
    TmaPair tm;
    __nv_bfloat16 *C;
    int64_t ldc;
    int M, N, K;
    int *status;
    // all-gather fusion (0 = off): rows [r * shard_rows, (r + 1) * shard_rows) of A become valid when
    // ready[r] >= epoch (flags in this GPU's memory, written by the gather kernel)
    const uint32_t *ready;
    uint32_t ready_epoch;
    int shard_rows;
    uint32_t spin_limit;
    // reduce-scatter fusion (0 = off): partial tiles are pushed to the owner of their rows
    Team team;
    uint64_t rs_land_off;   // slot offset of the landing zone [world][rows_per_rank][N] bf16... (see mf_tp.cu)
    int rs_rows_per_rank;
};

template <int BN, int STAGES> __global__ void __launch_bounds__(kGemmThreads, 1) k_gemm_bf16(const __grid_constant__ GemmArgs g)
{
    extern __shared__ uint8_t smem_raw[];
    GemmSmem<BN, STAGES> sm(smem_raw);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int m_tiles = (g.M + BM - 1) / BM;
    const int n_tiles = (g.N + BN - 1) / BN;
    const int total = m_tiles * n_tiles;
    const int k_iters = (g.K * 2 + KSPAN - 1) / KSPAN;
    AbortCtl ac{sm.abort_flag(), g.status};

    if (threadIdx.x == 0) {
        *sm.abort_flag() = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(sm.full(s), 1);
            mbar_init(sm.empty(s), 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(sm.tfull(i), 1);
            mbar_init(sm.tempty(i), 4);
        }
        mbar_fence_init();
        tma_prefetch_desc(&g.tm.a);
        tma_prefetch_desc(&g.tm.b);
    }
    if (warp == 1) {
        tmem_alloc(sm.tmem_slot(), 2 * BN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *sm.tmem_slot();

    // tile order: bands of 8 row-tiles, columns inside a band vary slowest, so CTAs running together share B tiles
    auto tile_mn = [&](int t, int &mt, int &nt) {
        const int band = 8;
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
            for (int t = blockIdx.x; t < total; t += gridDim.x) {
                int mt, nt;
                tile_mn(t, mt, nt);
                if (g.ready != nullptr) {
                    // every shard that this tile's rows touch must have landed in local memory
                    const int r0 = mt * BM / g.shard_rows, r1 = min(g.M - 1, mt * BM + BM - 1) / g.shard_rows;
                    bool ok = true;
                    for (int r = r0; r <= r1 && ok; r++) ok = wait_flag(g.ready + r, g.ready_epoch, g.spin_limit);
                    if (!ok) {
                        *ac.abort_smem = 1;
                        atomicCAS(g.status, 0, 0x301);
                        break;
                    }
                    fence_proxy_async_smem();
                    asm volatile("fence.proxy.async.global;" ::: "memory");  // generic-proxy stores -> TMA reads
                }
                bool fine = true;
                for (int kb = 0; kb < k_iters && fine; kb++) {
                    fine = mbar_wait(sm.empty(ps.stage), ps.phase ^ 1, ac, 0x302);
                    if (!fine) break;
                    mbar_expect_tx(sm.full(ps.stage), GemmSmem<BN, STAGES>::kStageBytes);
                    tma_load_2d(sm.a(ps.stage), &g.tm.a, kb * (KSPAN / 2), mt * BM, sm.full(ps.stage));
                    tma_load_2d(sm.b(ps.stage), &g.tm.b, kb * (KSPAN / 2), nt * BN, sm.full(ps.stage));
                    ps.advance<STAGES>();
                }
                if (!fine) break;
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            PipeState ps;
            int acc = 0;
            uint32_t acc_phase = 0;
            const uint32_t idesc = umma_idesc(1, 1, BM, BN);
            bool fine = true;
            for (int t = blockIdx.x; t < total && fine; t += gridDim.x) {
                fine = mbar_wait(sm.tempty(acc), acc_phase ^ 1, ac, 0x303);
                if (!fine) break;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < k_iters; kb++) {
                    fine = mbar_wait(sm.full(ps.stage), ps.phase, ac, 0x304);
                    if (!fine) break;
                    tc_fence_after();
                    const uint64_t da = umma_desc_sw128(sm.a(ps.stage));
                    const uint64_t db = umma_desc_sw128(sm.b(ps.stage));
#pragma unroll
                    for (int k = 0; k < KSPAN / 32; k++)  // 32 bytes = 16 bf16 = one UMMA K step
                        umma_bf16(d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb | k) != 0);
                    umma_commit(sm.empty(ps.stage));
                    ps.advance<STAGES>();
                }
                if (!fine) break;
                umma_commit(sm.tfull(acc));
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else {
        const int quad = warp & 3;  // TMEM lane quadrant this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int t = blockIdx.x; t < total; t += gridDim.x) {
            int mt, nt;
            tile_mn(t, mt, nt);
            // the whole warp must take the same branch: the TMEM loads below are warp-collective
            if (!__all_sync(0xffffffffu, mbar_wait(sm.tfull(acc), acc_phase, ac, 0x305))) break;
            tc_fence_after();
            const int row = mt * BM + quad * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
            for (int c = 0; c < BN / 32; c++) {
                uint32_t v[32];
                tmem_ld32(taddr + (uint32_t)(c * 32), v);
                tmem_ld_wait();
                const int col = nt * BN + c * 32;
                if (row < g.M && col < g.N) {
                    __nv_bfloat16 *dst = g.C + (int64_t)row * g.ldc + col;
                    if (col + 32 <= g.N && ((g.ldc & 7) == 0)) {
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            uint4 pk;
                            __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                            for (int e = 0; e < 4; e++)
                                h[e] = __floats2bfloat162_rn(__uint_as_float(v[q * 8 + 2 * e]), __uint_as_float(v[q * 8 + 2 * e + 1]));
                            *reinterpret_cast<uint4 *>(dst + q * 8) = pk;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; e++)
                            if (col + e < g.N) dst[e] = __float2bfloat16_rn(__uint_as_float(v[e]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sm.tempty(acc));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 2 * BN);
    }
}

}  // namespace mfk

using namespace mfk;

extern "C" {

// C[M,N] (bf16, row stride ldc) = A[M,K] . B[N,K]^T, all bf16 row-major with K contiguous.
// status: device int, must be zero on entry; non-zero afterwards means a pipeline wait gave up.
int mf_gemm_bf16(const void *A, const void *B, void *C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int *status,
                 int sms, void *stream)
{
    if (M <= 0 || N <= 0 || K <= 0 || (K & 7) != 0) return -1;
    constexpr int BN = 256, STAGES = 4;
    GemmArgs g{};
    int rc = make_tmap_2d(&g.tm.a, A, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, BM, false);
    if (rc == 0) rc = make_tmap_2d(&g.tm.b, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, BN, false);
    if (rc != 0) return rc;
    g.C = static_cast<__nv_bfloat16 *>(C);
    g.ldc = ldc;
    g.M = M;
    g.N = N;
    g.K = K;
    g.status = status;
    g.ready = nullptr;
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = tiles < sms ? tiles : sms;
    auto kern = k_gemm_bf16<BN, STAGES>;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<BN, STAGES>::kDynBytes) != cudaSuccess) return -2;
        attr_set = true;
    }
    kern<<<grid, kGemmThreads, GemmSmem<BN, STAGES>::kDynBytes, (cudaStream_t)stream>>>(g);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

}  // extern "C"
