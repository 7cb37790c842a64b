// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = A[M,K] . B[N,K]^T, fp32 accumulation in TMEM.
// Persistent kernel, one CTA per SM, two TMEM accumulators so that the epilogue of tile i overlaps the main loop of
// tile i+1. Two tilings (template parameter PAIR):
//   PAIR false: every CTA works alone on 128 x 256 tiles (cta_group::1), 4-stage TMA ring of 48 KiB stages.
//   PAIR true : the two CTAs of a cluster (the two SMs of one TPC) share one 256 x 256 tile (cta_group::2). Each CTA loads
//       its own 128 rows of A and its own 128 of the tile's 256 rows of B (half the B bytes per SM), 6 stages of 32 KiB.
//       The leader CTA's MMA thread issues the MMAs, which read both CTAs' shared memory and write 128 rows x 256 columns
//       of accumulators into EACH CTA's tensor memory; each CTA's epilogue warps store their own 128 rows. The pair form
//       of the TMA load counts its bytes on the LEADER's "full" barrier (every CTA fetches its own tiles; the leader's
//       producer expects the bytes of both); the leader commits each stage's MMAs to its own "empty" barrier and to the
//       peer's (two plain commits, the second on the peer's barrier address from mapa), likewise the accumulator's
//       "full" barrier; the peer's epilogue warps release the accumulator on the leader's barrier with a remote arrive.
//
// The same kernel carries the two tensor-parallel fusions (template parameter MODE):
//   MODE 1, all-gather -> GEMM : the A operand is a gather buffer in THIS GPU's slot of the symmetric
//       heap. Four extra "copy" warps per CTA push this rank's activation shard into every peer's
//       gather buffer with plain stores over NVLink and raise a per-shard ready flag there; the TMA
//       producer waits on the flag of the shard a tile's rows belong to before its first load, and
//       tiles are visited in the order in which shards arrive. No TMA load ever touches a peer's
//       memory, and none uses cluster multicast.
//   MODE 2, GEMM -> reduce-scatter : the epilogue sends each finished tile of partial sums to the rank
//       that owns those rows (peer stores into its landing zone) and bumps a per-tile arrival counter
//       there; when a CTA runs out of GEMM tiles it adds the W partial tiles of owned rows in a fixed
//       order, applies the scale and writes the output shard.
// EPI 1 fuses SwiGLU: B holds, per 256-row tile, 128 gate rows followed by their 128 up rows, and the
// epilogue writes silu(gate) * up (128 columns per tile).
#include <cuda_bf16.h>

#include <stdlib.h>

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
    Team team;
    uint32_t epoch;          // flag value of this call (grows by one per call)
    uint32_t seq;            // number of fused calls so far including this one (targets of the counters)
    // MODE 1
    const __nv_bfloat16 *x_local;  // this rank's shard [shard_rows, K]
    int64_t ldx;
    int shard_rows;
    uint64_t ag_buf_off;     // slot offset of the gather buffer [W * shard_rows, K]
    uint64_t ag_ready_off;   // slot offset of W ready flags (u32)
    uint32_t *push_count;    // local device counters [W], monotonic
    // MODE 2
    uint64_t rs_land_off;    // slot offset of the landing zone [W][rows_per_rank][N] bf16
    uint64_t rs_count_off;   // slot offset of per-owned-tile arrival counters (u32), monotonic
    int rows_per_rank;
    __nv_bfloat16 *y_out;    // [rows_per_rank, N]
    int64_t ldy;
    float scale;
};

constexpr int kCopyWarps = 4;

// Maps the t-th tile of this CTA's walk to (row tile, column tile).
// Row tiles are TM rows high (128, or 256 for a CTA pair).
template <int MODE, int BN, int TM> __device__ __forceinline__ void tile_mn(const GemmArgs &g, int t, int m_tiles, int n_tiles, int &mt, int &nt)
{
    if (MODE == 0) {
        // bands of 8 row tiles; inside a band the column varies slowest so that CTAs running together share B tiles
        const int band = 8;
        const int per_band = band * n_tiles;
        const int b = t / per_band;
        const int rows_in_band = min(band, m_tiles - b * band);
        const int r = t - b * per_band;
        nt = r / rows_in_band;
        mt = b * band + r % rows_in_band;
    } else {
        // blocks of rows owned by one rank, visited starting with this rank (MODE 1: the order in which shards
        // arrive) or with the next rank (MODE 2: remote owners first, own rows last)
        const int rows = MODE == 1 ? g.shard_rows : g.rows_per_rank;
        const int mt_per = rows / TM;
        const int per_block = mt_per * n_tiles;
        const int i = t / per_block;
        const int owner = (int)((g.team.rank + (MODE == 2 ? 1 : 0) + i) % g.team.world);
        const int r = t - i * per_block;
        nt = r / mt_per;
        mt = owner * mt_per + r % mt_per;
    }
}

template <int MODE, int EPI, int BN, int STAGES, bool PAIR>
__global__ void __launch_bounds__(kGemmThreads + (MODE == 1 ? kCopyWarps * 32 : 0), 1) k_gemm_bf16(const __grid_constant__ GemmArgs g)
{
    extern __shared__ uint8_t smem_raw[];
    using SM = GemmSmem<BN, STAGES, PAIR ? BN / 2 : BN>;
    constexpr int TM = PAIR ? 2 * BM : BM;  // rows of one tile
    SM sm(smem_raw);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t crank = PAIR ? cluster_ctarank() : 0;          // 0: the CTA that issues the MMAs
    const int walker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;  // tile walkers: CTAs, or CTA pairs
    const int walkers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int m_tiles = (g.M + TM - 1) / TM;
    const int n_tiles = (g.N + BN - 1) / BN;
    const int total = m_tiles * n_tiles;
    const int k_iters = (g.K * 2 + KSPAN - 1) / KSPAN;
    const uint32_t me = g.team.rank;
    AbortCtl ac{sm.abort_flag(), g.status};

    if (threadIdx.x == 0) {
        *sm.abort_flag() = 0;
        for (int s = 0; s < STAGES; s++) {
            mbar_init(sm.full(s), 1);
            mbar_init(sm.empty(s), 1);
        }
        for (int i = 0; i < 2; i++) {
            mbar_init(sm.tfull(i), 1);
            mbar_init(sm.tempty(i), PAIR ? 8 : 4);  // the epilogue warps of every CTA of the tile (counted in the leader)
        }
        mbar_fence_init();
        tma_prefetch_desc(&g.tm.a);
        tma_prefetch_desc(&g.tm.b);
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_pair(sm.tmem_slot(), 2 * BN);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(sm.tmem_slot(), 2 * BN);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // both CTAs' barriers are initialised and both halves of the tensor memory are allocated
    tc_fence_after();
    const uint32_t tmem_base = *sm.tmem_slot();

    if (warp == 0) {
        if (elect_one()) {
            PipeState ps;
            for (int t = walker; t < total; t += walkers) {
                int mt, nt;
                tile_mn<MODE, BN, TM>(g, t, m_tiles, n_tiles, mt, nt);
                if (MODE == 1) {
                    // the shard holding this tile's rows must have landed in this GPU's gather buffer
                    const int r = mt * TM / g.shard_rows;
                    const uint32_t *ready = reinterpret_cast<const uint32_t *>(peer_ptr(g.team, me, g.ag_ready_off)) + r;
                    if (!wait_flag(ready, g.epoch, g.team.spin_limit)) {
                        *ac.abort_smem = 1;
                        atomicCAS(g.status, 0, 0x301);
                        break;
                    }
                    asm volatile("fence.proxy.async.global;" ::: "memory");  // peers' generic-proxy stores before our TMA reads
                }
                bool fine = true;
                for (int kb = 0; kb < k_iters; kb++) {
                    fine = mbar_wait(sm.empty(ps.stage), ps.phase ^ 1, ac, 0x302);
                    if (!fine) break;
                    if (PAIR) {
                        // both CTAs' tiles are counted on the leader's barrier
                        if (crank == 0) mbar_expect_tx(sm.full(ps.stage), 2 * SM::kStageBytes);
                        const uint32_t lead_full = mapa_u32(smem_u32(sm.full(ps.stage)), 0);
                        tma_load_2d_pair(sm.a(ps.stage), &g.tm.a, kb * (KSPAN / 2), mt * TM + (int)crank * BM, lead_full);
                        tma_load_2d_pair(sm.b(ps.stage), &g.tm.b, kb * (KSPAN / 2), nt * BN + (int)crank * (BN / 2), lead_full);
                    } else {
                        mbar_expect_tx(sm.full(ps.stage), SM::kStageBytes);
                        tma_load_2d(sm.a(ps.stage), &g.tm.a, kb * (KSPAN / 2), mt * BM, sm.full(ps.stage));
                        tma_load_2d(sm.b(ps.stage), &g.tm.b, kb * (KSPAN / 2), nt * BN, sm.full(ps.stage));
                    }
                    ps.advance<STAGES>();
                }
                if (!fine) break;
            }
        }
    } else if (warp == 1) {
        if (crank == 0 && elect_one()) {
            PipeState ps;
            int acc = 0;
            uint32_t acc_phase = 0;
            const uint32_t idesc = umma_idesc(1, 1, TM, BN);
            bool fine = true;
            for (int t = walker; t < total && fine; t += walkers) {
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
                    for (int k = 0; k < KSPAN / 32; k++) {  // 32 bytes = 16 bf16 = one UMMA K step
                        if (PAIR) umma_bf16_pair(d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb | k) != 0);
                        else umma_bf16(d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb | k) != 0);
                    }
                    if (PAIR) {
                        // the stage is free in both CTAs once these MMAs have read it
                        const uint32_t e = smem_u32(sm.empty(ps.stage));
                        umma_commit_pair(e);
                        umma_commit_pair(mapa_u32(e, 1));
                    } else {
                        umma_commit(sm.empty(ps.stage));
                    }
                    ps.advance<STAGES>();
                }
                if (!fine) break;
                if (PAIR) {
                    const uint32_t f = smem_u32(sm.tfull(acc));
                    umma_commit_pair(f);
                    umma_commit_pair(mapa_u32(f, 1));
                } else {
                    umma_commit(sm.tfull(acc));
                }
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else if (warp < 6) {
        const int quad = warp & 3;  // TMEM lane quadrant this warp may read
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int t = walker; t < total; t += walkers) {
            int mt, nt;
            tile_mn<MODE, BN, TM>(g, t, m_tiles, n_tiles, mt, nt);
            if (PAIR) mt = 2 * mt + (int)crank;  // from here on: this CTA's 128-row tile
            // the whole warp must take the same branch: the TMEM loads below are warp-collective
            if (!__all_sync(0xffffffffu, mbar_wait(sm.tfull(acc), acc_phase, ac, 0x305))) break;
            tc_fence_after();
            const int row = mt * BM + quad * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN);
            if (EPI == 1) {
                // columns [0,128) of the tile are gate, [128,256) the matching up projections
#pragma unroll 1
                for (int c = 0; c < BN / 64; c++) {
                    uint32_t gt[32], up[32];
                    tmem_ld32(taddr + (uint32_t)(c * 32), gt);
                    tmem_ld32(taddr + (uint32_t)(BN / 2 + c * 32), up);
                    tmem_ld_wait();
                    const int col = nt * (BN / 2) + c * 32;
                    if (row < g.M && col < g.N / 2) {
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
            } else {
                __nv_bfloat16 *dst_row;
                if (MODE == 2) {
                    const int owner = mt * BM / g.rows_per_rank;
                    const int lrow = row - owner * g.rows_per_rank;
                    dst_row = reinterpret_cast<__nv_bfloat16 *>(peer_ptr(g.team, owner, g.rs_land_off)) +
                              ((int64_t)me * g.rows_per_rank + lrow) * g.N;
                } else {
                    dst_row = g.C + (int64_t)row * g.ldc;
                }
                const bool vec_ok = MODE == 2 ? (g.N & 7) == 0 : (g.ldc & 7) == 0;
                if (vec_ok && nt * BN + BN <= g.N) {
                    // full tile: 64 columns at a time through shared memory, so that every store instruction
                    // writes 4 rows x 128 contiguous bytes instead of 32 rows x 16 bytes (what counts on NVLink)
                    uint8_t *stg = sm.out_stage(warp - 2);
                    const int64_t ld = MODE == 2 ? (int64_t)g.N : g.ldc;
                    __nv_bfloat16 *tile_dst;
                    if (MODE == 2) {
                        const int owner = mt * BM / g.rows_per_rank;
                        tile_dst = reinterpret_cast<__nv_bfloat16 *>(peer_ptr(g.team, owner, g.rs_land_off)) +
                                   ((int64_t)me * g.rows_per_rank + (mt * BM + quad * 32 - owner * g.rows_per_rank)) * g.N;
                    } else {
                        tile_dst = g.C + (int64_t)(mt * BM + quad * 32) * g.ldc;
                    }
#pragma unroll 1
                    for (int c2 = 0; c2 < BN / 64; c2++) {
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
                                *reinterpret_cast<uint4 *>(stg + lane * SM::kOutRowBytes + half * 64 + q * 16) = pk;
                            }
                        }
                        __syncwarp();
                        const int col = nt * BN + c2 * 64 + (lane & 7) * 8;
#pragma unroll
                        for (int it = 0; it < 8; it++) {
                            const int r = it * 4 + (lane >> 3);
                            const uint4 val = *reinterpret_cast<const uint4 *>(stg + r * SM::kOutRowBytes + (lane & 7) * 16);
                            if (mt * BM + quad * 32 + r < g.M) *reinterpret_cast<uint4 *>(tile_dst + (int64_t)r * ld + col) = val;
                        }
                        __syncwarp();
                    }
                } else {
#pragma unroll 1
                for (int c = 0; c < BN / 32; c++) {
                    uint32_t v[32];
                    tmem_ld32(taddr + (uint32_t)(c * 32), v);
                    tmem_ld_wait();
                    const int col = nt * BN + c * 32;
                    if (row < g.M && col < g.N) {
                        __nv_bfloat16 *dst = dst_row + col;
                        if (col + 32 <= g.N && vec_ok) {
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
                }
            }
            tc_fence_before();
            if (MODE == 2) {
                // all four epilogue warps have stored their rows of the tile: tell the owner
                asm volatile("bar.sync 1, 128;" ::: "memory");  // orders all four warps' stores before the counting thread, whose fence + release publishes them
                if (warp == 2 && lane == 0) {
                    __threadfence_system();
                    const int owner = mt * BM / g.rows_per_rank;
                    const int ltile = (mt - owner * (g.rows_per_rank / BM)) * n_tiles + nt;
                    uint32_t *cnt = reinterpret_cast<uint32_t *>(peer_ptr(g.team, owner, g.rs_count_off)) + ltile;
                    asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
                }
            }
            __syncwarp();
            if (lane == 0) {
                // this CTA's half of the accumulator is out of tensor memory: tell the MMA thread (in the leader)
                if (!PAIR || crank == 0) mbar_arrive(sm.tempty(acc));
                else mbar_arrive_cluster(mapa_u32(smem_u32(sm.tempty(acc)), 0));
            }
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
    } else if (MODE == 1) {
        // copy warps: push rows [b*per, (b+1)*per) of the local shard to every rank's gather buffer, nearest
        // consumer first (own buffer, then rank me-1 which needs our shard second, ...)
        const int ct = threadIdx.x - kGemmThreads;  // 0..127
        const int per = (g.shard_rows + gridDim.x - 1) / gridDim.x;
        const int r0 = min(g.shard_rows, (int)blockIdx.x * per), r1 = min(g.shard_rows, r0 + per);
        const int vec_per_row = g.K / 8;  // 16-byte vectors per row
        for (uint32_t i = 0; i < g.team.world; i++) {
            const uint32_t p = (me + g.team.world - i) % g.team.world;
            __nv_bfloat16 *dst = reinterpret_cast<__nv_bfloat16 *>(peer_ptr(g.team, p, g.ag_buf_off)) + (int64_t)me * g.shard_rows * g.K;
            const int64_t nvec = (int64_t)(r1 - r0) * vec_per_row;
            constexpr int kStep = kCopyWarps * 32;
            int64_t v = ct;
            // eight independent 16-byte loads in flight per thread, then eight peer stores
            for (; v + 7 * kStep < nvec; v += 8 * kStep) {
                uint4 val[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int64_t q = v + u * kStep;
                    val[u] = __ldg(reinterpret_cast<const uint4 *>(g.x_local + (int64_t)(r0 + (int)(q / vec_per_row)) * g.ldx + (q % vec_per_row) * 8));
                }
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    const int64_t q = v + u * kStep;
                    *reinterpret_cast<uint4 *>(dst + (int64_t)(r0 + (int)(q / vec_per_row)) * g.K + (q % vec_per_row) * 8) = val[u];
                }
            }
            for (; v < nvec; v += kStep) {
                const int rr = r0 + (int)(v / vec_per_row);
                const int cc = (int)(v % vec_per_row) * 8;
                const uint4 val = __ldg(reinterpret_cast<const uint4 *>(g.x_local + (int64_t)rr * g.ldx + cc));
                *reinterpret_cast<uint4 *>(dst + (int64_t)rr * g.K + cc) = val;
            }
            asm volatile("bar.sync 2, 128;" ::: "memory");
            if (ct == 0) {
                // the CTA that completes the shard for peer p raises the flag there; this thread's fence covers the copy
                // warps' stores (ordered before it by the barrier), and the counter links the CTAs' fences together
                __threadfence_system();
                const uint32_t done = atomicAdd(g.push_count + p, 1u) + 1;
                if (done == gridDim.x * g.seq) {
                    __threadfence_system();
                    st_release_sys(reinterpret_cast<uint32_t *>(peer_ptr(g.team, p, g.ag_ready_off)) + me, g.epoch);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();  // nobody signals a barrier of a CTA that has left, and both halves are freed together
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) tmem_dealloc_pair(tmem_base, 2 * BN);
        else tmem_dealloc(tmem_base, 2 * BN);
    }
    if (MODE == 2) {
        // reduce the W partial tiles of every tile whose rows this rank owns
        __shared__ int ok_sh;
        const int own_tiles = (g.rows_per_rank / BM) * n_tiles;
        const uint32_t *cnt = reinterpret_cast<const uint32_t *>(peer_ptr(g.team, me, g.rs_count_off));
        const __nv_bfloat16 *land = reinterpret_cast<const __nv_bfloat16 *>(peer_ptr(g.team, me, g.rs_land_off));
        for (int t = blockIdx.x; t < own_tiles; t += gridDim.x) {
            if (threadIdx.x == 0) {
                ok_sh = (!*ac.abort_smem && wait_flag(cnt + t, g.team.world * g.seq, g.team.spin_limit)) ? 1 : 0;
                if (!ok_sh) atomicCAS(g.status, 0, 0x306);
            }
            __syncthreads();
            if (!ok_sh) break;
            const int ml = t / n_tiles, nt = t % n_tiles;
            const int cols = min(BN, g.N - nt * BN);
            const int vecs = BM * (cols / 8);
            for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
                const int lr = ml * BM + v / (cols / 8);
                const int col = nt * BN + (v % (cols / 8)) * 8;
                float accv[8];
#pragma unroll
                for (int e = 0; e < 8; e++) accv[e] = 0.f;
                // partials are fetched eight at a time (independent loads in flight), added in rank order
                for (uint32_t s0 = 0; s0 < g.team.world; s0 += 8) {
                    uint4 raw[8];
#pragma unroll
                    for (int u = 0; u < 8; u++)
                        if (s0 + u < g.team.world)
                            raw[u] = __ldcg(reinterpret_cast<const uint4 *>(land + ((int64_t)(s0 + u) * g.rows_per_rank + lr) * g.N + col));
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        if (s0 + u >= g.team.world) continue;
                        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw[u]);
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float2 f = __bfloat1622float2(h[e]);
                            accv[2 * e] += f.x;
                            accv[2 * e + 1] += f.y;
                        }
                    }
                }
                uint4 pk;
                __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                for (int e = 0; e < 4; e++) h[e] = __floats2bfloat162_rn(accv[2 * e] * g.scale, accv[2 * e + 1] * g.scale);
                *reinterpret_cast<uint4 *>(g.y_out + (int64_t)lr * g.ldy + col) = pk;
            }
            __syncthreads();
        }
    }
}

}  // namespace mfk

using namespace mfk;

namespace {
constexpr int kBN = 256, kStages = 4, kPairStages = 6;

template <int MODE, int EPI, bool PAIR> int launch_gemm(const GemmArgs &g, int grid, cudaStream_t s)
{
    using SM = GemmSmem<kBN, PAIR ? kPairStages : kStages, PAIR ? kBN / 2 : kBN>;
    static_assert(SM::kDynBytes <= 227 * 1024, "shared memory of the bf16 GEMM");
    auto kern = k_gemm_bf16<MODE, EPI, kBN, PAIR ? kPairStages : kStages, PAIR>;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SM::kDynBytes) != cudaSuccess) {
            (void)cudaGetLastError();
            return -2;
        }
        attr_set = true;
    }
    const int threads = kGemmThreads + (MODE == 1 ? kCopyWarps * 32 : 0);
    if (!PAIR) {
        kern<<<grid, threads, SM::kDynBytes, s>>>(g);
        cudaError_t e = cudaGetLastError();
        return e == cudaSuccess ? 0 : (int)e;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)grid);  // even: CTAs 2c and 2c + 1 form cluster c
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = SM::kDynBytes;
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

// MF_GEMM_PAIR: 0 never pairs, 1 pairs wherever the shape allows, unset: the library decides.
int pair_forced()
{
    static const int forced = [] {
        const char *e = getenv("MF_GEMM_PAIR");
        return e == nullptr || *e == 0 ? -1 : (atoi(e) != 0 ? 1 : 0);
    }();
    return forced;
}

int fill_common(GemmArgs &g, const void *A, const void *B, int M, int N, int K, int64_t lda, int64_t ldb, int *status, bool pair = false)
{
    if (M <= 0 || N <= 0 || K <= 0 || (K & 7) != 0) return -1;
    int rc = make_tmap_2d(&g.tm.a, A, 2, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, BM, false);
    if (rc == 0) rc = make_tmap_2d(&g.tm.b, B, 2, (uint64_t)N, (uint64_t)K, (uint64_t)ldb * 2, pair ? kBN / 2 : kBN, false);
    g.M = M;
    g.N = N;
    g.K = K;
    g.status = status;
    return rc;
}
}  // namespace

extern "C" {

// C = A[M,K] . B[N,K]^T (bf16, K contiguous) with one CTA per 128 x 256 tile. swiglu != 0: B is tile-interleaved (128 gate rows,
// 128 up rows per 256) and C is [M, N/2] = silu(gate) * up. status: device int, zero on entry; non-zero = a pipeline wait gave up.
int mf_gemm_bf16_one(const void *A, const void *B, void *C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int *status,
                     int sms, int swiglu, void *stream)
{
    GemmArgs g{};
    int rc = fill_common(g, A, B, M, N, K, lda, ldb, status);
    if (rc != 0) return rc;
    if (swiglu && (N % kBN) != 0) return -3;
    g.C = static_cast<__nv_bfloat16 *>(C);
    g.ldc = ldc;
    const int tiles = ((M + BM - 1) / BM) * ((N + kBN - 1) / kBN);
    const int grid = tiles < sms ? tiles : sms;
    return swiglu ? launch_gemm<0, 1, false>(g, grid, (cudaStream_t)stream) : launch_gemm<0, 0, false>(g, grid, (cudaStream_t)stream);
}

// The same product on CTA pairs (256 x 256 tiles). Needs at least two SMs.
int mf_gemm_bf16_pair(const void *A, const void *B, void *C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int *status,
                      int sms, int swiglu, void *stream)
{
    if (sms < 2) return -1;
    GemmArgs g{};
    int rc = fill_common(g, A, B, M, N, K, lda, ldb, status, true);
    if (rc != 0) return rc;
    if (swiglu && (N % kBN) != 0) return -3;
    g.C = static_cast<__nv_bfloat16 *>(C);
    g.ldc = ldc;
    const int tiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + kBN - 1) / kBN);
    const int grid = 2 * (tiles < sms / 2 ? tiles : sms / 2);
    return swiglu ? launch_gemm<0, 1, true>(g, grid, (cudaStream_t)stream) : launch_gemm<0, 0, true>(g, grid, (cudaStream_t)stream);
}

// The same product; picks the CTA-pair tiling (256 x 256 tiles on two SMs) when its tiles fill the
// SM pairs about as well as the 128 x 256 tiles fill the SMs, else the one-CTA kernel. MF_GEMM_PAIR=0 / 1 forces the choice.
int mf_gemm_bf16(const void *A, const void *B, void *C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int *status,
                 int sms, int swiglu, void *stream)
{
    const int forced = pair_forced();
    bool pair = forced == 1 && sms >= 2;
    if (forced < 0 && sms >= 2 && M > 0 && N > 0) {
        const long t1 = (long)((M + BM - 1) / BM) * ((N + kBN - 1) / kBN), s1 = sms;
        const long t2 = (long)((M + 2 * BM - 1) / (2 * BM)) * ((N + kBN - 1) / kBN), s2 = sms / 2;
        // share of the last wave's slots that do work, weighted by how much of each tile is inside the matrix
        const double fill1 = (double)M * N / ((double)((t1 + s1 - 1) / s1) * s1 * BM * kBN);
        const double fill2 = (double)M * N / ((double)((t2 + s2 - 1) / s2) * s2 * 2 * BM * kBN);
        pair = fill2 * 1.04 >= fill1;
    }
    if (pair) return mf_gemm_bf16_pair(A, B, C, M, N, K, lda, ldb, ldc, status, sms, swiglu, stream);
    return mf_gemm_bf16_one(A, B, C, M, N, K, lda, ldb, ldc, status, sms, swiglu, stream);
}

// All-gather -> GEMM. x_local [shard_rows, K] is this rank's sequence shard; the gather buffer
// [world * shard_rows, K] sits at ag_buf_off of every slot. C [world * shard_rows, N or N/2].
int mf_ag_gemm_bf16(const Team *team, const void *x_local, int64_t ldx, int shard_rows, const void *B, int64_t ldb, void *C, int64_t ldc,
                    int N, int K, uint64_t ag_buf_off, uint64_t ag_ready_off, uint32_t *push_count, uint32_t epoch, uint32_t seq,
                    int *status, int sms, int swiglu, void *stream)
{
    if (team == nullptr || shard_rows <= 0 || (shard_rows % BM) != 0 || team->emu) return -1;
    GemmArgs g{};
    const int M = shard_rows * (int)team->world;
    const void *A = reinterpret_cast<const void *>(team->heap_base + (uint64_t)team->rank * team->stride + ag_buf_off);
    // pairs need every shard to be whole 256-row tiles, and a grid of whole clusters
    const bool pair = pair_forced() != 0 && (shard_rows % (2 * BM)) == 0 && (sms & 1) == 0 && sms >= 2;
    int rc = fill_common(g, A, B, M, N, K, K, ldb, status, pair);
    if (rc != 0) return rc;
    if (swiglu && (N % kBN) != 0) return -3;
    g.C = static_cast<__nv_bfloat16 *>(C);
    g.ldc = ldc;
    g.team = *team;
    g.epoch = epoch;
    g.seq = seq;
    g.x_local = static_cast<const __nv_bfloat16 *>(x_local);
    g.ldx = ldx;
    g.shard_rows = shard_rows;
    g.ag_buf_off = ag_buf_off;
    g.ag_ready_off = ag_ready_off;
    g.push_count = push_count;
    // every CTA carries copy warps whose work peers wait for: the grid must be fully resident
    if (pair) return swiglu ? launch_gemm<1, 1, true>(g, sms, (cudaStream_t)stream) : launch_gemm<1, 0, true>(g, sms, (cudaStream_t)stream);
    return swiglu ? launch_gemm<1, 1, false>(g, sms, (cudaStream_t)stream) : launch_gemm<1, 0, false>(g, sms, (cudaStream_t)stream);
}

// GEMM -> reduce-scatter. A [M, K] (M = world * rows_per_rank), B [N, K]; y_out [rows_per_rank, N] = scale * sum over ranks.
int mf_gemm_rs_bf16(const Team *team, const void *A, int64_t lda, const void *B, int64_t ldb, void *y_out, int64_t ldy, int rows_per_rank,
                    int N, int K, uint64_t rs_land_off, uint64_t rs_count_off, uint32_t epoch, uint32_t seq, float scale, int *status,
                    int sms, void *stream)
{
    if (team == nullptr || rows_per_rank <= 0 || (rows_per_rank % BM) != 0 || (N & 7) != 0 || team->emu) return -1;
    GemmArgs g{};
    const int M = rows_per_rank * (int)team->world;
    const bool pair = pair_forced() != 0 && (rows_per_rank % (2 * BM)) == 0 && (sms & 1) == 0 && sms >= 2;
    int rc = fill_common(g, A, B, M, N, K, lda, ldb, status, pair);
    if (rc != 0) return rc;
    g.team = *team;
    g.epoch = epoch;
    g.seq = seq;
    g.rs_land_off = rs_land_off;
    g.rs_count_off = rs_count_off;
    g.rows_per_rank = rows_per_rank;
    g.y_out = static_cast<__nv_bfloat16 *>(y_out);
    g.ldy = ldy;
    g.scale = scale;
    return pair ? launch_gemm<2, 0, true>(g, sms, (cudaStream_t)stream) : launch_gemm<2, 0, false>(g, sms, (cudaStream_t)stream);
}

}  // extern "C"
