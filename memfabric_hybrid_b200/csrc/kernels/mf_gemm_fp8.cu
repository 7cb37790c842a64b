// Grouped expert GEMM in fp8 e4m3 with DeepSeek-style block scales on the 5th-generation tensor cores:
//   activations A [rows, K] fp8, one fp32 scale per row per 128 elements of K        (1 x 128)
//   weights     B [experts, N, K] fp8, one fp32 scale per 128 x 128 block            (128 x 128)
//   rows are grouped by expert: group g owns rows [row_off[g], row_off[g+1]) (device array, no host sync)
// Each 128-wide K block is multiplied by tcgen05.mma (kind::f8f6f4, fp32 accumulate) into its own TMEM
// buffer; the epilogue warps read it back, multiply by (row scale x block scale) and add it to fp32
// accumulators in registers, while the tensor core already works on the next K block (four TMEM
// buffers rotate). Operands arrive by TMA from THIS GPU's memory (the dispatch kernel has stored peers'
// tokens here before); no load touches a peer.
// Epilogues:
//   EPI 1  gate/up + SwiGLU : B is tile-interleaved (64 gate rows, 64 up rows per 128); out[row, 64 cols] =
//                             silu(gate) * up, bf16
//   EPI 2  down + combine   : out row x routing weight is stored straight into the combine slot of the
//                             token's home rank (peer stores over NVLink): the weighted all-to-all back is
//                             the epilogue of this GEMM
//   EPI 0  plain            : bf16 rows to local memory
// Parity of role: app/zbal/src/csrc/operators/npu/aicore/ops/fused_deep_moe/* (GMM1 + dequant + SwiGLU,
// GMM2 + dequant + combine) of the reference.
#include <cuda_bf16.h>

#include "mf_gemm.cuh"
#include "mf_team.cuh"

namespace mfk {

constexpr int FBN = 128;       // tile columns
constexpr int FSTAGES = 6;     // 32 KiB per stage
constexpr int kAccBufs = 4;    // TMEM buffers of FBN columns
constexpr int kMaxGroups = 64;

struct Fp8Args {
    TmaPair tm;                // A: [rows, K] fp8; B: [G * N, K] fp8
    const float *a_scale;      // [rows, K/128]
    const float *b_scale;      // [G, N/128, K/128]  (N in ORIGINAL row order: for EPI 1 gate rows then up rows)
    const int *row_off;        // [G + 1] device
    int G, N, K;               // N: rows of B per group (EPI 1: 2 x intermediate)
    int max_rows;              // rows of the A buffer (upper bound on row_off[G])
    __nv_bfloat16 *out;        // EPI 0/1 output
    int64_t ldo;
    int *status;
    // EPI 2
    Team team;
    const int4 *recv_info;     // [rows] {source rank, token, k slot, weight bits}
    uint64_t comb_off;         // slot offset of the combine slots [T * topk][N] bf16
    int topk;
};

constexpr int kFp8Threads = 64 + 8 * 32;  // TMA warp, MMA warp, eight epilogue warps

template <int EPI> __global__ void __launch_bounds__(kFp8Threads, 1) k_grouped_fp8(const __grid_constant__ Fp8Args g)
{
    extern __shared__ uint8_t smem_raw[];
    GemmSmem<FBN, FSTAGES> sm(smem_raw);
    __shared__ int tile_start[kMaxGroups + 1];  // first linear tile of every group
    __shared__ int s_row_off[kMaxGroups + 1];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_tiles = g.N / FBN;
    const int k_blocks = g.K / 128;
    AbortCtl ac{sm.abort_flag(), g.status};

    // barriers: full/empty per smem stage; tfull/tempty per TMEM buffer (GemmSmem has room for 4 + 4)
    if (threadIdx.x == 0) {
        *sm.abort_flag() = 0;
        for (int s = 0; s < FSTAGES; s++) {
            mbar_init(sm.full(s), 1);
            mbar_init(sm.empty(s), 1);
        }
        for (int i = 0; i < kAccBufs; i++) {
            mbar_init(sm.tfull(i), 1);
            mbar_init(sm.tempty(i), 8);
        }
        mbar_fence_init();
        tma_prefetch_desc(&g.tm.a);
        tma_prefetch_desc(&g.tm.b);
        int run = 0;
        for (int i = 0; i <= g.G; i++) {
            const int ro = min(g.row_off[i], g.max_rows);
            s_row_off[i] = ro;
            tile_start[i] = run;
            if (i < g.G) run += ((min(g.row_off[i + 1], g.max_rows) - ro + BM - 1) / BM) * n_tiles;
        }
    }
    if (warp == 1) {
        tmem_alloc(sm.tmem_slot(), kAccBufs * FBN);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *sm.tmem_slot();
    const int total = tile_start[g.G];

    // linear tile -> (group, first row, row limit, column tile); inside a group the row tile varies fastest
    auto locate = [&](int t, int &grp, int &row0, int &row_end, int &nt) {
        int lo = 0;
        while (lo + 1 < g.G && tile_start[lo + 1] <= t) lo++;
        grp = lo;
        const int local = t - tile_start[lo];
        const int mt_cnt = (s_row_off[lo + 1] - s_row_off[lo] + BM - 1) / BM;
        nt = local / mt_cnt;
        row0 = s_row_off[lo] + (local % mt_cnt) * BM;
        row_end = s_row_off[lo + 1];
    };

    if (warp == 0) {
        if (elect_one()) {
            PipeState ps;
            bool fine = true;
            for (int t = blockIdx.x; t < total && fine; t += gridDim.x) {
                int grp, row0, row_end, nt;
                locate(t, grp, row0, row_end, nt);
                for (int kb = 0; kb < k_blocks; kb++) {
                    fine = mbar_wait(sm.empty(ps.stage), ps.phase ^ 1, ac, 0x502);
                    if (!fine) break;
                    mbar_expect_tx(sm.full(ps.stage), GemmSmem<FBN, FSTAGES>::kStageBytes);
                    tma_load_2d(sm.a(ps.stage), &g.tm.a, kb * 128, row0, sm.full(ps.stage));
                    tma_load_2d(sm.b(ps.stage), &g.tm.b, kb * 128, grp * g.N + nt * FBN, sm.full(ps.stage));
                    ps.advance<FSTAGES>();
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            PipeState ps;
            int buf = 0;
            uint32_t buf_phase = 0;
            const uint32_t idesc = umma_idesc(0, 0, BM, FBN);  // e4m3 x e4m3
            bool fine = true;
            for (int t = blockIdx.x; t < total && fine; t += gridDim.x) {
                for (int kb = 0; kb < k_blocks; kb++) {
                    fine = mbar_wait(sm.tempty(buf), buf_phase ^ 1, ac, 0x503);
                    if (!fine) break;
                    fine = mbar_wait(sm.full(ps.stage), ps.phase, ac, 0x504);
                    if (!fine) break;
                    tc_fence_after();
                    const uint32_t d = tmem_base + (uint32_t)(buf * FBN);
                    const uint64_t da = umma_desc_sw128(sm.a(ps.stage));
                    const uint64_t db = umma_desc_sw128(sm.b(ps.stage));
#pragma unroll
                    for (int k = 0; k < 4; k++)  // 32 bytes = 32 fp8 = one UMMA K step
                        umma_fp8(d, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, k != 0);
                    umma_commit(sm.empty(ps.stage));
                    umma_commit(sm.tfull(buf));
                    ps.advance<FSTAGES>();
                    if (++buf == kAccBufs) {
                        buf = 0;
                        buf_phase ^= 1;
                    }
                }
            }
        }
    } else {
        // eight epilogue warps: warp w reads TMEM lane quadrant w % 4 (the hardware's rule) and one half of
        // the tile's columns, so a thread carries 64 fp32 accumulators and the per-K-block promotion
        // (TMEM -> registers, x scale, add) is spread over twice the threads of a 4-warp epilogue.
        // EPI 1 keeps a gate column and its up column in the same thread: half h owns gate columns
        // [32h, 32h+32) and up columns [64+32h, 64+32h+32).
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;
        const int col0 = EPI == 1 ? half * 32 : half * 64;
        const int col1 = EPI == 1 ? 64 + half * 32 : half * 64 + 32;
        int buf = 0;
        uint32_t buf_phase = 0;
        const int kgroups = g.K / 128;
        const int nblocks = g.N / 128;
        using SM = GemmSmem<FBN, FSTAGES>;
        constexpr int kRowB = 80;  // staged row: 64 bytes of bf16 + 16 of padding (conflict-free 16-byte writes)
        uint8_t *stg = sm.out_stage(0) + (warp - 2) * (32 * kRowB);
        static_assert(8 * 32 * kRowB <= SM::kOutBytes, "epilogue staging does not fit");
        for (int t = blockIdx.x; t < total; t += gridDim.x) {
            int grp, row0, row_end, nt;
            locate(t, grp, row0, row_end, nt);
            const int row = row0 + quad * 32 + lane;
            const bool row_ok = row < row_end;
            const float *as = g.a_scale + (int64_t)(row_ok ? row : row0) * kgroups;
            // block-scale rows of B that this tile's columns fall into
            int nb0, nb1;
            if (EPI == 1) {
                nb0 = (nt * 64) / 128;                  // gate rows nt*64 .. +64
                nb1 = (g.N / 2 + nt * 64) / 128;        // up rows N/2 + nt*64 .. +64
            } else {
                nb0 = nb1 = nt;
            }
            const float *bs0 = g.b_scale + ((int64_t)grp * nblocks + nb0) * kgroups;
            const float *bs1 = g.b_scale + ((int64_t)grp * nblocks + nb1) * kgroups;
            float acc[64];
#pragma unroll
            for (int i = 0; i < 64; i++) acc[i] = 0.f;
            bool fine = true;
            for (int kb = 0; kb < k_blocks; kb++) {
                fine = __all_sync(0xffffffffu, mbar_wait(sm.tfull(buf), buf_phase, ac, 0x505));
                if (!fine) break;
                tc_fence_after();
                const float sa = __ldg(as + kb);
                const float s0 = sa * __ldg(bs0 + kb), s1 = sa * __ldg(bs1 + kb);
                const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * FBN);
                uint32_t v0[32], v1[32];
                tmem_ld32(taddr + (uint32_t)col0, v0);   // both loads in flight before the wait
                tmem_ld32(taddr + (uint32_t)col1, v1);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(sm.tempty(buf));  // the data is in registers: the tensor core may reuse the buffer
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    acc[j] = fmaf(__uint_as_float(v0[j]), s0, acc[j]);
                    acc[32 + j] = fmaf(__uint_as_float(v1[j]), s1, acc[32 + j]);
                }
                if (++buf == kAccBufs) {
                    buf = 0;
                    buf_phase ^= 1;
                }
            }
            if (!fine) break;
            if (EPI == 1) {
                if (row_ok) {
                    __nv_bfloat16 *dst = g.out + (int64_t)row * g.ldo + nt * 64 + half * 32;
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        uint4 pk;
                        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const float g0 = acc[q * 8 + 2 * e], g1 = acc[q * 8 + 2 * e + 1];
                            const float u0 = acc[32 + q * 8 + 2 * e], u1 = acc[32 + q * 8 + 2 * e + 1];
                            h[e] = __floats2bfloat162_rn(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
                        }
                        *reinterpret_cast<uint4 *>(dst + q * 8) = pk;
                    }
                }
            } else {
                // rows leave through shared memory: lane = row on the way in, 4 lanes x 16 bytes per row on the
                // way out, so that one store instruction writes 8 rows x 64 contiguous bytes (peer stores of
                // 16-byte fragments are what made this epilogue slow)
                unsigned long long dst = 0;
                float w = 1.f;
                if (row_ok) {
                    if (EPI == 2) {
                        const int4 info = __ldg(g.recv_info + row);
                        w = __int_as_float(info.w);
                        dst = reinterpret_cast<unsigned long long>(reinterpret_cast<__nv_bfloat16 *>(peer_ptr(g.team, (uint32_t)info.x, g.comb_off)) +
                                                                   ((int64_t)info.y * g.topk + info.z) * g.N + nt * FBN + half * 64);
                    } else {
                        dst = reinterpret_cast<unsigned long long>(g.out + (int64_t)row * g.ldo + nt * FBN + half * 64);
                    }
                }
#pragma unroll
                for (int c = 0; c < 2; c++) {
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        uint4 pk;
                        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                        for (int e = 0; e < 4; e++) h[e] = __floats2bfloat162_rn(acc[c * 32 + q * 8 + 2 * e] * w, acc[c * 32 + q * 8 + 2 * e + 1] * w);
                        *reinterpret_cast<uint4 *>(stg + lane * kRowB + q * 16) = pk;
                    }
                    __syncwarp();
#pragma unroll
                    for (int it = 0; it < 4; it++) {
                        const int r = it * 8 + (lane >> 2);
                        const unsigned long long d = __shfl_sync(0xffffffffu, dst, r);
                        const uint4 val = *reinterpret_cast<const uint4 *>(stg + r * kRowB + (lane & 3) * 16);
                        if (d != 0) *reinterpret_cast<uint4 *>(d + (unsigned long long)(c * 64 + (lane & 3) * 16)) = val;
                    }
                    __syncwarp();
                }
            }
        }
    }
    if (EPI == 2) __threadfence_system();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kAccBufs * FBN);
    }
}

}  // namespace mfk

using namespace mfk;

namespace {
template <int EPI> int launch_fp8(const Fp8Args &g, int grid, cudaStream_t s)
{
    auto kern = k_grouped_fp8<EPI>;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<FBN, FSTAGES>::kDynBytes) != cudaSuccess) {
            (void)cudaGetLastError();
            return -2;
        }
        attr_set = true;
    }
    kern<<<grid, kFp8Threads, GemmSmem<FBN, FSTAGES>::kDynBytes, s>>>(g);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
}  // namespace

extern "C" {

// epi: 0 plain, 1 SwiGLU (out [rows, N/2]), 2 weighted push into the combine slots of the tokens' home ranks.
int mf_grouped_gemm_fp8(const void *A, const float *a_scale, int max_rows, const void *B, const float *b_scale, const int *row_off, int G,
                        int N, int K, void *out, int64_t ldo, int epi, const Team *team, const void *recv_info, uint64_t comb_off, int topk,
                        int *status, int sms, void *stream)
{
    if (G <= 0 || G > kMaxGroups || N <= 0 || K <= 0 || (N % FBN) != 0 || (K % 128) != 0 || max_rows <= 0) return -1;
    if (epi == 1 && (N / 2) % 64 != 0) return -1;
    if (epi == 2 && (team == nullptr || recv_info == nullptr)) return -1;
    Fp8Args g{};
    int rc = make_tmap_2d(&g.tm.a, A, 1, (uint64_t)max_rows, (uint64_t)K, (uint64_t)K, BM, true);
    if (rc == 0) rc = make_tmap_2d(&g.tm.b, B, 1, (uint64_t)G * N, (uint64_t)K, (uint64_t)K, FBN, true);
    if (rc != 0) return rc;
    g.a_scale = a_scale;
    g.b_scale = b_scale;
    g.row_off = row_off;
    g.G = G;
    g.N = N;
    g.K = K;
    g.max_rows = max_rows;
    g.out = static_cast<__nv_bfloat16 *>(out);
    g.ldo = ldo;
    g.status = status;
    if (team != nullptr) g.team = *team;
    g.recv_info = static_cast<const int4 *>(recv_info);
    g.comb_off = comb_off;
    g.topk = topk;
    cudaStream_t s = (cudaStream_t)stream;
    switch (epi) {
        case 0: return launch_fp8<0>(g, sms, s);
        case 1: return launch_fp8<1>(g, sms, s);
        case 2: return launch_fp8<2>(g, sms, s);
        default: return -1;
    }
}

}  // extern "C"
