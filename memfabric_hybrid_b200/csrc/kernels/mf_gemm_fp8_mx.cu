// Grouped expert GEMM in fp8 e4m3 whose block scales are applied by the tensor core itself
// (tcgen05.mma kind::mxf8f6f4.block_scale): the whole K loop of a tile accumulates in ONE TMEM buffer and
// nothing is pulled out of TMEM per K block.
//   activations A [rows, K] fp8, one power-of-two fp32 scale per row per 128 elements of K      (1 x 128)
//   weights     B [experts, N, K] fp8, one power-of-two fp32 scale per 128 x 128 block          (128 x 128)
//   rows grouped by expert: group g owns rows [row_off[g], row_off[g+1]) (device array, no host sync)
// The scales must be powers of two (every quantiser of this library produces such scales): a producer
// warp turns them into UE8M0 bytes (the fp32 exponent) in the tensor core's scale layout in shared
// memory, four K blocks per 32-bit word; the MMA thread copies a group of them into TMEM (tcgen05.cp)
// and picks the byte of the current K block through the instruction descriptor.
// Tile 128 x 256 (48 KiB of operands per 128 of K: 3/4 of the L2 traffic per FLOP of a 128 x 128 tile),
// four TMA stages, operands from THIS GPU's memory only, no multicast.
// Warps: 0 TMA, 1 MMA (+ TMEM allocation), 2 scale producer, 4..11 epilogue (two per TMEM lane quadrant).
// The epilogue warps first move their part of the accumulator into registers and hand TMEM back, so the
// next tile's MMAs overlap the epilogue arithmetic and stores.
// Epilogues:
//   EPI 0  plain            : bf16 rows to local memory
//   EPI 1  gate/up + SwiGLU : B is tile-interleaved (128 gate rows, 128 up rows per 256); out[row, 128 cols] bf16
//   EPI 2  down + combine   : row x routing weight stored straight into the combine slot of the token's home
//                             rank (peer stores over NVLink)
//   EPI 3  gate/up + SwiGLU + re-quantisation: the 128 outputs of a tile row are one 1 x 128 block of the next
//                             GEMM's fp8 input: amax, power-of-two scale, e4m3 bytes and the scale are written
//                             here, so the activation never exists in bf16 in memory
// Parity of role: app/zbal/doc/fused_deep_moe.md:106-127,213-281 (GMM1 -> dequant + SwiGLU + dynamic re-quant
// -> GMM2 -> combine) of the reference.
#include <cuda_bf16.h>

#include "mf_fp8.cuh"
#include "mf_gemm.cuh"
#include "mf_team.cuh"

namespace mfk {

constexpr int XBN = 256;
constexpr int XSTAGES = 4;
constexpr int XSFBUFS = 4;
constexpr int kXThreads = 384;
constexpr int kXMaxGroups = 64;
constexpr int kXTmemCols = 512;
constexpr uint32_t kXSfaCol = 256;  // TMEM columns [256, 260): scales of A; [260, 268): scales of B
constexpr uint32_t kXSfbCol = 260;

struct XSmem {
    static constexpr int kABytes = BM * 128;
    static constexpr int kBBytes = XBN * 128;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kSfOff = XSTAGES * kStageBytes;
    static constexpr int kSfBufBytes = 512 + 1024;  // A chunk, two B chunks
    static constexpr int kBarOff = kSfOff + XSFBUFS * kSfBufBytes;
    static constexpr int kAmaxOff = kBarOff + 512;
    static constexpr int kOutOff = kBarOff + 512 + 2048;
    static constexpr int kOutRowB = 80;
    static constexpr int kOutBytes = 8 * 32 * kOutRowB;
    static constexpr int kTotal = kOutOff + kOutBytes;
    static constexpr int kDynBytes = kTotal + 1024;
    uint8_t *base;
    __device__ explicit XSmem(uint8_t *raw) : base(reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023)) {}
    __device__ uint8_t *a(int s) const { return base + s * kStageBytes; }
    __device__ uint8_t *b(int s) const { return base + s * kStageBytes + kABytes; }
    __device__ uint8_t *sf(int i) const { return base + kSfOff + i * kSfBufBytes; }
    __device__ uint64_t *bar(int i) const { return reinterpret_cast<uint64_t *>(base + kBarOff) + i; }
    __device__ uint64_t *full(int s) const { return bar(s); }
    __device__ uint64_t *empty(int s) const { return bar(XSTAGES + s); }
    __device__ uint64_t *sf_full(int i) const { return bar(2 * XSTAGES + i); }
    __device__ uint64_t *sf_empty(int i) const { return bar(2 * XSTAGES + XSFBUFS + i); }
    __device__ uint64_t *tfull() const { return bar(2 * XSTAGES + 2 * XSFBUFS); }
    __device__ uint64_t *tempty() const { return bar(2 * XSTAGES + 2 * XSFBUFS + 1); }
    __device__ uint32_t *tmem_slot() const { return reinterpret_cast<uint32_t *>(base + kBarOff + 256); }
    __device__ volatile int *abort_flag() const { return reinterpret_cast<volatile int *>(base + kBarOff + 264); }
    __device__ float *amax(int parity) const { return reinterpret_cast<float *>(base + kAmaxOff) + parity * 256; }
    __device__ uint8_t *out_stage(int epi_warp) const { return base + kOutOff + epi_warp * 32 * kOutRowB; }
};
static_assert(XSmem::kDynBytes <= 227 * 1024, "shared memory of the block-scaled fp8 GEMM");

struct XArgs {
    TmaPair tm;            // A: [rows, K] fp8; B: [G * N, K] fp8
    const float *a_scale;  // [rows, K/128]
    const float *b_scale;  // [G, N/128, K/128]  (N in ORIGINAL row order: for EPI 1/3 gate rows then up rows)
    const int *row_off;    // [G + 1] device
    int G, N, K;
    int max_rows;
    void *out;             // EPI 0/1: bf16; EPI 3: e4m3 bytes
    int64_t ldo;           // elements per output row
    float *out_scale;      // EPI 3: [rows, N/256]
    int *status;
    Team team;             // EPI 2
    const int4 *recv_info;
    uint64_t comb_off;
    int topk;
};

__device__ __forceinline__ void named_bar_sync(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

template <int EPI> __global__ void __launch_bounds__(kXThreads, 1) k_grouped_fp8_mx(const __grid_constant__ XArgs g)
{
    extern __shared__ uint8_t smem_raw[];
    XSmem sm(smem_raw);
    __shared__ int tile_start[kXMaxGroups + 1];
    __shared__ int s_row_off[kXMaxGroups + 1];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_tiles = g.N / XBN;
    const int k_blocks = g.K / 128;
    const int sf_groups = (k_blocks + 3) / 4;
    AbortCtl ac{sm.abort_flag(), g.status};

    if (threadIdx.x == 0) {
        *sm.abort_flag() = 0;
        for (int s = 0; s < XSTAGES; s++) {
            mbar_init(sm.full(s), 1);
            mbar_init(sm.empty(s), 1);
        }
        for (int i = 0; i < XSFBUFS; i++) {
            mbar_init(sm.sf_full(i), 32);
            mbar_init(sm.sf_empty(i), 1);
        }
        mbar_init(sm.tfull(), 1);
        mbar_init(sm.tempty(), 8);
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
        tmem_alloc(sm.tmem_slot(), kXTmemCols);
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
                    fine = mbar_wait(sm.empty(ps.stage), ps.phase ^ 1, ac, 0x602);
                    if (!fine) break;
                    mbar_expect_tx(sm.full(ps.stage), XSmem::kStageBytes);
                    tma_load_2d(sm.a(ps.stage), &g.tm.a, kb * 128, row0, sm.full(ps.stage));
                    tma_load_2d(sm.b(ps.stage), &g.tm.b, kb * 128, grp * g.N + nt * XBN, sm.full(ps.stage));
                    ps.advance<XSTAGES>();
                }
            }
        }
    } else if (warp == 1) {
        if (elect_one()) {
            PipeState ps, sf;
            uint32_t tphase = 0;
            bool fine = true;
            const uint32_t sfa = tmem_base + kXSfaCol, sfb = tmem_base + kXSfbCol;
            for (int t = blockIdx.x; t < total && fine; t += gridDim.x) {
                fine = mbar_wait(sm.tempty(), tphase ^ 1, ac, 0x603);  // the epilogue has taken the previous tile out of TMEM
                if (!fine) break;
                tphase ^= 1;
                for (int kb = 0; kb < k_blocks; kb++) {
                    if ((kb & 3) == 0) {
                        fine = mbar_wait(sm.sf_full(sf.stage), sf.phase, ac, 0x606);
                        if (!fine) break;
                        tc_fence_after();
                        const uint8_t *chunk = sm.sf(sf.stage);
                        tmem_cp_sf(sfa, umma_desc_sf(chunk));
                        tmem_cp_sf(sfb, umma_desc_sf(chunk + 512));
                        tmem_cp_sf(sfb + 4, umma_desc_sf(chunk + 1024));
                    }
                    fine = mbar_wait(sm.full(ps.stage), ps.phase, ac, 0x604);
                    if (!fine) break;
                    tc_fence_after();
                    const uint64_t da = umma_desc_sw128(sm.a(ps.stage));
                    const uint64_t db = umma_desc_sw128(sm.b(ps.stage));
                    const uint32_t idesc = umma_idesc_bs(BM, XBN, (uint32_t)(kb & 3), (uint32_t)(kb & 3));
#pragma unroll
                    for (int k = 0; k < 4; k++)  // 32 bytes = 32 fp8 = one UMMA K step
                        umma_fp8_bs(tmem_base, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb | k) != 0, sfa, sfb);
                    umma_commit(sm.empty(ps.stage));
                    ps.advance<XSTAGES>();
                    if ((kb & 3) == 3 || kb == k_blocks - 1) {
                        umma_commit(sm.sf_empty(sf.stage));  // the scale chunk has been copied and its MMAs are done
                        sf.advance<XSFBUFS>();
                    }
                }
                if (fine) umma_commit(sm.tfull());
            }
        }
    } else if (warp == 2) {
        // scale producer: lane l writes the 16 bytes of rows l, l + 32, l + 64, l + 96 (one 32-bit word of four
        // K-block scale bytes per row) and its share of the two B chunks
        PipeState sf;
        const int nblocks = g.N / 128;
        bool fine = true;
        for (int t = blockIdx.x; t < total && fine; t += gridDim.x) {
            int grp, row0, row_end, nt;
            locate(t, grp, row0, row_end, nt);
            int nb0, nb1;
            if (EPI == 1 || EPI == 3) {
                nb0 = nt;                  // gate rows nt * 128 .. + 128
                nb1 = nblocks / 2 + nt;    // up rows N/2 + nt * 128 .. + 128
            } else {
                nb0 = 2 * nt;
                nb1 = 2 * nt + 1;
            }
            const float *bs0 = g.b_scale + ((int64_t)grp * nblocks + nb0) * k_blocks;
            const float *bs1 = g.b_scale + ((int64_t)grp * nblocks + nb1) * k_blocks;
            for (int gq = 0; gq < sf_groups; gq++) {
                int ok = 1;
                if (lane == 0) ok = mbar_wait(sm.sf_empty(sf.stage), sf.phase ^ 1, ac, 0x607) ? 1 : 0;
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    fine = false;
                    break;
                }
                uint32_t wa[4], wb0 = 0, wb1 = 0;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int kb = gq * 4 + j;
                    const bool on = kb < k_blocks;
                    wb0 |= (on ? ue8m0_byte(__ldg(bs0 + kb)) : 127u) << (8 * j);
                    wb1 |= (on ? ue8m0_byte(__ldg(bs1 + kb)) : 127u) << (8 * j);
                }
#pragma unroll
                for (int r1 = 0; r1 < 4; r1++) {
                    const int row = min(row0 + r1 * 32 + lane, g.max_rows - 1);
                    const float *as = g.a_scale + (int64_t)row * k_blocks;
                    uint32_t w = 0;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int kb = gq * 4 + j;
                        w |= (kb < k_blocks ? ue8m0_byte(__ldg(as + kb)) : 127u) << (8 * j);
                    }
                    wa[r1] = w;
                }
                uint8_t *chunk = sm.sf(sf.stage);
                *reinterpret_cast<uint4 *>(chunk + lane * 16) = make_uint4(wa[0], wa[1], wa[2], wa[3]);
                *reinterpret_cast<uint4 *>(chunk + 512 + lane * 16) = make_uint4(wb0, wb0, wb0, wb0);
                *reinterpret_cast<uint4 *>(chunk + 1024 + lane * 16) = make_uint4(wb1, wb1, wb1, wb1);
                fence_proxy_async_smem();  // the tensor core's copy unit reads these bytes through the async proxy
                mbar_arrive(sm.sf_full(sf.stage));
                sf.advance<XSFBUFS>();
            }
        }
    } else if (warp >= 4) {
        // eight epilogue warps: warp w reads TMEM lane quadrant w % 4 (the hardware's rule); the two warps of a
        // quadrant split the tile's 256 columns
        const int quad = warp & 3;
        const int half = (warp - 4) >> 2;
        uint32_t tphase = 0;
        uint8_t *stg = sm.out_stage(warp - 4);
        constexpr int kRowB = XSmem::kOutRowB;
        for (int t = blockIdx.x; t < total; t += gridDim.x) {
            int grp, row0, row_end, nt;
            locate(t, grp, row0, row_end, nt);
            const int row = row0 + quad * 32 + lane;
            const bool row_ok = row < row_end;
            if (!__all_sync(0xffffffffu, mbar_wait(sm.tfull(), tphase, ac, 0x605))) break;
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16);
            uint32_t v[4][32];
            if (EPI == 1 || EPI == 3) {
                // a gate column and its up column in the same thread: half h owns gate [64h, 64h + 64), up [128 + 64h, ...)
                tmem_ld32(taddr + (uint32_t)(64 * half), v[0]);
                tmem_ld32(taddr + (uint32_t)(64 * half + 32), v[1]);
                tmem_ld32(taddr + (uint32_t)(128 + 64 * half), v[2]);
                tmem_ld32(taddr + (uint32_t)(128 + 64 * half + 32), v[3]);
            } else {
#pragma unroll
                for (int c = 0; c < 4; c++) tmem_ld32(taddr + (uint32_t)(128 * half + 32 * c), v[c]);
            }
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sm.tempty());  // the accumulator is in registers: the next tile may start
            if (EPI == 1 || EPI == 3) {
                float o[64];
#pragma unroll
                for (int c = 0; c < 2; c++)
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const float gt = __uint_as_float(v[c][j]), up = __uint_as_float(v[2 + c][j]);
                        o[c * 32 + j] = gt / (1.f + __expf(-gt)) * up;
                    }
                if (EPI == 1) {
                    if (row_ok) {
                        __nv_bfloat16 *dst = static_cast<__nv_bfloat16 *>(g.out) + (int64_t)row * g.ldo + nt * 128 + half * 64;
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            uint4 pk;
                            __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                            for (int e = 0; e < 4; e++) h[e] = __floats2bfloat162_rn(o[q * 8 + 2 * e], o[q * 8 + 2 * e + 1]);
                            *reinterpret_cast<uint4 *>(dst + q * 8) = pk;
                        }
                    }
                } else {
                    // the activation is rounded to bf16 first (the precision it would have had in memory), then
                    // quantised: the two warps of a quadrant exchange their maxima through shared memory
                    float amax = 0.f;
#pragma unroll
                    for (int j = 0; j < 64; j++) {
                        o[j] = __bfloat162float(__float2bfloat16_rn(o[j]));
                        amax = fmaxf(amax, fabsf(o[j]));
                    }
                    float *ex = sm.amax((int)tphase);
                    ex[(quad * 2 + half) * 32 + lane] = amax;
                    named_bar_sync(1 + quad, 64);
                    amax = fmaxf(amax, ex[(quad * 2 + (half ^ 1)) * 32 + lane]);
                    const float scale = pow2_scale_e4m3(amax);
                    const float mul = 1.f / scale;  // exact: a power of two
                    if (row_ok) {
                        uint8_t *dst = static_cast<uint8_t *>(g.out) + (int64_t)row * g.ldo + nt * 128 + half * 64;
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            uint4 pk;
                            pk.x = pack4_e4m3(o[q * 16 + 0], o[q * 16 + 1], o[q * 16 + 2], o[q * 16 + 3], mul);
                            pk.y = pack4_e4m3(o[q * 16 + 4], o[q * 16 + 5], o[q * 16 + 6], o[q * 16 + 7], mul);
                            pk.z = pack4_e4m3(o[q * 16 + 8], o[q * 16 + 9], o[q * 16 + 10], o[q * 16 + 11], mul);
                            pk.w = pack4_e4m3(o[q * 16 + 12], o[q * 16 + 13], o[q * 16 + 14], o[q * 16 + 15], mul);
                            *reinterpret_cast<uint4 *>(dst + q * 16) = pk;
                        }
                        if (half == 0) g.out_scale[(int64_t)row * (g.N / XBN) + nt] = scale;
                    }
                }
            } else {
                // rows leave through shared memory: lane = row on the way in, 4 lanes x 16 bytes per row on the way
                // out, so that one store instruction writes 8 rows x 64 contiguous bytes
                unsigned long long dst = 0;
                float w = 1.f;
                if (row_ok) {
                    if (EPI == 2) {
                        const int4 info = __ldg(g.recv_info + row);
                        w = __int_as_float(info.w);
                        dst = reinterpret_cast<unsigned long long>(reinterpret_cast<__nv_bfloat16 *>(peer_ptr(g.team, (uint32_t)info.x, g.comb_off)) +
                                                                   ((int64_t)info.y * g.topk + info.z) * g.N + nt * XBN + half * 128);
                    } else {
                        dst = reinterpret_cast<unsigned long long>(static_cast<__nv_bfloat16 *>(g.out) + (int64_t)row * g.ldo + nt * XBN + half * 128);
                    }
                }
#pragma unroll
                for (int c = 0; c < 4; c++) {
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        uint4 pk;
                        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                        for (int e = 0; e < 4; e++)
                            h[e] = __floats2bfloat162_rn(__uint_as_float(v[c][q * 8 + 2 * e]) * w, __uint_as_float(v[c][q * 8 + 2 * e + 1]) * w);
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
            tphase ^= 1;
        }
    }
    if (EPI == 2) __threadfence_system();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kXTmemCols);
    }
}

}  // namespace mfk

using namespace mfk;

namespace {
template <int EPI> int launch_mx(const XArgs &g, int grid, cudaStream_t s)
{
    auto kern = k_grouped_fp8_mx<EPI>;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, XSmem::kDynBytes) != cudaSuccess) {
            (void)cudaGetLastError();
            return -2;
        }
        attr_set = true;
    }
    kern<<<grid, kXThreads, XSmem::kDynBytes, s>>>(g);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}
}  // namespace

extern "C" {

// 1 when the block-scaled kernel takes this shape (the caller guarantees power-of-two scales).
int mf_grouped_gemm_fp8_mx_supported(int G, int N, int K, int epi)
{
    if (G <= 0 || G > kXMaxGroups || N <= 0 || K <= 0 || (N % XBN) != 0 || (K % 128) != 0) return 0;
    return epi >= 0 && epi <= 3;
}

// epi: 0 plain (out bf16 [rows, N]), 1 SwiGLU (out bf16 [rows, N/2]), 2 weighted push into the combine slots of the
// tokens' home ranks, 3 SwiGLU + fp8 re-quantisation (out e4m3 [rows, N/2], out_scale fp32 [rows, N/256]).
int mf_grouped_gemm_fp8_mx(const void *A, const float *a_scale, int max_rows, const void *B, const float *b_scale, const int *row_off, int G,
                           int N, int K, void *out, int64_t ldo, float *out_scale, int epi, const Team *team, const void *recv_info,
                           uint64_t comb_off, int topk, int *status, int sms, void *stream)
{
    if (!mf_grouped_gemm_fp8_mx_supported(G, N, K, epi) || max_rows <= 0) return -1;
    if (epi == 2 && (team == nullptr || recv_info == nullptr)) return -1;
    if (epi == 3 && (out_scale == nullptr || (ldo & 15) != 0)) return -1;
    XArgs g{};
    int rc = make_tmap_2d(&g.tm.a, A, 1, (uint64_t)max_rows, (uint64_t)K, (uint64_t)K, BM, true);
    if (rc == 0) rc = make_tmap_2d(&g.tm.b, B, 1, (uint64_t)G * N, (uint64_t)K, (uint64_t)K, XBN, true);
    if (rc != 0) return rc;
    g.a_scale = a_scale;
    g.b_scale = b_scale;
    g.row_off = row_off;
    g.G = G;
    g.N = N;
    g.K = K;
    g.max_rows = max_rows;
    g.out = out;
    g.ldo = ldo;
    g.out_scale = out_scale;
    g.status = status;
    if (team != nullptr) g.team = *team;
    g.recv_info = static_cast<const int4 *>(recv_info);
    g.comb_off = comb_off;
    g.topk = topk;
    cudaStream_t s = (cudaStream_t)stream;
    switch (epi) {
        case 0: return launch_mx<0>(g, sms, s);
        case 1: return launch_mx<1>(g, sms, s);
        case 2: return launch_mx<2>(g, sms, s);
        case 3: return launch_mx<3>(g, sms, s);
        default: return -1;
    }
}

}  // extern "C"
