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
// The same mainloop also runs the two tensor-parallel fusions on dense operands (MODE 1 / MODE 2):
//   MODE 1  all-gather -> GEMM : warp 3 of every CTA quantises its rows of this rank's bf16 sequence shard to
//                                fp8 + 1 x 128 scales into the rank's own gather buffer (first, so the first
//                                tiles can start), then copies those bytes into every peer's gather buffer,
//                                nearest consumer first; the TMA and scale warps wait for a shard's flag
//                                before they touch its rows. Operands are read from THIS GPU's buffer only.
//   MODE 2  GEMM -> reduce-scatter : the epilogue stores each partial tile (bf16) into the landing zone of the
//                                rank that owns the rows and counts it there; after its tiles a CTA adds up
//                                the landed partials of the tiles it owns.
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
    Team team;             // EPI 2, MODE 1, MODE 2
    const int4 *recv_info;
    uint64_t comb_off;
    int topk;
    uint32_t epoch;        // flag value of this call (grows by one per call)
    uint32_t seq;          // number of fused calls so far on these counters, including this one
    // MODE 1
    const __nv_bfloat16 *x_local;  // this rank's shard [shard_rows, K] bf16
    int64_t ldx;
    int shard_rows;
    uint64_t ag_buf_off;     // slot offset of the gather buffer [W * shard_rows, K] e4m3
    uint64_t ag_scale_off;   // slot offset of its scales [W * shard_rows, K / 128] fp32
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

__device__ __forceinline__ void named_bar_sync(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

template <int MODE, int EPI> __global__ void __launch_bounds__(kXThreads, 1) k_grouped_fp8_mx(const __grid_constant__ XArgs g)
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
        if (MODE == 0) {
            int run = 0;
            for (int i = 0; i <= g.G; i++) {
                const int ro = min(g.row_off[i], g.max_rows);
                s_row_off[i] = ro;
                tile_start[i] = run;
                if (i < g.G) run += ((min(g.row_off[i + 1], g.max_rows) - ro + BM - 1) / BM) * n_tiles;
            }
        } else {
            s_row_off[0] = 0;
            s_row_off[1] = g.max_rows;
            tile_start[0] = 0;
            tile_start[1] = (g.max_rows / BM) * n_tiles;
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
    const int total = tile_start[MODE == 0 ? g.G : 1];
    const uint32_t me = g.team.rank;

    // linear tile -> (group, first row, row limit, column tile); inside a group the row tile varies fastest
    auto locate = [&](int t, int &grp, int &row0, int &row_end, int &nt) {
        if (MODE != 0) {
            // blocks of rows owned by one rank, visited starting with this rank (MODE 1: the order in which the shards
            // arrive) or with the next rank (MODE 2: remote owners first, own rows last)
            const int rows = MODE == 1 ? g.shard_rows : g.rows_per_rank;
            const int mt_per = rows / BM;
            const int per_block = mt_per * n_tiles;
            const int i = t / per_block;
            const int owner = (int)((me + (MODE == 2 ? 1 : 0) + i) % g.team.world);
            const int r = t - i * per_block;
            grp = 0;
            nt = r / mt_per;
            row0 = (owner * mt_per + r % mt_per) * BM;
            row_end = g.max_rows;
            return;
        }
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
                if (MODE == 1) {
                    // the shard holding this tile's rows must have landed in this GPU's gather buffer
                    const uint32_t *ready = reinterpret_cast<const uint32_t *>(peer_ptr(g.team, me, g.ag_ready_off)) + row0 / g.shard_rows;
                    if (!wait_flag(ready, g.epoch, g.team.spin_limit)) {
                        *ac.abort_smem = 1;
                        atomicCAS(g.status, 0, 0x601);
                        break;
                    }
                    asm volatile("fence.proxy.async.global;" ::: "memory");  // peers' generic-proxy stores before our TMA reads
                }
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
            if (MODE == 1) {
                // the scales of a shard arrive with its rows
                int ok = 1;
                if (lane == 0) {
                    const uint32_t *ready = reinterpret_cast<const uint32_t *>(peer_ptr(g.team, me, g.ag_ready_off)) + row0 / g.shard_rows;
                    ok = wait_flag(ready, g.epoch, g.team.spin_limit) ? 1 : 0;
                    if (!ok) {
                        *ac.abort_smem = 1;
                        atomicCAS(g.status, 0, 0x608);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) {
                    fine = false;
                    break;
                }
            }
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
                        // MODE 1: written by peers during this kernel, so not through the read-only path
                        w |= (kb < k_blocks ? ue8m0_byte(MODE == 1 ? __ldcg(as + kb) : __ldg(as + kb)) : 127u) << (8 * j);
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
                // rows leave through shared memory: lane = row on the way in, 16 lanes x 16 bytes per row on the way out
                unsigned long long dst = 0;
                float w = 1.f;
                if (row_ok) {
                    if (EPI == 2) {
                        const int4 info = __ldg(g.recv_info + row);
                        w = __int_as_float(info.w);
                        dst = reinterpret_cast<unsigned long long>(reinterpret_cast<__nv_bfloat16 *>(peer_ptr(g.team, (uint32_t)info.x, g.comb_off)) +
                                                                   ((int64_t)info.y * g.topk + info.z) * g.N + nt * XBN + half * 128);
                    } else if (MODE == 2) {
                        // the partial tile goes to the landing zone of the rank that owns these rows
                        const int owner = row0 / g.rows_per_rank;
                        dst = reinterpret_cast<unsigned long long>(reinterpret_cast<__nv_bfloat16 *>(peer_ptr(g.team, (uint32_t)owner, g.rs_land_off)) +
                                                                   ((int64_t)me * g.rows_per_rank + (row - owner * g.rows_per_rank)) * g.N + nt * XBN + half * 128);
                    } else {
                        dst = reinterpret_cast<unsigned long long>(static_cast<__nv_bfloat16 *>(g.out) + (int64_t)row * g.ldo + nt * XBN + half * 128);
                    }
                }
                // Eight rows at a time: the lanes that own them write their whole 256-byte row segments (this warp's 128
                // columns) into the staging buffer, then the warp stores them 2 rows x 256 contiguous bytes per instruction
                // (16 lanes x 16 bytes per row). Over NVLink a write carries up to 256 bytes of payload: 64-byte pieces spent
                // almost half of the link on packet overhead.
                constexpr int kWideRowB = 272;  // 256 + 16: both the row writes and the 16-lanes-per-row reads stay conflict-free
                static_assert(8 * kWideRowB <= 32 * kRowB, "staging buffer of an epilogue warp");
#pragma unroll
                for (int p = 0; p < 4; p++) {
                    if ((lane >> 3) == p) {
                        uint8_t *mine = stg + (lane & 7) * kWideRowB;
#pragma unroll
                        for (int c = 0; c < 4; c++) {
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                uint4 pk;
                                __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
                                for (int e = 0; e < 4; e++)
                                    h[e] = __floats2bfloat162_rn(__uint_as_float(v[c][q * 8 + 2 * e]) * w, __uint_as_float(v[c][q * 8 + 2 * e + 1]) * w);
                                *reinterpret_cast<uint4 *>(mine + c * 64 + q * 16) = pk;
                            }
                        }
                    }
                    __syncwarp();
#pragma unroll
                    for (int it = 0; it < 4; it++) {
                        const int r = it * 2 + (lane >> 4);
                        const unsigned long long d = __shfl_sync(0xffffffffu, dst, p * 8 + r);
                        const uint4 val = *reinterpret_cast<const uint4 *>(stg + r * kWideRowB + (lane & 15) * 16);
                        if (d != 0) *reinterpret_cast<uint4 *>(d + (unsigned long long)((lane & 15) * 16)) = val;
                    }
                    __syncwarp();
                }
                if (MODE == 2) {
                    // all eight epilogue warps have stored their part of the tile: tell the owner
                    named_bar_sync(9, 256);  // orders all eight warps' stores before the counting thread, whose fence + release publishes them
                    if (warp == 4 && lane == 0) {
                        __threadfence_system();
                        const int owner = row0 / g.rows_per_rank;
                        const int ltile = ((row0 - owner * g.rows_per_rank) / BM) * n_tiles + nt;
                        uint32_t *cnt = reinterpret_cast<uint32_t *>(peer_ptr(g.team, (uint32_t)owner, g.rs_count_off)) + ltile;
                        asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(cnt) : "memory");
                    }
                }
            }
            tphase ^= 1;
        }
    } else if (MODE == 1 && warp == 3) {
        // all-gather side. Pass 1: this CTA's rows of the rank's bf16 shard -> e4m3 + one power-of-two scale per 128
        // elements, into the rank's OWN gather buffer (lane = 16 elements, 8 lanes = one 128-group, four steps of 512
        // elements in flight). Pass 2: those bytes and scales to every peer, nearest consumer first.
        const int per = (g.shard_rows + (int)gridDim.x - 1) / (int)gridDim.x;
        const int r0 = min(g.shard_rows, (int)blockIdx.x * per), r1 = min(g.shard_rows, r0 + per);
        const int K = g.K, kg = K / 128;
        const int64_t shard_q = (int64_t)me * g.shard_rows * K, shard_s = (int64_t)me * g.shard_rows * kg;
        uint8_t *own_q = peer_ptr(g.team, me, g.ag_buf_off) + shard_q;
        float *own_s = reinterpret_cast<float *>(peer_ptr(g.team, me, g.ag_scale_off)) + shard_s;
        for (int row = r0; row < r1; row++) {
            const __nv_bfloat16 *src = g.x_local + (int64_t)row * g.ldx;
            for (int c0 = 0; c0 < K; c0 += 2048) {
                uint4 raw[4][2];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int c = c0 + u * 512 + lane * 16;
                    if (c < K) {
                        raw[u][0] = __ldg(reinterpret_cast<const uint4 *>(src + c));
                        raw[u][1] = __ldg(reinterpret_cast<const uint4 *>(src + c) + 1);
                    } else {
                        raw[u][0] = raw[u][1] = make_uint4(0, 0, 0, 0);
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int c = c0 + u * 512 + lane * 16;
                    float f[16];
                    const __nv_bfloat162 *h0 = reinterpret_cast<const __nv_bfloat162 *>(&raw[u][0]);
                    const __nv_bfloat162 *h1 = reinterpret_cast<const __nv_bfloat162 *>(&raw[u][1]);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        float2 pr = __bfloat1622float2(h0[i]);
                        f[2 * i] = pr.x;
                        f[2 * i + 1] = pr.y;
                        pr = __bfloat1622float2(h1[i]);
                        f[8 + 2 * i] = pr.x;
                        f[8 + 2 * i + 1] = pr.y;
                    }
                    float amax = 0.f;
#pragma unroll
                    for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(f[i]));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                    const float scale = pow2_scale_e4m3(amax);
                    const float mul = 1.f / scale;
                    if (c < K) {
                        uint4 q;
                        q.x = pack4_e4m3(f[0], f[1], f[2], f[3], mul);
                        q.y = pack4_e4m3(f[4], f[5], f[6], f[7], mul);
                        q.z = pack4_e4m3(f[8], f[9], f[10], f[11], mul);
                        q.w = pack4_e4m3(f[12], f[13], f[14], f[15], mul);
                        *reinterpret_cast<uint4 *>(own_q + (int64_t)row * K + c) = q;
                        if ((lane & 7) == 0) own_s[(int64_t)row * kg + c / 128] = scale;
                    }
                }
            }
        }
        auto raise = [&](uint32_t p) {
            // the CTA that completes this rank's shard in the buffer of rank p raises the flag there
            __syncwarp();
            if (lane == 0) {
                __threadfence_system();  // covers the whole warp's stores (ordered before it by the warp barrier)
                const uint32_t done = atomicAdd(g.push_count + p, 1u) + 1;
                if (done == gridDim.x * g.seq) {
                    __threadfence_system();
                    st_release_sys(reinterpret_cast<uint32_t *>(peer_ptr(g.team, p, g.ag_ready_off)) + me, g.epoch);
                }
            }
            __syncwarp();
        };
        raise(me);
        const int64_t nq = (int64_t)(r1 - r0) * K / 16, ns = (int64_t)(r1 - r0) * kg;
        const uint4 *from_q = reinterpret_cast<const uint4 *>(own_q + (int64_t)r0 * K);
        const float *from_s = own_s + (int64_t)r0 * kg;
        for (uint32_t i = 1; i < g.team.world; i++) {
            const uint32_t p = (me + g.team.world - i) % g.team.world;
            uint4 *to_q = reinterpret_cast<uint4 *>(peer_ptr(g.team, p, g.ag_buf_off) + shard_q + (int64_t)r0 * K);
            float *to_s = reinterpret_cast<float *>(peer_ptr(g.team, p, g.ag_scale_off)) + shard_s + (int64_t)r0 * kg;
            int64_t v = lane;
            for (; v + 7 * 32 < nq; v += 8 * 32) {  // eight independent 16-byte loads in flight per lane, then eight peer stores
                uint4 val[8];
#pragma unroll
                for (int u = 0; u < 8; u++) val[u] = __ldcg(from_q + v + u * 32);
#pragma unroll
                for (int u = 0; u < 8; u++) to_q[v + u * 32] = val[u];
            }
            for (; v < nq; v += 32) to_q[v] = __ldcg(from_q + v);
            for (int64_t e = lane; e < ns; e += 32) to_s[e] = __ldcg(from_s + e);
            raise(p);
        }
    }
    if (EPI == 2) __threadfence_system();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kXTmemCols);
    }
    if (MODE == 2) {
        // add up the W partial tiles of every tile whose rows this rank owns
        __shared__ int ok_sh;
        const int own_tiles = (g.rows_per_rank / BM) * n_tiles;
        const uint32_t *cnt = reinterpret_cast<const uint32_t *>(peer_ptr(g.team, me, g.rs_count_off));
        const __nv_bfloat16 *land = reinterpret_cast<const __nv_bfloat16 *>(peer_ptr(g.team, me, g.rs_land_off));
        for (int t = blockIdx.x; t < own_tiles; t += gridDim.x) {
            if (threadIdx.x == 0) {
                ok_sh = (!*ac.abort_smem && wait_flag(cnt + t, g.team.world * g.seq, g.team.spin_limit)) ? 1 : 0;
                if (!ok_sh) atomicCAS(g.status, 0, 0x609);
            }
            __syncthreads();
            if (!ok_sh) break;
            const int ml = t / n_tiles, nt = t % n_tiles;
            constexpr int kVecRow = XBN / 8;
            for (int v = threadIdx.x; v < BM * kVecRow; v += blockDim.x) {
                const int lr = ml * BM + v / kVecRow;
                const int col = nt * XBN + (v % kVecRow) * 8;
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
template <int MODE, int EPI> int launch_mx(const XArgs &g, int grid, cudaStream_t s)
{
    auto kern = k_grouped_fp8_mx<MODE, EPI>;
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
        case 0: return launch_mx<0, 0>(g, sms, s);
        case 1: return launch_mx<0, 1>(g, sms, s);
        case 2: return launch_mx<0, 2>(g, sms, s);
        case 3: return launch_mx<0, 3>(g, sms, s);
        default: return -1;
    }
}

// All-gather -> GEMM in fp8. x_local [shard_rows, K] bf16 is this rank's sequence shard; it is quantised (e4m3, one
// power-of-two scale per 128 elements) on its way into the gather buffers ([world * shard_rows, K] bytes at ag_buf_off,
// scales [world * shard_rows, K / 128] fp32 at ag_scale_off of every slot). B [N, K] e4m3 with b_scale [N/128, K/128].
// epi 0: out bf16 [world * shard_rows, N]; 1: SwiGLU, out bf16 [.., N/2] (B interleaved per 128 rows); 3: SwiGLU +
// re-quantisation, out e4m3 [.., N/2] with out_scale [.., N/256].
int mf_ag_gemm_fp8(const Team *team, const void *x_local, int64_t ldx, int shard_rows, const void *B, const float *b_scale, void *out, int64_t ldo,
                   float *out_scale, int N, int K, uint64_t ag_buf_off, uint64_t ag_scale_off, uint64_t ag_ready_off, uint32_t *push_count,
                   uint32_t epoch, uint32_t seq, int *status, int sms, int epi, void *stream)
{
    if (team == nullptr || team->emu || shard_rows <= 0 || (shard_rows % BM) != 0 || (K % 512) != 0 || (ldx & 7) != 0 ||
        !mf_grouped_gemm_fp8_mx_supported(1, N, K, epi) || epi == 2)
        return -1;
    if (epi == 3 && (out_scale == nullptr || (ldo & 15) != 0)) return -1;
    XArgs g{};
    const int M = shard_rows * (int)team->world;
    const uint64_t slot = team->heap_base + (uint64_t)team->rank * team->stride;
    int rc = make_tmap_2d(&g.tm.a, reinterpret_cast<const void *>(slot + ag_buf_off), 1, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, true);
    if (rc == 0) rc = make_tmap_2d(&g.tm.b, B, 1, (uint64_t)N, (uint64_t)K, (uint64_t)K, XBN, true);
    if (rc != 0) return rc;
    g.a_scale = reinterpret_cast<const float *>(slot + ag_scale_off);
    g.b_scale = b_scale;
    g.G = 1;
    g.N = N;
    g.K = K;
    g.max_rows = M;
    g.out = out;
    g.ldo = ldo;
    g.out_scale = out_scale;
    g.status = status;
    g.team = *team;
    g.epoch = epoch;
    g.seq = seq;
    g.x_local = static_cast<const __nv_bfloat16 *>(x_local);
    g.ldx = ldx;
    g.shard_rows = shard_rows;
    g.ag_buf_off = ag_buf_off;
    g.ag_scale_off = ag_scale_off;
    g.ag_ready_off = ag_ready_off;
    g.push_count = push_count;
    cudaStream_t s = (cudaStream_t)stream;
    // every CTA carries a copy warp whose work peers wait for: the grid must be fully resident (one CTA per SM)
    switch (epi) {
        case 0: return launch_mx<1, 0>(g, sms, s);
        case 1: return launch_mx<1, 1>(g, sms, s);
        case 3: return launch_mx<1, 3>(g, sms, s);
        default: return -1;
    }
}

// GEMM -> reduce-scatter in fp8. A [M, K] e4m3 (M = world * rows_per_rank) with a_scale [M, K/128], B [N, K] e4m3 with
// b_scale [N/128, K/128]; y_out [rows_per_rank, N] bf16 = scale * sum over ranks of A . B^T.
int mf_gemm_rs_fp8(const Team *team, const void *A, const float *a_scale, const void *B, const float *b_scale, void *y_out, int64_t ldy,
                   int rows_per_rank, int N, int K, uint64_t rs_land_off, uint64_t rs_count_off, uint32_t epoch, uint32_t seq, float scale,
                   int *status, int sms, void *stream)
{
    if (team == nullptr || team->emu || rows_per_rank <= 0 || (rows_per_rank % BM) != 0 || (ldy & 7) != 0 ||
        !mf_grouped_gemm_fp8_mx_supported(1, N, K, 0))
        return -1;
    XArgs g{};
    const int M = rows_per_rank * (int)team->world;
    int rc = make_tmap_2d(&g.tm.a, A, 1, (uint64_t)M, (uint64_t)K, (uint64_t)K, BM, true);
    if (rc == 0) rc = make_tmap_2d(&g.tm.b, B, 1, (uint64_t)N, (uint64_t)K, (uint64_t)K, XBN, true);
    if (rc != 0) return rc;
    g.a_scale = a_scale;
    g.b_scale = b_scale;
    g.G = 1;
    g.N = N;
    g.K = K;
    g.max_rows = M;
    g.status = status;
    g.team = *team;
    g.epoch = epoch;
    g.seq = seq;
    g.rs_land_off = rs_land_off;
    g.rs_count_off = rs_count_off;
    g.rows_per_rank = rows_per_rank;
    g.y_out = static_cast<__nv_bfloat16 *>(y_out);
    g.ldy = ldy;
    g.scale = scale;
    return launch_mx<2, 0>(g, sms, (cudaStream_t)stream);
}

}  // extern "C"
