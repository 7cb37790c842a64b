// Expert-parallel MoE communication kernels (DeepEP-style) on the symmetric heap.
//   moe_layout   : from topk_idx[T,K]: tokens per expert, tokens per rank, per-(token,k) index inside its
//                  expert (token order), token-in-rank mask
//   moe_notify   : all ranks exchange their per-expert send counts (peer stores + one barrier); every rank
//                  derives, on the device, the receive layout [local expert][source rank] of its own buffer
//                  and the offset at which each of ITS expert groups starts in the destination's buffer.
//                  Nothing is copied to the host: counts stay on the device.
//   moe_dispatch : FUSES the 1x128 block-scaled fp8 e4m3 quantisation of a token with the all-to-all: the
//                  quantised row, its 56 scales, its routing weight and its origin are stored straight into
//                  the receive buffers of the ranks that own its experts (peer stores over NVLink)
//   moe_combine_reduce : sums the K weighted expert outputs that peers pushed into this rank's combine
//                  slots (the push itself happens in the epilogue of the down-projection GEMM)
// Parity of role: app/zbal/src/csrc/operators/npu/aicore/ops/dispatch_combine_normal/
// zbal_kernel_{dispatch_layout,notify_dispatch,dispatch_normal,combine_normal}.h of the reference.
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <stdlib.h>

#include <map>
#include <mutex>
#include <utility>
#include <cuda_fp8.h>

#include "mf_devtrace.cuh"
#include "mf_fp8.cuh"
#include "mf_team.cuh"

namespace mfk {

constexpr int kQuantGroup = 128;

struct MoeShape {
    int T;        // tokens of this rank
    int K;        // experts per token
    int E;        // experts in total
    int H;        // hidden size (multiple of 128)
    int max_recv; // rows of the receive buffers
};

// Offsets (in each rank's slot) of the MoE communication area.
struct MoeHeap {
    uint64_t counts;      // int32 [W][E]           send counts, row s written by rank s
    uint64_t recv_x;      // fp8   [max_recv][H]
    uint64_t recv_scale;  // f32   [max_recv][H/128]
    uint64_t recv_info;   // int4  [max_recv]        {source rank, token, k slot, weight bits}
    uint64_t comb;        // bf16  [T_max * K][H]    combine slots of this rank's own tokens
    uint64_t flags;       // u32   [4][kMaxRanks]    0 dispatch done, 1 combine done
};

// ---- layout --------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) k_moe_layout_expert(const int *__restrict__ topk_idx, int n_entries, int *tokens_per_expert,
                                                            int *send_idx)
{
    // one CTA per expert: positions in token order by a block-wide running prefix
    const int e = blockIdx.x;
    __shared__ int warp_cnt[32];
    __shared__ int running;
    if (threadIdx.x == 0) running = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int base = 0; base < n_entries; base += blockDim.x) {
        const int i = base + threadIdx.x;
        const bool hit = i < n_entries && topk_idx[i] == e;
        const unsigned m = __ballot_sync(0xffffffffu, hit);
        if (lane == 0) warp_cnt[warp] = __popc(m);
        __syncthreads();
        int before = running;
        for (int w = 0; w < warp; w++) before += warp_cnt[w];
        if (hit) send_idx[i] = before + __popc(m & ((1u << lane) - 1));
        __syncthreads();
        if (threadIdx.x == 0) {
            int s = 0;
            for (int w = 0; w < (int)(blockDim.x >> 5); w++) s += warp_cnt[w];
            running += s;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) tokens_per_expert[e] = running;
}

// The same positions in O(entries) work: chunk c (1024 consecutive entries = one CTA) ranks its entries per expert in token
// order and leaves its per-expert counts in chunk_cnt[c][E]; the second kernel turns the counts of the earlier chunks into
// offsets and adds them. Entry ids outside [0, E) (unselected slots) get position 0 and count nowhere.
constexpr int kLayoutChunk = 1024;
__global__ void __launch_bounds__(kLayoutChunk) k_moe_layout_chunk_rank(const int *__restrict__ topk_idx, int n_entries, int E, int *send_idx,
                                                                        int *chunk_cnt)
{
    extern __shared__ uint16_t warp_cnt[];  // [32 warps][E]: hits of expert e in warp w, then their exclusive prefix over w
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) warp_cnt[i] = 0;
    __syncthreads();
    const int i = (int)blockIdx.x * kLayoutChunk + threadIdx.x;
    int e = i < n_entries ? topk_idx[i] : -1;
    if (e >= E) e = -1;
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1));
    if (e >= 0 && rank_in_warp == 0) warp_cnt[warp * E + e] = (uint16_t)__popc(peers);
    __syncthreads();
    for (int x = threadIdx.x; x < E; x += blockDim.x) {
        int run = 0;
        for (int w = 0; w < 32; w++) {
            const int c = warp_cnt[w * E + x];
            warp_cnt[w * E + x] = (uint16_t)run;
            run += c;
        }
        chunk_cnt[(int64_t)blockIdx.x * E + x] = run;
    }
    __syncthreads();
    if (i < n_entries) send_idx[i] = e >= 0 ? (int)warp_cnt[warp * E + e] + rank_in_warp : 0;
}

__global__ void __launch_bounds__(kLayoutChunk) k_moe_layout_chunk_offset(const int *__restrict__ topk_idx, int n_entries, int E, int *send_idx,
                                                                          const int *__restrict__ chunk_cnt, int *tokens_per_expert)
{
    extern __shared__ int before[];  // [E]: hits of expert e in the chunks before this one
    const int c = blockIdx.x;
    for (int x = threadIdx.x; x < E; x += blockDim.x) {
        int run = 0;
        for (int q = 0; q < c; q++) run += __ldg(chunk_cnt + (int64_t)q * E + x);
        before[x] = run;
        if (c == (int)gridDim.x - 1) tokens_per_expert[x] = run + __ldg(chunk_cnt + (int64_t)c * E + x);
    }
    __syncthreads();
    const int i = c * kLayoutChunk + threadIdx.x;
    if (i < n_entries) {
        const int e = topk_idx[i];
        if (e >= 0 && e < E) send_idx[i] += before[e];
    }
}

__global__ void k_moe_layout_rank(const int *__restrict__ topk_idx, int T, int K, int experts_per_rank, int world, int *tokens_per_rank,
                                  uint8_t *is_token_in_rank)
{
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    uint32_t mask = 0;
    for (int k = 0; k < K; k++) {
        const int e = topk_idx[t * K + k];
        if (e >= 0) mask |= 1u << (e / experts_per_rank);
    }
    for (int r = 0; r < world; r++) {
        const bool in = (mask >> r) & 1u;
        is_token_in_rank[t * world + r] = in ? 1 : 0;
        if (in) atomicAdd(tokens_per_rank + r, 1);
    }
}

// ---- notify ---------------------------------------------------------------------------------------
// outputs (device, local): recv_per_expert[El], row_off[El + 1], put_off[E], src_off[El][W]
// All threads of ONE CTA call it. Returns false (uniformly) when the count exchange timed out.
__device__ __forceinline__ bool notify_body(const Team &team, const MoeHeap &hp, int E, const int *tokens_per_expert, int *recv_per_expert,
                                            int *row_off, int *put_off, int *src_off, uint32_t epoch, uint32_t channel = 8)
{
    const uint32_t me = team_rank(team);
    const uint32_t W = team.world;
    const int El = E / (int)W;
    // 1. my counts into row `me` of everybody's table
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int c = tokens_per_expert[e];
        for (uint32_t k = 0; k < W; k++) {
            const uint32_t r = (me + k) % W;
            reinterpret_cast<int *>(peer_ptr(team, r, hp.counts))[me * E + e] = c;
        }
    }
    if (!team_barrier(team, me, channel, epoch)) return false;
    const int *tbl = reinterpret_cast<const int *>(peer_ptr(team, me, hp.counts));
    __shared__ int per_expert[1024];  // totals of every expert over all sources
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int s = 0;
        for (uint32_t r = 0; r < W; r++) s += __ldcg(tbl + r * E + e);
        per_expert[e] = s;
    }
    __syncthreads();
    // 2. my receive layout
    if (threadIdx.x == 0) {
        int run = 0;
        for (int le = 0; le < El; le++) {
            row_off[le] = run;
            recv_per_expert[le] = per_expert[me * El + le];
            run += per_expert[me * El + le];
        }
        row_off[El] = run;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < El * (int)W; i += blockDim.x) {
        const int le = i / (int)W, s = i % (int)W;
        int off = row_off[le];
        for (int r = 0; r < s; r++) off += __ldcg(tbl + r * E + me * El + le);
        src_off[i] = off;
    }
    // 3. where my group for expert e starts in its owner's buffer
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int d = e / El, le = e % El;
        int off = 0;
        for (int l2 = 0; l2 < le; l2++) off += per_expert[d * El + l2];
        for (uint32_t r = 0; r < me; r++) off += __ldcg(tbl + r * E + e);
        put_off[e] = off;
    }
    return true;
}

__global__ void __launch_bounds__(1024) k_moe_notify(Team team, MoeHeap hp, int E, const int *tokens_per_expert, int *recv_per_expert,
                                                     int *row_off, int *put_off, int *src_off, uint32_t epoch)
{
    notify_body(team, hp, E, tokens_per_expert, recv_per_expert, row_off, put_off, src_off, epoch);
}

// ---- dispatch -------------------------------------------------------------------------------------
// 448 threads per token row: thread i owns elements [16 i, 16 i + 16); 8 consecutive threads form a 128-group.
struct DispatchArgs {
    Team team;
    MoeHeap hp;
    MoeShape sh;
    const __nv_bfloat16 *x;     // [T, H]
    const int *topk_idx;        // [T, K]
    const float *topk_w;        // [T, K]
    const int *send_idx;        // [T, K]
    const int *put_off;         // [E]
    uint32_t *done_count;       // local counter, monotonic
    uint32_t epoch;
    uint32_t seq;
    int *status;
    int raw_bf16;               // 1: rows travel as bf16 (receive rows are 2 H bytes, no scales)
    const float *smooth;        // optional [H]: every row is multiplied by it before quantisation (smooth quant); fp8 rows only
};

// Loads this thread's 32 bytes of the first token row a CTA will handle (callers may do it early, e.g. while
// another CTA still computes the layout).
__device__ __forceinline__ void dispatch_preload(const DispatchArgs &a, uint4 &lo, uint4 &hi)
{
    lo = make_uint4(0, 0, 0, 0);
    hi = make_uint4(0, 0, 0, 0);
    const int vec = threadIdx.x;
    if (vec < a.sh.H / 16 && (int)blockIdx.x < a.sh.T) {
        const uint4 *src = reinterpret_cast<const uint4 *>(a.x + (int64_t)blockIdx.x * a.sh.H + vec * 16);
        lo = __ldg(src);
        hi = __ldg(src + 1);
    }
}

constexpr int kTokBatch = 32;  // tokens whose routing table a CTA resolves in one pass

__device__ __forceinline__ void dispatch_body(const DispatchArgs &a, uint4 nxt_lo, uint4 nxt_hi)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const int H = a.sh.H, K = a.sh.K, El = a.sh.E / (int)t.world;
    const int groups = H / kQuantGroup;
    const int vec = threadIdx.x;          // 16-element vector index inside the row
    const int vecs = H / 16;
    // Routing table of the next kTokBatch tokens of this CTA (destination rank, row there, weight), resolved by all
    // threads at once: the chain expert id -> put offset -> position is two dependent global loads, which would
    // otherwise sit in front of every single token.
    __shared__ int dst_rank[kTokBatch][16];
    __shared__ int dst_pos[kTokBatch][16];
    __shared__ float dst_w[kTokBatch][16];
    __shared__ __align__(16) float s_scale[2][64];  // the row's 1 x 128 scales, leaving as one burst per destination
    const int stride = (int)gridDim.x;
    // smooth-quant factors of this thread's 16 columns: the same for every token
    float smooth[16];
#pragma unroll
    for (int i = 0; i < 16; i++) smooth[i] = 1.f;
    const bool smoothed = a.smooth != nullptr && !a.raw_bf16;
    if (smoothed && vec < vecs) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 s4 = __ldg(reinterpret_cast<const float4 *>(a.smooth + vec * 16) + i);
            smooth[4 * i] = s4.x, smooth[4 * i + 1] = s4.y, smooth[4 * i + 2] = s4.z, smooth[4 * i + 3] = s4.w;
        }
    }
    for (int base = blockIdx.x; base < a.sh.T; base += stride * kTokBatch) {
        __syncthreads();  // the previous batch's table is no longer read
        for (int e = threadIdx.x; e < kTokBatch * K; e += blockDim.x) {
            const int j = e / K, k = e - j * K;
            const int tok = base + j * stride;
            int rk = -1;
            if (tok < a.sh.T) {
                const int ex = a.topk_idx[tok * K + k];
                if (ex >= 0) {
                    const int pos = a.put_off[ex] + a.send_idx[tok * K + k];
                    rk = pos < a.sh.max_recv ? ex / El : -1;
                    if (pos >= a.sh.max_recv) atomicCAS(a.status, 0, 0x401);  // receive buffer too small: dropped, reported
                    dst_pos[j][k] = pos;
                    dst_w[j][k] = a.topk_w[tok * K + k];
                }
            }
            dst_rank[j][k] = rk;
        }
        __syncthreads();
        // the row of the NEXT token is fetched while the stores of the current one drain
        for (int j = 0; j < kTokBatch; j++) {
            const int tok = base + j * stride;
            if (tok >= a.sh.T) break;
            uint4 q;
            uint4 raw_lo = make_uint4(0, 0, 0, 0), raw_hi = make_uint4(0, 0, 0, 0);
            float *sc = s_scale[j & 1];
            {
                float f[16];
#pragma unroll
                for (int i = 0; i < 16; i++) f[i] = 0.f;
                if (vec < vecs) {
                    const uint4 lo = nxt_lo, hi = nxt_hi;
                    raw_lo = lo;
                    raw_hi = hi;
                    const int nxt = tok + stride;
                    if (nxt < a.sh.T) {
                        const uint4 *src = reinterpret_cast<const uint4 *>(a.x + (int64_t)nxt * H + vec * 16);
                        nxt_lo = __ldg(src);
                        nxt_hi = __ldg(src + 1);
                    }
                    const __nv_bfloat162 *h0 = reinterpret_cast<const __nv_bfloat162 *>(&lo);
                    const __nv_bfloat162 *h1 = reinterpret_cast<const __nv_bfloat162 *>(&hi);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        float2 p = __bfloat1622float2(h0[i]);
                        f[2 * i] = p.x;
                        f[2 * i + 1] = p.y;
                        p = __bfloat1622float2(h1[i]);
                        f[8 + 2 * i] = p.x;
                        f[8 + 2 * i + 1] = p.y;
                    }
                }
                if (smoothed) {
#pragma unroll
                    for (int i = 0; i < 16; i++) f[i] *= smooth[i];
                }
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(f[i]));
                // the 8 threads of a 128-group are consecutive lanes of one warp; every lane takes part
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                const float scale = pow2_scale_e4m3(amax);   // a power of two: the expert GEMM feeds it to the tensor core as a UE8M0 byte
                const float mul = 1.f / scale;
                q.x = pack4_e4m3(f[0], f[1], f[2], f[3], mul);
                q.y = pack4_e4m3(f[4], f[5], f[6], f[7], mul);
                q.z = pack4_e4m3(f[8], f[9], f[10], f[11], mul);
                q.w = pack4_e4m3(f[12], f[13], f[14], f[15], mul);
                if (!a.raw_bf16 && vec < vecs && (vec & 7) == 0) sc[vec >> 3] = scale;
            }
            if (!a.raw_bf16) __syncthreads();  // the row's scales are complete (the buffers alternate: one barrier per token)
            for (int k = 0; k < K; k++) {
                const int d = dst_rank[j][k];
                if (d < 0) continue;
                const int64_t pos = dst_pos[j][k];
                if (vec < vecs) {
                    if (a.raw_bf16) {
                        uint4 *row = reinterpret_cast<uint4 *>(peer_ptr(t, d, a.hp.recv_x) + pos * H * 2 + vec * 32);
                        row[0] = raw_lo;
                        row[1] = raw_hi;
                    } else {
                        *reinterpret_cast<uint4 *>(peer_ptr(t, d, a.hp.recv_x) + pos * H + vec * 16) = q;
                    }
                }
                if (!a.raw_bf16) {
                    // scales: groups * 4 bytes, contiguous in the receiver's array: 16-byte stores from the last warp's lanes
                    // (one or two NVLink packets per row instead of one partial write per 128-group)
                    const int sv = threadIdx.x - ((int)blockDim.x - 32);
                    float *srow = reinterpret_cast<float *>(peer_ptr(t, d, a.hp.recv_scale)) + pos * groups;
                    if (sv >= 0) {
                        if (((pos * groups) & 3) == 0 && (groups & 3) == 0) {
                            if (sv < groups / 4) reinterpret_cast<float4 *>(srow)[sv] = reinterpret_cast<const float4 *>(sc)[sv];
                        } else {
                            for (int g = sv; g < groups; g += 32) srow[g] = sc[g];
                        }
                    }
                }
                if (threadIdx.x == 0) {
                    int4 info = make_int4((int)me, tok, k, __float_as_int(dst_w[j][k]));
                    reinterpret_cast<int4 *>(peer_ptr(t, d, a.hp.recv_info))[pos] = info;
                }
            }
        }
    }
    // the CTA that finishes last tells every peer that all of this rank's rows have been stored (the barrier orders the
    // CTA's stores before thread 0, whose system fence covers them; the counter links the CTAs' fences)
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t done = atomicAdd(a.done_count, 1u) + 1;
        // seq > 0: the counter only grows and the host numbers the calls; seq == 0: the last CTA puts it back
        // to zero, so the same launch parameters work again (CUDA-graph replay)
        const bool last = a.seq != 0 ? done == gridDim.x * a.seq : done == gridDim.x;
        if (last) {
            if (a.seq == 0) *a.done_count = 0;
            __threadfence_system();
            for (uint32_t r = 0; r < t.world; r++)
                st_release_sys(reinterpret_cast<uint32_t *>(peer_ptr(t, r, a.hp.flags)) + me, a.epoch);
        }
    }
}

// ---- warp-per-token dispatch ------------------------------------------------------------------------------
// Every warp takes whole tokens: it quantises the row into its own shared-memory buffer (e4m3 row, then the row's scales),
// and for every destination its lane 0 hands the copy unit ONE bulk store of the whole row, the scales leave as one
// 16-byte store per lane and the info record as one store from the lane that resolved the destination. Nothing in the
// loop involves another warp, so there is no CTA barrier per token, and a row costs one copy instruction per destination
// instead of one 16-byte store per thread per destination. Two buffers per warp: the copy unit reads the previous token's
// buffer while the next row is quantised.
constexpr int kDwWarps = 12;
constexpr int kDwLoads = 14;  // independent 16-byte loads per lane in flight (256 elements per warp load)
__host__ __device__ constexpr int dw_buf_bytes(int H) { return (H + (H / kQuantGroup) * 4 + 127) / 128 * 128; }  // e4m3 row + its scales
__host__ __device__ constexpr int dw_smem_bytes(int H) { return kDwWarps * 2 * dw_buf_bytes(H); }

__device__ __forceinline__ void bulk_store(void *gdst, const void *ssrc, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"((uint32_t)__cvta_generic_to_shared(ssrc)), "r"(bytes)
                 : "memory");
}

__global__ void __launch_bounds__(kDwWarps * 32) k_moe_dispatch_warp(DispatchArgs a)
{
    extern __shared__ __align__(128) uint8_t dw_smem[];
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const int H = a.sh.H, K = a.sh.K, El = a.sh.E / (int)t.world;
    const int groups = H / kQuantGroup;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stride_buf = dw_buf_bytes(H);
    uint8_t *bufs = dw_smem + (size_t)warp * 2 * stride_buf;
    const int wid = (int)blockIdx.x * kDwWarps + warp, wtotal = (int)gridDim.x * kDwWarps;
    const bool smoothed = a.smooth != nullptr;
    int which = 0;
    for (int tok = wid; tok < a.sh.T; tok += wtotal, which ^= 1) {
        uint8_t *buf = bufs + which * stride_buf;
        float *sc = reinterpret_cast<float *>(buf + H);
        // routing of this token: lane k resolves destination k (two dependent loads, overlapped with the row loads below)
        int d_rank = -1, d_pos = 0;
        float d_w = 0.f;
        if (lane < K) {
            const int ex = a.topk_idx[tok * K + lane];
            if (ex >= 0) {
                const int pos = a.put_off[ex] + a.send_idx[tok * K + lane];
                if (pos < a.sh.max_recv) {
                    d_rank = ex / El;
                    d_pos = pos;
                    d_w = a.topk_w[tok * K + lane];
                } else {
                    atomicCAS(a.status, 0, 0x401);  // receive buffer too small: dropped, reported
                }
            }
        }
        // the copy unit must be done READING this buffer (the token before the previous one)
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
        __syncwarp();
        // quantise: one warp load covers 256 elements = two 128-groups (lanes 0-15 and 16-31); half a row of 7168 elements
        // is requested before the first conversion (14 independent 16-byte loads per lane), so a token costs two memory
        // latencies, not one per chunk.
        const __nv_bfloat16 *row = a.x + (int64_t)tok * H;
        for (int c0 = 0; c0 < H; c0 += kDwLoads * 256) {
            uint4 raw[kDwLoads];
#pragma unroll
            for (int u = 0; u < kDwLoads; u++) {
                const int col = c0 + u * 256 + lane * 8;
                raw[u] = col < H ? __ldg(reinterpret_cast<const uint4 *>(row + col)) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < kDwLoads; u++) {
                const int col = c0 + u * 256 + lane * 8;
                if (c0 + u * 256 >= H) break;  // uniform over the warp
                const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw[u]);
                float f[8];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 p = __bfloat1622float2(h[i]);
                    f[2 * i] = p.x;
                    f[2 * i + 1] = p.y;
                }
                if (smoothed && col < H) {
                    const float4 s0 = __ldg(reinterpret_cast<const float4 *>(a.smooth + col));
                    const float4 s1 = __ldg(reinterpret_cast<const float4 *>(a.smooth + col) + 1);
                    f[0] *= s0.x, f[1] *= s0.y, f[2] *= s0.z, f[3] *= s0.w;
                    f[4] *= s1.x, f[5] *= s1.y, f[6] *= s1.z, f[7] *= s1.w;
                }
                float amax = 0.f;
#pragma unroll
                for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(f[i]));
#pragma unroll
                for (int o = 1; o < 16; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                const float scale = pow2_scale_e4m3(amax);
                const float mul = 1.f / scale;
                if (col < H) {
                    uint2 q;
                    q.x = pack4_e4m3(f[0], f[1], f[2], f[3], mul);
                    q.y = pack4_e4m3(f[4], f[5], f[6], f[7], mul);
                    *reinterpret_cast<uint2 *>(buf + col) = q;
                    if ((lane & 15) == 0) sc[col / kQuantGroup] = scale;
                }
            }
        }
        // the info record of destination k leaves from lane k as a plain store
        if (lane < K && d_rank >= 0)
            reinterpret_cast<int4 *>(peer_ptr(t, d_rank, a.hp.recv_info))[d_pos] = make_int4((int)me, tok, lane, __float_as_int(d_w));
        // generic-proxy writes to shared memory before the copy unit reads them
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        const float4 my_sc = lane < groups / 4 ? reinterpret_cast<const float4 *>(sc)[lane] : make_float4(0.f, 0.f, 0.f, 0.f);
        const float4 my_sc2 = lane + 32 < groups / 4 ? reinterpret_cast<const float4 *>(sc)[lane + 32] : make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < K; k++) {
            const int d = __shfl_sync(0xffffffffu, d_rank, k);
            const int pos = __shfl_sync(0xffffffffu, d_pos, k);
            if (d < 0) continue;
            // the row goes through the copy unit (one instruction for 7 KiB), its scales as one 16-byte store per lane
            if (lane == 0) bulk_store(peer_ptr(t, d, a.hp.recv_x) + (int64_t)pos * H, buf, (uint32_t)H);
            float4 *srow = reinterpret_cast<float4 *>(reinterpret_cast<float *>(peer_ptr(t, d, a.hp.recv_scale)) + (int64_t)pos * groups);
            if (lane < groups / 4) srow[lane] = my_sc;
            if (lane + 32 < groups / 4) srow[lane + 32] = my_sc2;
        }
        if (lane == 0) asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    // every bulk store of this warp has been performed before the CTA reports in
    if (lane == 0) {
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        asm volatile("fence.proxy.async;" ::: "memory");  // the copy unit's writes, as the generic proxy (the fences below) sees them
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        const uint32_t done = atomicAdd(a.done_count, 1u) + 1;
        const bool last = a.seq != 0 ? done == gridDim.x * a.seq : done == gridDim.x;
        if (last) {
            if (a.seq == 0) *a.done_count = 0;
            __threadfence_system();
            for (uint32_t r = 0; r < t.world; r++)
                st_release_sys(reinterpret_cast<uint32_t *>(peer_ptr(t, r, a.hp.flags)) + me, a.epoch);
        }
    }
}

__global__ void __launch_bounds__(448) k_moe_dispatch(DispatchArgs a)
{
    uint4 lo, hi;
    dispatch_preload(a, lo, hi);
    dispatch_body(a, lo, hi);
}

// Waits until every rank raised flag row `which` (0 dispatch, 1 combine) to `epoch`.
__global__ void k_moe_wait_all(Team t, MoeHeap hp, int which, uint32_t epoch, int *status)
{
    const uint32_t me = team_rank(t);
    if (threadIdx.x < t.world) {
        const uint32_t *f = reinterpret_cast<const uint32_t *>(peer_ptr(t, me, hp.flags)) + which * kMaxRanks + threadIdx.x;
        if (!wait_flag(f, epoch, t.spin_limit)) {
            report_timeout(t, me, 0x410 + which, epoch);
            atomicCAS(status, 0, 0x410 + which);
        }
    }
}

// Raises flag row `which` on every peer once all CTAs of the preceding kernel on this stream are done
// (stream order makes this launch the "last CTA").
__global__ void k_moe_signal_all(Team t, MoeHeap hp, int which, uint32_t epoch)
{
    const uint32_t me = team_rank(t);
    __threadfence_system();
    if (threadIdx.x < t.world)
        st_release_sys(reinterpret_cast<uint32_t *>(peer_ptr(t, threadIdx.x, hp.flags)) + which * kMaxRanks + me, epoch);
}

// out[t, :] = sum over the valid k slots of comb[t * K + k, :]; the rows were already multiplied by the
// routing weights when they were pushed.
__device__ __forceinline__ void combine_reduce_body(const Team &t, const MoeHeap &hp, const MoeShape &sh, const int *topk_idx, __nv_bfloat16 *out,
                                                    const float *topk_w);
__global__ void __launch_bounds__(256, 4) k_moe_combine_reduce(Team t, MoeHeap hp, MoeShape sh, const int *topk_idx, __nv_bfloat16 *out)
{
    combine_reduce_body(t, hp, sh, topk_idx, out, nullptr);
}

// Rows of bf16 -> fp8 e4m3 with one power-of-two scale per 128 elements (the activation format of the expert GEMMs).
// rows_dev: device int with the number of valid rows (the receive count), read here so the host never waits.
__global__ void __launch_bounds__(256) k_quant_rows_fp8(const __nv_bfloat16 *__restrict__ x, int64_t ldx, const int *rows_dev, int cols,
                                                        uint8_t *__restrict__ q, float *__restrict__ scales)
{
    const int rows = *rows_dev;
    const int groups = cols / kQuantGroup;
    const int lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    for (int64_t g = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); g < (int64_t)rows * groups; g += warps_total) {
        const int64_t r = g / groups;
        const int gi = (int)(g % groups);
        const uint2 raw = __ldg(reinterpret_cast<const uint2 *>(x + r * ldx + gi * kQuantGroup) + lane);
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
        const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float scale = pow2_scale_e4m3(amax);
        const float mul = 1.f / scale;
        uint32_t w = (uint32_t)__nv_cvt_float_to_fp8(a.x * mul, __NV_SATFINITE, __NV_E4M3) |
                     (uint32_t)__nv_cvt_float_to_fp8(a.y * mul, __NV_SATFINITE, __NV_E4M3) << 8 |
                     (uint32_t)__nv_cvt_float_to_fp8(b.x * mul, __NV_SATFINITE, __NV_E4M3) << 16 |
                     (uint32_t)__nv_cvt_float_to_fp8(b.y * mul, __NV_SATFINITE, __NV_E4M3) << 24;
        reinterpret_cast<uint32_t *>(q + r * cols + gi * kQuantGroup)[lane] = w;
        if (lane == 0) scales[r * groups + gi] = scale;
    }
}

// ---- standalone combine (push) ---------------------------------------------------------------------
// Expert outputs y[r, :] (bf16, local, row r of the receive layout) go back to the token's home rank:
// slot (token, k) of its combine area, multiplied by the routing weight that travelled with the row
// (weighted != 0) or as they are. The number of valid rows is read from the device.
struct CombinePushArgs {
    Team team;
    MoeHeap hp;
    const __nv_bfloat16 *y;
    int64_t ldy;
    const int *rows_dev;
    int H, K, weighted;
};

__device__ __forceinline__ void combine_push_body(const CombinePushArgs &a)
{
    const Team &t = a.team;
    const uint32_t me = team_rank(t);
    const int rows = *a.rows_dev;
    const int vecs = a.H / 8;
    const int4 *info = reinterpret_cast<const int4 *>(peer_ptr(t, me, a.hp.recv_info));
    // one warp per row, four 16-byte loads in flight per lane before the first store: at decode sizes the
    // push is bound by NVLink latency, so rows must overlap rather than queue behind one another
    const int lane = threadIdx.x & 31;
    const int warps = gridDim.x * (blockDim.x >> 5);
    for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
        const int4 in = __ldcg(info + r);
        const uint32_t home = (uint32_t)in.x;
        if (home >= t.world) continue;
        const float w = a.weighted ? __int_as_float(in.w) : 1.f;
        uint4 *dst = reinterpret_cast<uint4 *>(reinterpret_cast<__nv_bfloat16 *>(peer_ptr(t, home, a.hp.comb)) + ((int64_t)in.y * a.K + in.z) * a.H);
        const uint4 *src = reinterpret_cast<const uint4 *>(a.y + (int64_t)r * a.ldy);
        for (int v0 = lane; v0 < vecs; v0 += 128) {
            uint4 raw[4];
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (v0 + 32 * u < vecs) raw[u] = __ldg(src + v0 + 32 * u);
#pragma unroll
            for (int u = 0; u < 4; u++) {
                if (v0 + 32 * u >= vecs) continue;
                if (w != 1.f) {
                    __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&raw[u]);
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        float2 f = __bfloat1622float2(h[e]);
                        h[e] = __floats2bfloat162_rn(f.x * w, f.y * w);
                    }
                }
                dst[v0 + 32 * u] = raw[u];
            }
        }
    }
}

__global__ void __launch_bounds__(256) k_moe_combine_push(CombinePushArgs a) { combine_push_body(a); }

// topk_w: optional [T, K] weights applied here (rows that were pushed unweighted); NULL = plain sum
__device__ __forceinline__ void combine_reduce_body(const Team &t, const MoeHeap &hp, const MoeShape &sh, const int *topk_idx, __nv_bfloat16 *out,
                                                    const float *topk_w)
{
    const uint32_t me = team_rank(t);
    const __nv_bfloat16 *comb = reinterpret_cast<const __nv_bfloat16 *>(peer_ptr(t, me, hp.comb));
    const int vecs = sh.H / 8;
    // One work item = one 16-byte column vector of one token; items are dealt out grid-wide, so every thread stays busy
    // whatever T is. The slot loads do not wait for the routing table: every slot of the combine area exists, so all of a
    // token's slots are fetched at once and the ones that were not selected are dropped by a select afterwards (never by
    // a multiplication: a stale slot may hold anything).
    const int64_t items = (int64_t)sh.T * vecs;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t it = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; it < items; it += step) {
        const int tok = (int)(it / vecs), v = (int)(it - (int64_t)tok * vecs);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k0 = 0; k0 < sh.K; k0 += 8) {
            uint4 raw[8];
            float wk[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int k = min(k0 + u, sh.K - 1);
                raw[u] = __ldcs(reinterpret_cast<const uint4 *>(comb + ((int64_t)tok * sh.K + k) * sh.H) + v);   // read once: streaming
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int k = k0 + u;
                const bool on = k < sh.K && __ldg(topk_idx + tok * sh.K + k) >= 0;
                wk[u] = on ? (topk_w != nullptr ? __ldg(topk_w + tok * sh.K + k) : 1.f) : 0.f;
                if (!on) raw[u] = make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw[u]);
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const float2 f = __bfloat1622float2(h[e]);
                    acc[2 * e] += f.x * wk[u];
                    acc[2 * e + 1] += f.y * wk[u];
                }
            }
        }
        uint4 pk;
        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&pk);
#pragma unroll
        for (int e = 0; e < 4; e++) h[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
        *(reinterpret_cast<uint4 *>(out + (int64_t)tok * sh.H) + v) = pk;
    }
}

// ---- low-latency pair (decode) -----------------------------------------------------------------------
// One cooperative launch per direction instead of six: the launches, not the bytes, dominate at 128
// tokens. Dispatch: CTA 0 builds the layout (shared-memory histogram; the order of rows inside an expert
// group is the order in which the atomics land) and runs the count exchange, the grid then pushes the
// tokens and CTA 0 waits for every peer's rows. Combine: the grid pushes the expert outputs home, CTA 0
// signals and waits for all peers, the grid reduces the K slots of each token.
// The pair numbers its calls with a counter in device memory and uses flag rows and a barrier channel of
// its own (the caller passes MoeHeap.flags advanced by two rows), so a captured launch can be replayed
// as a CUDA graph and may be mixed with the multi-launch path on the same buffers.
// A wait that runs out is recorded in the status word; the kernel still reaches every grid-wide
// synchronisation and returns (the results of that call are then unspecified).
struct LLDispatchArgs {
    DispatchArgs d;          // d.send_idx and d.put_off are OUTPUTS here (device scratch of T*K and E ints)
    int *tokens_per_expert;  // [E] scratch
    int *recv_per_expert;    // [El]
    int *row_off;            // [El + 1]
    int *src_off;            // [El * W]
    uint32_t *epoch_dev;     // call counter in device memory: this call uses *epoch_dev + 1 and stores it back at the
                             // end, so a captured launch can be replayed (d.epoch is ignored, d.seq must be 0)
};

__global__ void __launch_bounds__(448) k_moe_ll_dispatch(LLDispatchArgs a)
{
    cooperative_groups::grid_group grid = cooperative_groups::this_grid();
    a.d.epoch = *reinterpret_cast<volatile uint32_t *>(a.epoch_dev) + 1;
    const Team &t = a.d.team;
    const uint32_t me = team_rank(t);
    const int E = a.d.sh.E, n = a.d.sh.T * a.d.sh.K;
    __shared__ int cnt[1024];
    uint4 pre_lo, pre_hi;
    dispatch_preload(a.d, pre_lo, pre_hi);  // every CTA fetches its first row while CTA 0 works out the layout
    if (blockIdx.x == 0) {
        MF_PROF_START(PF_LAYOUT);
        for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
        __syncthreads();
        int *send_idx = const_cast<int *>(a.d.send_idx);
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const int e = a.d.topk_idx[i];
            send_idx[i] = (e >= 0 && e < E) ? atomicAdd(&cnt[e], 1) : 0;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < E; e += blockDim.x) a.tokens_per_expert[e] = cnt[e];
        __syncthreads();
        if (!notify_body(t, a.d.hp, E, a.tokens_per_expert, a.recv_per_expert, a.row_off, const_cast<int *>(a.d.put_off), a.src_off, a.d.epoch, 9))
            if (threadIdx.x == 0) atomicCAS(a.d.status, 0, 0x420);
        __threadfence();
        MF_PROF_STOP(PF_LAYOUT);
    }
    grid.sync();  // every CTA has read the call counter before this point
    if (blockIdx.x == 0 && threadIdx.x == 0) *a.epoch_dev = a.d.epoch;
    MF_PROF_START(PF_DISPATCH);
    dispatch_body(a.d, pre_lo, pre_hi);
    MF_PROF_STOP(PF_DISPATCH);
    if (blockIdx.x == 0) MF_PROF_START(PF_WAIT_PEERS);
    if (blockIdx.x == 0 && threadIdx.x < t.world) {
        const uint32_t *f = reinterpret_cast<const uint32_t *>(peer_ptr(t, me, a.d.hp.flags)) + threadIdx.x;
        if (!wait_flag(f, a.d.epoch, t.spin_limit)) {
            report_timeout(t, me, 0x421, a.d.epoch);
            atomicCAS(a.d.status, 0, 0x421);
        }
    }
    if (blockIdx.x == 0) {
        __syncthreads();
        MF_PROF_STOP(PF_WAIT_PEERS);
    }
}

struct LLCombineArgs {
    CombinePushArgs p;
    MoeShape sh;
    const int *topk_idx;   // [T, K] of this rank's own tokens
    __nv_bfloat16 *out;    // [T, H]
    uint32_t epoch;        // used when epoch_dev is NULL
    int *status;
    const float *topk_w;   // optional [T, K]: weights applied on the home side
    const uint32_t *epoch_dev;  // the call counter the matching k_moe_ll_dispatch left behind
};

__global__ void __launch_bounds__(256) k_moe_ll_combine(LLCombineArgs a)
{
    cooperative_groups::grid_group grid = cooperative_groups::this_grid();
    const Team &t = a.p.team;
    const uint32_t me = team_rank(t);
    if (a.epoch_dev != nullptr) a.epoch = *reinterpret_cast<const volatile uint32_t *>(a.epoch_dev);
    MF_PROF_START(PF_PUSH);
    combine_push_body(a.p);
    __threadfence_system();
    MF_PROF_STOP(PF_PUSH);
    grid.sync();
    if (blockIdx.x == 0) MF_PROF_START(PF_WAIT_PEERS);
    if (blockIdx.x == 0 && threadIdx.x < t.world) {
        st_release_sys(reinterpret_cast<uint32_t *>(peer_ptr(t, threadIdx.x, a.p.hp.flags)) + kMaxRanks + me, a.epoch);
        const uint32_t *f = reinterpret_cast<const uint32_t *>(peer_ptr(t, me, a.p.hp.flags)) + kMaxRanks + threadIdx.x;
        if (!wait_flag(f, a.epoch, t.spin_limit)) {
            report_timeout(t, me, 0x422, a.epoch);
            atomicCAS(a.status, 0, 0x422);
        }
    }
    if (blockIdx.x == 0) {
        __syncthreads();
        MF_PROF_STOP(PF_WAIT_PEERS);
    }
    grid.sync();
    MF_PROF_START(PF_COMBINE);
    combine_reduce_body(t, a.p.hp, a.sh, a.topk_idx, a.out, a.topk_w);
    MF_PROF_STOP(PF_COMBINE);
}

}  // namespace mfk

using namespace mfk;

MF_DEVTRACE_DEFINE_SETTER(mf_moe_set_devtrace)

extern "C" {

// Counter scratch of the chunked layout: one buffer per (device, stream), grown on demand and kept for the life of the process
// (work on one stream is ordered, so consecutive layouts on it may share the buffer; different streams never do).
static int *layout_scratch(cudaStream_t s, size_t bytes)
{
    static std::mutex mu;
    static std::map<std::pair<int, cudaStream_t>, std::pair<int *, size_t>> bufs;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> g(mu);
    auto &b = bufs[{dev, s}];
    if (b.second < bytes) {
        // the old buffer may still be read by work in flight on the stream: it is left to the process (a few hundred KB)
        int *p = nullptr;
        const size_t want = bytes < (256u << 10) ? (256u << 10) : bytes * 2;
        if (cudaMalloc(reinterpret_cast<void **>(&p), want) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        b = {p, want};
    }
    return b.first;
}

int mf_moe_layout(const int *topk_idx, int T, int K, int E, int world, int *tokens_per_expert, int *tokens_per_rank, int *send_idx,
                  uint8_t *is_token_in_rank, void *stream)
{
    if (T <= 0 || K <= 0 || K > 16 || E <= 0 || E > 1024 || world <= 0 || E % world != 0) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    cudaMemsetAsync(tokens_per_rank, 0, sizeof(int) * world, s);
    // chunked ranking needs chunks x E counters; very large problems keep the one-CTA-per-expert kernel
    const int n = T * K, chunks = (n + kLayoutChunk - 1) / kLayoutChunk;
    int *chunk_cnt = (int64_t)chunks * E <= (4 << 20) ? layout_scratch(s, sizeof(int) * (size_t)chunks * E) : nullptr;
    if (chunk_cnt != nullptr) {
        static bool attr = false;
        if (!attr) {
            cudaFuncSetAttribute(k_moe_layout_chunk_rank, cudaFuncAttributeMaxDynamicSharedMemorySize, 32 * 1024 * 2);
            attr = true;
        }
        k_moe_layout_chunk_rank<<<chunks, kLayoutChunk, 32 * E * sizeof(uint16_t), s>>>(topk_idx, n, E, send_idx, chunk_cnt);
        k_moe_layout_chunk_offset<<<chunks, kLayoutChunk, E * sizeof(int), s>>>(topk_idx, n, E, send_idx, chunk_cnt, tokens_per_expert);
    } else {
        k_moe_layout_expert<<<E, 1024, 0, s>>>(topk_idx, T * K, tokens_per_expert, send_idx);
    }
    k_moe_layout_rank<<<(T + 255) / 256, 256, 0, s>>>(topk_idx, T, K, E / world, world, tokens_per_rank, is_token_in_rank);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

int mf_moe_notify(const Team *team, const MoeHeap *hp, int E, const int *tokens_per_expert, int *recv_per_expert, int *row_off,
                  int *put_off, int *src_off, uint32_t epoch, void *stream)
{
    if (team == nullptr || hp == nullptr || team->emu || E > 1024 || E % (int)team->world != 0) return -1;
    k_moe_notify<<<1, 1024, 0, (cudaStream_t)stream>>>(*team, *hp, E, tokens_per_expert, recv_per_expert, row_off, put_off, src_off, epoch);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

int mf_moe_dispatch(const DispatchArgs *a, int ctas, void *stream)
{
    if (a == nullptr || a->team.emu || a->sh.H % 128 != 0 || a->sh.H / 16 > 448 || a->sh.K > 16) return -1;
    // fp8 rows whose scales make whole 16-byte units: every warp pushes whole tokens through the copy unit
    static const bool warp_ok = [] {
        const char *e = getenv("MF_MOE_DISPATCH_WARP");
        return e == nullptr || atoi(e) != 0;
    }();
    const int smem = dw_smem_bytes(a->sh.H);
    if (warp_ok && !a->raw_bf16 && a->sh.H % 512 == 0 && smem <= 220 * 1024) {
        static int attr_for = 0;
        if (smem > attr_for) {
            if (cudaFuncSetAttribute(k_moe_dispatch_warp, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
                (void)cudaGetLastError();
                return -2;
            }
            attr_for = smem;
        }
        k_moe_dispatch_warp<<<ctas, kDwWarps * 32, smem, (cudaStream_t)stream>>>(*a);
        cudaError_t e = cudaGetLastError();
        return e == cudaSuccess ? 0 : (int)e;
    }
    k_moe_dispatch<<<ctas, 448, 0, (cudaStream_t)stream>>>(*a);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

int mf_moe_wait_all(const Team *team, const MoeHeap *hp, int which, uint32_t epoch, int *status, void *stream)
{
    k_moe_wait_all<<<1, 32, 0, (cudaStream_t)stream>>>(*team, *hp, which, epoch, status);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

int mf_moe_signal_all(const Team *team, const MoeHeap *hp, int which, uint32_t epoch, void *stream)
{
    k_moe_signal_all<<<1, 32, 0, (cudaStream_t)stream>>>(*team, *hp, which, epoch);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

int mf_moe_combine_reduce(const Team *team, const MoeHeap *hp, const MoeShape *sh, const int *topk_idx, void *out, int ctas, void *stream)
{
    if (sh->H % 8 != 0) return -1;
    k_moe_combine_reduce<<<ctas, 256, 0, (cudaStream_t)stream>>>(*team, *hp, *sh, topk_idx, static_cast<__nv_bfloat16 *>(out));
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

int mf_moe_combine_push(const Team *team, const MoeHeap *hp, const void *y, int64_t ldy, const int *rows_dev, int H, int K, int weighted,
                        int ctas, void *stream)
{
    if (team == nullptr || hp == nullptr || team->emu || H % 8 != 0 || ctas <= 0) return -1;
    CombinePushArgs a{*team, *hp, static_cast<const __nv_bfloat16 *>(y), ldy, rows_dev, H, K, weighted};
    k_moe_combine_push<<<ctas, 256, 0, (cudaStream_t)stream>>>(a);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

// Cooperative: ctas must not exceed what the device can hold at once (one CTA per SM is always safe).
int mf_moe_ll_dispatch(const DispatchArgs *d, int *tokens_per_expert, int *recv_per_expert, int *row_off, int *src_off, uint32_t *epoch_dev,
                       int ctas, void *stream)
{
    if (epoch_dev == nullptr || d == nullptr || d->seq != 0) return -1;
    if (d == nullptr || d->team.emu || d->sh.H % 128 != 0 || d->sh.H / 16 > 448 || d->sh.K > 16 || d->sh.E > 1024 ||
        d->sh.E % (int)d->team.world != 0 || ctas <= 0)
        return -1;
    LLDispatchArgs a{*d, tokens_per_expert, recv_per_expert, row_off, src_off, epoch_dev};
    void *params[] = {&a};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(k_moe_ll_dispatch), dim3(ctas), dim3(448), params, 0,
                                                (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : (int)e;
}

int mf_moe_ll_combine(const Team *team, const MoeHeap *hp, const MoeShape *sh, const void *y, int64_t ldy, const int *rows_dev, int weighted,
                      const int *topk_idx, const float *topk_w, void *out, uint32_t epoch, const uint32_t *epoch_dev, int *status, int ctas,
                      void *stream)
{
    if (team == nullptr || hp == nullptr || sh == nullptr || team->emu || sh->H % 8 != 0 || ctas <= 0) return -1;
    LLCombineArgs a{{*team, *hp, static_cast<const __nv_bfloat16 *>(y), ldy, rows_dev, sh->H, sh->K, weighted}, *sh, topk_idx,
                    static_cast<__nv_bfloat16 *>(out), epoch, status, topk_w, epoch_dev};
    void *params[] = {&a};
    cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(k_moe_ll_combine), dim3(ctas), dim3(256), params, 0,
                                                (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : (int)e;
}

int mf_quant_rows_fp8(const void *x, int64_t ldx, const int *rows_dev, int cols, void *q, float *scales, int ctas, void *stream)
{
    if (cols % 128 != 0) return -1;
    k_quant_rows_fp8<<<ctas, 256, 0, (cudaStream_t)stream>>>(static_cast<const __nv_bfloat16 *>(x), ldx, rows_dev, cols,
                                                             static_cast<uint8_t *>(q), scales);
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? 0 : (int)e;
}

}  // extern "C"
