// Shared pieces of the tcgen05 GEMM kernels: host-side tensor-map creation, the shared-memory
// pipeline layout and the three warp roles' loop skeletons.
//   warp 0      TMA producer   : fills a ring of (A tile, B tile) stages, one mbarrier pair per stage
//   warp 1      MMA issuer     : one elected thread issues tcgen05.mma into a TMEM accumulator and
//                                commits completion to the stage's "empty" barrier / the tile's "full" barrier
//   warps 2..5  epilogue       : tcgen05.ld the accumulator (each warp its own 32-lane quadrant), apply
//                                the fused epilogue, store
// Operands are K-major ("TN": A[M,K], B[N,K], the layout of activations x nn.Linear weights); tiles are
// 128 x BN x 64 bytes-of-K-per-row = one 128-byte swizzle span per row.
#pragma once
#include <cuda_bf16.h>

#include "mf_umma.cuh"

namespace mfk {

constexpr int BM = 128;          // tile rows (UMMA M, one TMEM lane per row)
constexpr int KSPAN = 128;       // bytes of K per stage row = the 128-byte swizzle span
constexpr int kGemmThreads = 192;

struct alignas(64) TmaPair {
    CUtensorMap a;
    CUtensorMap b;
};

// dynamic shared memory: [stage][A 16 KiB | B BROWS*128 B] then barriers. BROWS = BN, or BN / 2 where a CTA pair shares the tile
template <int BN, int STAGES, int BROWS = BN> struct GemmSmem {
    static constexpr int kABytes = BM * KSPAN;
    static constexpr int kBBytes = BROWS * KSPAN;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarOff = STAGES * kStageBytes;
    // epilogue staging: each of the 4 epilogue warps turns 32 rows x 64 columns of bf16 around (one row per lane
    // out of TMEM -> 128 contiguous bytes per row on the way to memory); rows are padded to 144 bytes so that
    // both the per-lane row writes and the 8-lanes-per-row reads are free of bank conflicts
    static constexpr int kOutRowBytes = 144;
    static constexpr int kOutWarpBytes = 32 * kOutRowBytes;
    static constexpr int kOutOff = kBarOff + 1024;
    static constexpr int kOutBytes = 20480;  // >= 4 x kOutWarpBytes (bf16 GEMM) and >= 8 x 32 x 80 (fp8 GEMM, 8 warps x 32 columns)
    static constexpr int kTotal = kOutOff + kOutBytes;
    uint8_t *base;
    __device__ explicit GemmSmem(uint8_t *raw) : base(reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023)) {}
    __device__ uint8_t *a(int s) const { return base + s * kStageBytes; }
    __device__ uint8_t *b(int s) const { return base + s * kStageBytes + kABytes; }
    __device__ uint64_t *full(int s) const { return reinterpret_cast<uint64_t *>(base + kBarOff) + s; }
    __device__ uint64_t *empty(int s) const { return reinterpret_cast<uint64_t *>(base + kBarOff) + STAGES + s; }
    __device__ uint64_t *tfull(int i) const { return reinterpret_cast<uint64_t *>(base + kBarOff) + 2 * STAGES + i; }
    __device__ uint64_t *tempty(int i) const { return reinterpret_cast<uint64_t *>(base + kBarOff) + 2 * STAGES + 4 + i; }
    __device__ uint32_t *tmem_slot() const { return reinterpret_cast<uint32_t *>(base + kBarOff + 512); }
    __device__ uint8_t *out_stage(int epi_warp) const { return base + kOutOff + epi_warp * kOutWarpBytes; }
    __device__ volatile int *abort_flag() const { return reinterpret_cast<volatile int *>(base + kBarOff + 520); }
    static constexpr int kDynBytes = kTotal + 1024;  // slack for the 1024-byte alignment
};

struct PipeState {
    int stage = 0;
    uint32_t phase = 0;
    template <int STAGES> __device__ void advance()
    {
        if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
        }
    }
};

// Host: 2-D tensor map over a row-major [rows, cols_bytes / elem] matrix, box = (KSPAN bytes, box_rows), 128B swizzle.
int make_tmap_2d(CUtensorMap *out, const void *base, int elem_bytes, uint64_t rows, uint64_t cols, uint64_t row_stride_bytes,
                 uint32_t box_rows, bool is_fp8);

}  // namespace mfk
