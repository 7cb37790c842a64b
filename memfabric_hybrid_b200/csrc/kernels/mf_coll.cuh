// Element helpers of the collective kernels: 16-byte vectors of bf16 / fp16 / fp32 / int32, fp32
// accumulation, reduce operators, and the fused scale + cast epilogue.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "mf_team.cuh"

namespace mfk {

enum DType : int { DT_BF16 = 0, DT_F16 = 1, DT_F32 = 2, DT_I32 = 3 };
enum RedOp : int { OP_SUM = 0, OP_MAX = 1, OP_MIN = 2, OP_PROD = 3 };

template <typename T> struct Vec;  // 16 bytes of T, convertible to/from float lanes
template <> struct Vec<float> {
    static constexpr int N = 4;
    __device__ static void unpack(const uint4 &r, float (&f)[4])
    {
        f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
    }
    __device__ static void load(const float *p, float (&f)[4]) { unpack(__ldcg(reinterpret_cast<const uint4 *>(p)), f); }
    __device__ static void store(float *p, const float (&f)[4]) { *reinterpret_cast<float4 *>(p) = make_float4(f[0], f[1], f[2], f[3]); }
    __device__ static float to_f(float v) { return v; }
    __device__ static float from_f(float v) { return v; }
};
template <> struct Vec<int> {
    static constexpr int N = 4;
    // int32 travels through fp32 lanes only for |v| < 2^24; the integer kernels use their own exact path
    __device__ static void unpack(const uint4 &r, float (&f)[4])
    {
        f[0] = __uint_as_float(r.x); f[1] = __uint_as_float(r.y); f[2] = __uint_as_float(r.z); f[3] = __uint_as_float(r.w);
    }
    __device__ static void load(const int *p, float (&f)[4]) { unpack(__ldcg(reinterpret_cast<const uint4 *>(p)), f); }
    __device__ static void store(int *p, const float (&f)[4])
    {
        *reinterpret_cast<int4 *>(p) = make_int4(__float_as_int(f[0]), __float_as_int(f[1]), __float_as_int(f[2]), __float_as_int(f[3]));
    }
    __device__ static float to_f(int v) { return __int_as_float(v); }
    __device__ static int from_f(float v) { return __float_as_int(v); }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16 *p, float (&f)[8]) { unpack(__ldcg(reinterpret_cast<const uint4 *>(p)), f); }
    __device__ static void unpack(const uint4 &v, float (&f)[8])
    {
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 x = __bfloat1622float2(h[i]);
            f[2 * i] = x.x;
            f[2 * i + 1] = x.y;
        }
    }
    __device__ static void store(__nv_bfloat16 *p, const float (&f)[8])
    {
        uint4 v;
        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        *reinterpret_cast<uint4 *>(p) = v;
    }
    __device__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};
template <> struct Vec<__half> {
    static constexpr int N = 8;
    __device__ static void load(const __half *p, float (&f)[8]) { unpack(__ldcg(reinterpret_cast<const uint4 *>(p)), f); }
    __device__ static void unpack(const uint4 &v, float (&f)[8])
    {
        const __half2 *h = reinterpret_cast<const __half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            float2 x = __half22float2(h[i]);
            f[2 * i] = x.x;
            f[2 * i + 1] = x.y;
        }
    }
    __device__ static void store(__half *p, const float (&f)[8])
    {
        uint4 v;
        __half2 *h = reinterpret_cast<__half2 *>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        *reinterpret_cast<uint4 *>(p) = v;
    }
    __device__ static float to_f(__half v) { return __half2float(v); }
    __device__ static __half from_f(float v) { return __float2half_rn(v); }
};

template <bool INT> __device__ __forceinline__ float red_apply(float a, float b, int op)
{
    if (INT) {
        int x = __float_as_int(a), y = __float_as_int(b), r;
        switch (op) {
            case OP_MAX: r = max(x, y); break;
            case OP_MIN: r = min(x, y); break;
            case OP_PROD: r = x * y; break;
            default: r = x + y; break;
        }
        return __int_as_float(r);
    }
    switch (op) {
        case OP_MAX: return fmaxf(a, b);
        case OP_MIN: return fminf(a, b);
        case OP_PROD: return a * b;
        default: return a + b;
    }
}

}  // namespace mfk
