// Shared helpers for the sm_100a kernels: error reporting for the C ABI,
// element-type tags, 8-bit casts with the two rounding flavours the reference
// uses, and small vector load/store utilities.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/q8_kernels_b200.h"

namespace q8k {

// ---------------------------------------------------------------- host-side errors
void set_error_detail(const char* fmt, ...);

#define Q8K_REQUIRE(cond, code, ...)                      \
    do {                                                  \
        if (!(cond)) {                                    \
            q8k::set_error_detail(__VA_ARGS__);           \
            return (code);                                \
        }                                                 \
    } while (0)

#define Q8K_CUDA_OK(expr)                                                          \
    do {                                                                           \
        cudaError_t _e = (expr);                                                   \
        if (_e != cudaSuccess) {                                                   \
            q8k::set_error_detail("%s failed: %s", #expr, cudaGetErrorString(_e)); \
            return Q8K_ERR_CUDA;                                                   \
        }                                                                          \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---------------------------------------------------------------- element types
struct e4m3_t { uint8_t bits; };

template <int DT> struct DType;
template <> struct DType<Q8K_DT_F32>  { using type = float; };
template <> struct DType<Q8K_DT_F16>  { using type = __half; };
template <> struct DType<Q8K_DT_BF16> { using type = __nv_bfloat16; };
template <> struct DType<Q8K_DT_E4M3> { using type = e4m3_t; };
template <> struct DType<Q8K_DT_I8>   { using type = int8_t; };

inline int dtype_size(int dt) {
    switch (dt) {
        case Q8K_DT_F32: return 4;
        case Q8K_DT_F16: case Q8K_DT_BF16: return 2;
        case Q8K_DT_E4M3: case Q8K_DT_I8: return 1;
        default: return 0;
    }
}

// ---------------------------------------------------------------- scalar conversions
__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
    return __half2float(__half(h));
}

// fp32 -> e4m3, round to nearest even, saturating to +-448 (cvt.rn.satfinite).
// Used by the GEMM epilogue and inside attention.
__device__ __forceinline__ uint8_t float_to_e4m3_sat(float x) {
    return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ uint16_t float2_to_e4m3x2_sat(float lo, float hi) {
    return (uint16_t)__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3);
}

// fp32 -> e4m3 the way the c10 software cast does it: round to nearest even,
// and anything that rounds beyond 448 (|x| > 464, inf, NaN) becomes NaN with
// the sign kept.  For |x| <= 464 this equals the saturating hardware cast.
__device__ __forceinline__ uint8_t float_to_e4m3_c10(float x) {
    uint8_t r = float_to_e4m3_sat(x);
    const bool overflow = !(fabsf(x) <= 464.0f);          // true for NaN as well
    if (overflow) r = (uint8_t)(0x7F | ((__float_as_uint(x) >> 24) & 0x80));
    return r;
}

// Eight values at once, same bytes as float_to_e4m3_c10 on each: four packed saturating conversions, and
// only if some |x| exceeds 464 or a NaN went in (the conversion returns 0x7F for it, whatever its sign)
// the element-wise form.
__device__ __forceinline__ uint2 pack8_e4m3_c10(const float (&x)[8]) {
    uint2 w;
    w.x = (uint32_t)float2_to_e4m3x2_sat(x[0], x[1]) | ((uint32_t)float2_to_e4m3x2_sat(x[2], x[3]) << 16);
    w.y = (uint32_t)float2_to_e4m3x2_sat(x[4], x[5]) | ((uint32_t)float2_to_e4m3x2_sat(x[6], x[7]) << 16);
    const float m = fmaxf(fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3]))),
                          fmaxf(fmaxf(fabsf(x[4]), fabsf(x[5])), fmaxf(fabsf(x[6]), fabsf(x[7]))));
    const uint32_t nan_bytes = (((w.x & 0x7f7f7f7fu) + 0x01010101u) | ((w.y & 0x7f7f7f7fu) + 0x01010101u)) & 0x80808080u;
    if (m > 464.0f || nan_bytes != 0u) {
        union { uint2 v; uint8_t b[8]; } o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.b[j] = float_to_e4m3_c10(x[j]);
        w = o.v;
    }
    return w;
}

// Both values rounded to bf16 (nearest even) and widened again: one packed conversion and two bit moves.
__device__ __forceinline__ void round_through_bf16x2(float& a, float& b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&h);
    a = __uint_as_float(w << 16);
    b = __uint_as_float(w & 0xffff0000u);
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_float<e4m3_t>(e4m3_t v) { return e4m3_to_float(v.bits); }
template <> __device__ __forceinline__ float to_float<int8_t>(int8_t v) { return (float)v; }

// "plain C++ conversion" of the SIMT ops: bf16/fp16 RNE, e4m3 c10-style.
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ e4m3_t from_float<e4m3_t>(float v) { return e4m3_t{float_to_e4m3_c10(v)}; }

// ---------------------------------------------------------------- vector access
// N consecutive elements of T <-> fp32 registers.  N * sizeof(T) must be 4, 8,
// 16 or 32 bytes and the address aligned to min(16, N*sizeof(T)).
template <int BYTES> struct Vec;
template <> struct Vec<2>  { using type = uint16_t; };
template <> struct Vec<4>  { using type = uint32_t; };
template <> struct Vec<8>  { using type = uint2; };
template <> struct Vec<16> { using type = uint4; };

template <typename T, int N>
__device__ __forceinline__ void load_vec(const T* __restrict__ p, float (&out)[N]) {
    constexpr int BYTES = N * sizeof(T);
    if constexpr (BYTES <= 16) {
        using V = typename Vec<BYTES>::type;
        union { V v; T e[N]; } u;
        u.v = *reinterpret_cast<const V*>(p);
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = to_float<T>(u.e[i]);
    } else {
        static_assert(BYTES % 16 == 0, "vector width");
        constexpr int PER = 16 / sizeof(T);
#pragma unroll
        for (int c = 0; c < BYTES / 16; ++c) {
            union { uint4 v; T e[PER]; } u;
            u.v = reinterpret_cast<const uint4*>(p)[c];
#pragma unroll
            for (int i = 0; i < PER; ++i) out[c * PER + i] = to_float<T>(u.e[i]);
        }
    }
}

template <typename T, int N>
__device__ __forceinline__ void store_vec(T* __restrict__ p, const float (&in)[N]) {
    constexpr int BYTES = N * sizeof(T);
    if constexpr (BYTES <= 16) {
        using V = typename Vec<BYTES>::type;
        if constexpr (__is_same(T, __nv_bfloat16) && N % 2 == 0) {
            union { V v; __nv_bfloat162 e2[N / 2]; } u;
#pragma unroll
            for (int i = 0; i < N; i += 2) u.e2[i / 2] = __floats2bfloat162_rn(in[i], in[i + 1]);
            *reinterpret_cast<V*>(p) = u.v;
        } else {
            union { V v; T e[N]; } u;
#pragma unroll
            for (int i = 0; i < N; ++i) u.e[i] = from_float<T>(in[i]);
            *reinterpret_cast<V*>(p) = u.v;
        }
    } else {
        static_assert(BYTES % 16 == 0, "vector width");
        constexpr int PER = 16 / sizeof(T);
#pragma unroll
        for (int c = 0; c < BYTES / 16; ++c) {
            if constexpr (sizeof(T) == 2 && __is_same(T, __nv_bfloat16)) {
                union { uint4 v; __nv_bfloat162 e2[4]; } u;    // packed conversions, same rounding
#pragma unroll
                for (int i = 0; i < 8; i += 2) u.e2[i / 2] = __floats2bfloat162_rn(in[c * 8 + i], in[c * 8 + i + 1]);
                reinterpret_cast<uint4*>(p)[c] = u.v;
            } else {
                union { uint4 v; T e[PER]; } u;
#pragma unroll
                for (int i = 0; i < PER; ++i) u.e[i] = from_float<T>(in[c * PER + i]);
                reinterpret_cast<uint4*>(p)[c] = u.v;
            }
        }
    }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// sm_100 packed fp32 pairs: one issue slot does two lanes of FMA-pipe work, each lane rounded as
// the scalar instruction would be.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(d)
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
          "l"(*reinterpret_cast<unsigned long long*>(&c)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;"
        : "=l"(d)
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;"
        : "=l"(d)
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fsub2(float2 a, float2 b) {
    unsigned long long d;
    asm("sub.rn.f32x2 %0, %1, %2;"
        : "=l"(d)
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// tanh-GELU of the reference (csrc/gemm/q8_matmul_bias.cu:29-33).
__device__ __forceinline__ float gelu_tanh_precise(float x) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(u));
}

}  // namespace q8k
