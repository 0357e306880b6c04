// Pieces shared by the single-CTA and the CTA-pair 8-bit GEMM kernels.
#pragma once

#include "common.cuh"
#include "tcgen05.cuh"
#include "tensormap.cuh"

namespace q8k {

constexpr int kGemmBM = 128;
constexpr int kGemmBK = 128;          // bytes == elements along K per stage
constexpr int kGemmEpilogueThreads = 256;
constexpr int kGemmThreads = 64 + kGemmEpilogueThreads;

struct GemmParams {
    const float* a_scales;
    const float* b_scales;
    const float* bias;
    void* out;
    int* status;
    int M, N, K;
    int batch_a, batch_b;             // 1 when that operand carries a batch dim
    int m_tiles, n_tiles, total_tiles;
    // optional fused tail (bf16 output only): out = bf16(bf16(gate[row / rows_per_gate, n] * y) + resid[row, n])
    const __nv_bfloat16* resid;
    const __nv_bfloat16* gate;        // may be null: plain residual add
    int64_t rows_per_gate;
};

__device__ __forceinline__ float gelu_tanh_fast(float y) {
    // tanh.approx has ~2^-11 absolute error, far below the bf16 / e4m3 output step.
    const float u = 0.7978845608028654f * fmaf(0.044715f * y * y, y, y);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
    return 0.5f * y * (1.0f + t);
}

// Same function on a pair of adjacent columns with packed fp32 instructions (6 issue slots + 2
// tanh for two outputs): 0.5 y (1 + tanh(y (k0 + k0 k1 y^2))).
__device__ __forceinline__ float2 gelu_tanh_fast2(float2 y) {
    const float2 p = ffma2(fmul2(y, y), make_float2(0.7978845608028654f * 0.044715f, 0.7978845608028654f * 0.044715f),
                           make_float2(0.7978845608028654f, 0.7978845608028654f));
    const float2 u = fmul2(p, y);
    float2 t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.x) : "f"(u.x));
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.y) : "f"(u.y));
    const float2 h = fmul2(y, make_float2(0.5f, 0.5f));
    return ffma2(h, t, h);
}

// Epilogue arithmetic of one row on two adjacent columns: acc * (sa * sb[n]) + bias[n], then the
// optional GELU.  r0, r1 are the raw 32-bit accumulator words (int32 or fp32); sb / bias point
// at the pair's column in shared memory (8-byte aligned).
template <bool INT8, bool GELU>
__device__ __forceinline__ float2 epilogue_pair(uint32_t r0, uint32_t r1, float2 sa2, const float* sb, const float* bias) {
    const float2 acc = INT8 ? make_float2((float)(int)r0, (float)(int)r1)
                            : make_float2(__uint_as_float(r0), __uint_as_float(r1));
    float2 y = ffma2(acc, fmul2(sa2, *reinterpret_cast<const float2*>(sb)), *reinterpret_cast<const float2*>(bias));
    if constexpr (GELU) y = gelu_tanh_fast2(y);
    return y;
}

int gemm_num_sms();

// CTA-pair (cta_group::2) variant: 256 x 256 output tiles per cluster of two CTAs.  Returns
// Q8K_ERR_UNSUPPORTED (without touching the error detail) when the device cannot co-schedule
// the clusters, in which case the caller falls back to the single-CTA kernel.
int launch_gemm_pair(bool int8, bool gelu, bool out_e4m3, bool resid, const void* a, const void* b, const GemmParams& p,
                     int bs_a, int bs_b, cudaStream_t st);

}  // namespace q8k
