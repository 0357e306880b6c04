// Fast Walsh-Hadamard transform along the last dim, with an optional fused
// per-row absmax quantizer epilogue (the producer of the 8-bit GEMM operand).
//
// Arithmetic contract (csrc/fast_hadamard/fast_hadamard_transform_common.h:86-161
// of the reference): fp32 butterflies (a+b, a-b) applied for stride 1, 2, 4, ...
// in ascending order, then one multiply by `scale` and the output cast.  Every
// butterfly is one fp32 add, so any schedule that keeps the stage order gives the
// same bits.
//
// Two schedules, both one pass over HBM:
//  * rows of <= 256 elements: a group of G = n/8 lanes owns a row (8 elements
//    per lane, one 16-byte load), 32/G rows per warp; stages 0-2 in registers,
//    the rest by xor-shuffles inside the group.
//  * rows of 512 .. 16384 elements: warp `a` of the CTA owns elements
//    [512a, 512a+512), 16 consecutive elements per lane; stages 0-3 in
//    registers, 4-8 by xor-shuffles, then one swizzled shared-memory exchange
//    after which each thread holds all `A` values of a few columns and finishes
//    stages 9+ in registers, storing straight from that layout.

#include <type_traits>
#include "common.cuh"

namespace q8k {

enum class Epilogue { Cast, Quant };

template <int N>
__device__ __forceinline__ void fwht_regs(float (&v)[N]) {
#pragma unroll
    for (int s = 1; s < N; s <<= 1) {
#pragma unroll
        for (int j = 0; j < N / 2; ++j) {
            const int lo = j & (s - 1);
            const int i = ((j - lo) << 1) + lo;
            const float a = v[i], b = v[i + s];
            v[i] = __fadd_rn(a, b);
            v[i + s] = __fsub_rn(a, b);
        }
    }
}

// One butterfly stage between lanes that differ in bit `mask`.
template <int N>
__device__ __forceinline__ void fwht_lanes(float (&v)[N], int lane, int mask) {
    const bool upper = (lane & mask) != 0;
#pragma unroll
    for (int i = 0; i < N; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, v[i], mask);
        v[i] = upper ? __fsub_rn(other, v[i]) : __fadd_rn(v[i], other);
    }
}

// Round the scaled transform to the dtype the unfused chain would have stored.
template <typename T> __device__ __forceinline__ float round_through(float v) {
    return to_float<T>(from_float<T>(v));
}

template <typename Tq> __device__ __forceinline__ uint8_t quantize_one(float y) {
    if constexpr (std::is_same_v<Tq, int8_t>) return (uint8_t)(int8_t)(int)roundf(y);
    else return float_to_e4m3_c10(y);
}

template <int N> struct ByteVec;
template <> struct ByteVec<1>  { using type = uint8_t; };
template <> struct ByteVec<2>  { using type = uint16_t; };
template <> struct ByteVec<4>  { using type = uint32_t; };
template <> struct ByteVec<8>  { using type = uint2; };
template <> struct ByteVec<16> { using type = uint4; };

template <typename T, int N>
__device__ __forceinline__ void store_elems(T* p, const float (&v)[N]) {
    using V = typename ByteVec<N * sizeof(T)>::type;
    union { V vec; T e[N]; } u;
#pragma unroll
    for (int i = 0; i < N; ++i) u.e[i] = from_float<T>(v[i]);
    *reinterpret_cast<V*>(p) = u.vec;
}

template <typename Tq, int N>
__device__ __forceinline__ void store_quant(Tq* p, const float (&v)[N], float qscale, bool zero_row) {
    using V = typename ByteVec<N>::type;
    union { V vec; uint8_t b[N]; } u;
#pragma unroll
    for (int i = 0; i < N; ++i) u.b[i] = quantize_one<Tq>(zero_row ? 0.f : __fmul_rn(v[i], qscale));
    *reinterpret_cast<V*>(p) = u.vec;
}

// ------------------------------------------------------------------ small rows
// LOG_G = log2(lanes per row).  Tout is the cast output type (Cast) or the
// quantised type (Quant: int8_t or e4m3_t).
template <typename Tin, typename Tout, int LOG_G, Epilogue EPI>
__global__ void __launch_bounds__(128)
hadamard_small_kernel(const Tin* __restrict__ x, Tout* __restrict__ out, float* __restrict__ scales,
                      int64_t rows, int dim, int64_t x_row_stride, float scale) {
    constexpr int G = 1 << LOG_G;
    constexpr int ROWS_PER_CTA = 128 / G;
    const int lane = threadIdx.x & 31;
    const int sub = threadIdx.x & (G - 1);
    const int64_t row = (int64_t)blockIdx.x * ROWS_PER_CTA + (threadIdx.x >> LOG_G);
    const bool row_ok = row < rows;
    const int e = sub * 8;

    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    if (row_ok && e < dim) load_vec<Tin, 8>(x + row * x_row_stride + e, v);

    fwht_regs<8>(v);
#pragma unroll
    for (int m = 1; m < G; m <<= 1) fwht_lanes<8>(v, lane, m);

    if constexpr (EPI == Epilogue::Cast) {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(v[j], scale);
        if (row_ok && e < dim) store_elems<Tout, 8>(out + row * (int64_t)dim + e, v);
    } else {
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] = round_through<Tin>(__fmul_rn(v[j], scale));
            if (e + j < dim) amax = fmaxf(amax, fabsf(v[j]));
        }
#pragma unroll
        for (int m = 1; m < G; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        const float qmax = std::is_same_v<Tout, int8_t> ? 127.0f : 448.0f;
        const float qscale = __fdiv_rn(qmax, amax);
        if (row_ok && e < dim) store_quant<Tout, 8>(out + row * (int64_t)dim + e, v, qscale, amax == 0.f);
        if (row_ok && sub == 0) scales[row] = __fdiv_rn(1.0f, qscale);
    }
}

// ------------------------------------------------------------------ large rows
__device__ __forceinline__ int swizzle_chunk(int q) {          // q = float4 index inside a 512-float warp-row
    return (q & ~3) | ((q & 3) ^ ((q >> 3) & 3));
}

template <typename Tin, typename Tout, int LOG_A, Epilogue EPI>
__global__ void __launch_bounds__(32 << LOG_A)
hadamard_large_kernel(const Tin* __restrict__ x, Tout* __restrict__ out, float* __restrict__ scales,
                      int dim, int64_t x_row_stride, float scale) {
    constexpr int A = 1 << LOG_A;                  // warps per CTA == 512-element segments per row
    constexpr int T = 32 * A;
    constexpr int NB = (A <= 16) ? 16 / A : 1;     // columns per thread after the exchange
    constexpr int ACTIVE = 512 / NB;               // threads that own columns after the exchange
    extern __shared__ __align__(16) float xch[];   // [A][512], float4 chunks swizzled
    __shared__ float red[32];

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int64_t row = blockIdx.x;
    const Tin* xr = x + row * x_row_stride;
    const int e0 = warp * 512 + lane * 16;

    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = 0.f;
    {
        float h[8];
        if (e0 < dim) {
            load_vec<Tin, 8>(xr + e0, h);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = h[j];
        }
        if (e0 + 8 < dim) {
            load_vec<Tin, 8>(xr + e0 + 8, h);
#pragma unroll
            for (int j = 0; j < 8; ++j) v[8 + j] = h[j];
        }
    }

    fwht_regs<16>(v);
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) fwht_lanes<16>(v, lane, m);

    if constexpr (A == 1) {
        // the whole row lives in one warp: finish from the load layout
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            v[j] = __fmul_rn(v[j], scale);
            if constexpr (EPI == Epilogue::Quant) {
                v[j] = round_through<Tin>(v[j]);
                if (e0 + j < dim) amax = fmaxf(amax, fabsf(v[j]));
            }
        }
        float lo[8], hi[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { lo[j] = v[j]; hi[j] = v[8 + j]; }
        if constexpr (EPI == Epilogue::Cast) {
            Tout* o = out + row * (int64_t)dim + e0;
            if (e0 < dim) store_elems<Tout, 8>(o, lo);
            if (e0 + 8 < dim) store_elems<Tout, 8>(o + 8, hi);
        } else {
            amax = warp_max(amax);
            const float qmax = std::is_same_v<Tout, int8_t> ? 127.0f : 448.0f;
            const float qscale = __fdiv_rn(qmax, amax);
            Tout* o = out + row * (int64_t)dim + e0;
            if (e0 < dim) store_quant<Tout, 8>(o, lo, qscale, amax == 0.f);
            if (e0 + 8 < dim) store_quant<Tout, 8>(o + 8, hi, qscale, amax == 0.f);
            if (lane == 0) scales[row] = __fdiv_rn(1.0f, qscale);
        }
        return;
    } else {
        // exchange: thread (warp, lane) publishes its 16 values, then thread `tid`
        // collects columns [tid*NB, tid*NB+NB) of every segment.
        float4* xch4 = reinterpret_cast<float4*>(xch);
#pragma unroll
        for (int c = 0; c < 4; ++c)
            xch4[warp * 128 + swizzle_chunk(lane * 4 + c)] = make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
        __syncthreads();

        const int tid = threadIdx.x;
        const bool active = tid < ACTIVE;
        const int b0 = tid * NB;                    // first column owned
        float w[NB][A];                             // w[i][a] = value of column b0+i in segment a
        if (active) {
#pragma unroll
            for (int a = 0; a < A; ++a) {
                if constexpr (NB >= 4) {
#pragma unroll
                    for (int c = 0; c < NB / 4; ++c) {
                        const float4 f = xch4[a * 128 + swizzle_chunk(b0 / 4 + c)];
                        w[4 * c][a] = f.x; w[4 * c + 1][a] = f.y; w[4 * c + 2][a] = f.z; w[4 * c + 3][a] = f.w;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < NB; ++i) {
                        const int b = b0 + i;
                        w[i][a] = xch[a * 512 + swizzle_chunk(b >> 2) * 4 + (b & 3)];
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < NB; ++i) fwht_regs<A>(w[i]);
        }

        float amax = 0.f;
        if (active) {
#pragma unroll
            for (int i = 0; i < NB; ++i)
#pragma unroll
                for (int a = 0; a < A; ++a) {
                    w[i][a] = __fmul_rn(w[i][a], scale);
                    if constexpr (EPI == Epilogue::Quant) {
                        w[i][a] = round_through<Tin>(w[i][a]);
                        if (a * 512 + b0 + i < dim) amax = fmaxf(amax, fabsf(w[i][a]));
                    }
                }
        }
        float qscale = 0.f;
        bool zero_row = false;
        if constexpr (EPI == Epilogue::Quant) {
            amax = warp_max(amax);
            if (lane == 0) red[warp] = amax;
            __syncthreads();
            amax = red[0];
#pragma unroll
            for (int k = 1; k < A; ++k) amax = fmaxf(amax, red[k]);
            const float qmax = std::is_same_v<Tout, int8_t> ? 127.0f : 448.0f;
            qscale = __fdiv_rn(qmax, amax);
            zero_row = amax == 0.f;
            if (tid == 0) scales[row] = __fdiv_rn(1.0f, qscale);
        }
        if (active) {
#pragma unroll
            for (int a = 0; a < A; ++a) {
                const int e = a * 512 + b0;
                if (e < dim) {                      // dim % 8 == 0 and NB <= 8: a chunk never straddles dim
                    float o[NB];
#pragma unroll
                    for (int i = 0; i < NB; ++i) o[i] = w[i][a];
                    if constexpr (EPI == Epilogue::Cast) store_elems<Tout, NB>(out + row * (int64_t)dim + e, o);
                    else store_quant<Tout, NB>(out + row * (int64_t)dim + e, o, qscale, zero_row);
                }
            }
        }
    }
}

// ------------------------------------------------------------------ dispatch
template <typename Tin, typename Tout, Epilogue EPI>
static int launch_hadamard(const void* x, void* out, float* scales, int64_t rows, int dim,
                           int64_t stride, float scale, cudaStream_t st, const char* op) {
    int log_n = 3;
    while ((1 << log_n) < dim) ++log_n;
    const Tin* xi = (const Tin*)x;
    Tout* o = (Tout*)out;
    if (log_n <= 8) {
        const int log_g = log_n - 3;
        const int rows_per_cta = 128 >> log_g;
        const unsigned grid = (unsigned)((rows + rows_per_cta - 1) / rows_per_cta);
#define Q8K_HS(LG) case LG: hadamard_small_kernel<Tin, Tout, LG, EPI><<<grid, 128, 0, st>>>(xi, o, scales, rows, dim, stride, scale); break
        switch (log_g) { Q8K_HS(0); Q8K_HS(1); Q8K_HS(2); Q8K_HS(3); Q8K_HS(4); Q8K_HS(5); }
#undef Q8K_HS
    } else {
        const int log_a = log_n - 9;
        if (log_a > 5) { set_error_detail("%s: dim %d exceeds 16384", op, dim); return Q8K_ERR_UNSUPPORTED; }
        const size_t smem = (size_t)(512 << log_a) * sizeof(float);
#define Q8K_HL(LA)                                                                                        \
    case LA: {                                                                                            \
        auto kern = hadamard_large_kernel<Tin, Tout, LA, EPI>;                                            \
        if (smem > 48 * 1024)                                                                             \
            Q8K_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        kern<<<(unsigned)rows, 32 << LA, (LA == 0 ? 0 : smem), st>>>(xi, o, scales, dim, stride, scale);    \
    } break
        switch (log_a) { Q8K_HL(0); Q8K_HL(1); Q8K_HL(2); Q8K_HL(3); Q8K_HL(4); Q8K_HL(5); }
#undef Q8K_HL
    }
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

static int check_hadamard_args(const char* op, const void* x, int x_dtype, const void* out, int64_t rows,
                               int dim, int64_t stride) {
    Q8K_REQUIRE(rows >= 0 && rows <= 0x7fffffffLL, Q8K_ERR_INVALID_ARG, "%s: rows %lld out of range", op, (long long)rows);
    Q8K_REQUIRE(dim > 0 && dim % 8 == 0, Q8K_ERR_INVALID_ARG, "%s: dim %d must be a positive multiple of 8", op, dim);
    Q8K_REQUIRE(dim <= 16384, Q8K_ERR_UNSUPPORTED, "%s: dim %d exceeds 16384", op, dim);
    if (rows == 0) return Q8K_OK;
    Q8K_REQUIRE(x && out, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE(x_dtype == Q8K_DT_BF16 || x_dtype == Q8K_DT_E4M3, Q8K_ERR_UNSUPPORTED,
                "%s: input dtype %d is not bf16 or e4m3", op, x_dtype);
    const int in_align = x_dtype == Q8K_DT_BF16 ? 16 : 8;
    Q8K_REQUIRE((reinterpret_cast<uintptr_t>(x) % in_align) == 0 && (stride * dtype_size(x_dtype)) % in_align == 0 && stride >= dim,
                Q8K_ERR_INVALID_ARG, "%s: x must be %d-byte aligned with a row stride >= dim that keeps rows aligned", op, in_align);
    Q8K_REQUIRE(aligned16(out), Q8K_ERR_INVALID_ARG, "%s: out must be 16-byte aligned", op);
    return Q8K_OK;
}

}  // namespace q8k

using namespace q8k;

extern "C" int q8k_fast_hadamard_transform(const void* x, int x_dtype, void* out, int out_dtype,
                                           int64_t rows, int dim, int64_t x_row_stride, float scale,
                                           void* stream) {
    const char* op = "fast_hadamard_transform";
    if (int rc = check_hadamard_args(op, x, x_dtype, out, rows, dim, x_row_stride)) return rc;
    if (rows == 0) return Q8K_OK;
    cudaStream_t st = (cudaStream_t)stream;
    constexpr Epilogue C = Epilogue::Cast;
    if (x_dtype == Q8K_DT_BF16 && out_dtype == Q8K_DT_BF16) return launch_hadamard<__nv_bfloat16, __nv_bfloat16, C>(x, out, nullptr, rows, dim, x_row_stride, scale, st, op);
    if (x_dtype == Q8K_DT_BF16 && out_dtype == Q8K_DT_E4M3) return launch_hadamard<__nv_bfloat16, e4m3_t, C>(x, out, nullptr, rows, dim, x_row_stride, scale, st, op);
    if (x_dtype == Q8K_DT_E4M3 && out_dtype == Q8K_DT_BF16) return launch_hadamard<e4m3_t, __nv_bfloat16, C>(x, out, nullptr, rows, dim, x_row_stride, scale, st, op);
    if (x_dtype == Q8K_DT_E4M3 && out_dtype == Q8K_DT_E4M3) return launch_hadamard<e4m3_t, e4m3_t, C>(x, out, nullptr, rows, dim, x_row_stride, scale, st, op);
    set_error_detail("%s: output dtype %d is not bf16 or e4m3", op, out_dtype);
    return Q8K_ERR_UNSUPPORTED;
}

extern "C" int q8k_hadamard_quant(const void* x, int x_dtype, void* q, int q_dtype, float* scales,
                                  int64_t rows, int dim, int64_t x_row_stride, float scale, void* stream) {
    const char* op = "hadamard_quant";
    if (int rc = check_hadamard_args(op, x, x_dtype, q, rows, dim, x_row_stride)) return rc;
    if (rows == 0) return Q8K_OK;
    Q8K_REQUIRE(scales != nullptr, Q8K_ERR_INVALID_ARG, "%s: null scales pointer", op);
    cudaStream_t st = (cudaStream_t)stream;
    constexpr Epilogue Q = Epilogue::Quant;
    if (x_dtype == Q8K_DT_BF16 && q_dtype == Q8K_DT_I8)   return launch_hadamard<__nv_bfloat16, int8_t, Q>(x, q, scales, rows, dim, x_row_stride, scale, st, op);
    if (x_dtype == Q8K_DT_BF16 && q_dtype == Q8K_DT_E4M3) return launch_hadamard<__nv_bfloat16, e4m3_t, Q>(x, q, scales, rows, dim, x_row_stride, scale, st, op);
    if (x_dtype == Q8K_DT_E4M3 && q_dtype == Q8K_DT_I8)   return launch_hadamard<e4m3_t, int8_t, Q>(x, q, scales, rows, dim, x_row_stride, scale, st, op);
    if (x_dtype == Q8K_DT_E4M3 && q_dtype == Q8K_DT_E4M3) return launch_hadamard<e4m3_t, e4m3_t, Q>(x, q, scales, rows, dim, x_row_stride, scale, st, op);
    set_error_detail("%s: quantised dtype %d is not int8 or e4m3", op, q_dtype);
    return Q8K_ERR_UNSUPPORTED;
}
