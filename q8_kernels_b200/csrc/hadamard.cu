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
//  * rows of 512 .. 16384 elements: 16-64 threads per row with 32-128 values
//    each; the first 5-7 stages run in registers on consecutive elements, the
//    rest after one swizzled shared-memory exchange (two for 16384), all on
//    packed fp32 pairs; no shuffles.  Shared-memory traffic, not issue slots or
//    HBM, is what this schedule is sized for: 12 bytes per element in total.

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

// Two values at once: for bf16 one packed conversion (an ALU-pipe F2FP instead of two conversions on
// the 16-lane special-function unit) and two bit operations to widen the halves again.
template <typename T> __device__ __forceinline__ float2 round_through2(float a, float b) {
    if constexpr (std::is_same_v<T, __nv_bfloat16>) {
        const __nv_bfloat162 p = __floats2bfloat162_rn(a, b);  // a in the low half
        const uint32_t w = *reinterpret_cast<const uint32_t*>(&p);
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    } else {
        return make_float2(round_through<T>(a), round_through<T>(b));
    }
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
    if constexpr (std::is_same_v<T, __nv_bfloat16> && N % 2 == 0) {
        union { V vec; __nv_bfloat162 e2[N / 2]; } u;          // packed conversions, same rounding
#pragma unroll
        for (int i = 0; i < N; i += 2) u.e2[i / 2] = __floats2bfloat162_rn(v[i], v[i + 1]);
        *reinterpret_cast<V*>(p) = u.vec;
    } else {
        union { V vec; T e[N]; } u;
#pragma unroll
        for (int i = 0; i < N; ++i) u.e[i] = from_float<T>(v[i]);
        *reinterpret_cast<V*>(p) = u.vec;
    }
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
// One CTA per row of N = 2^LOG_N (padded) elements, T = N / V threads, V = 2^LOG_V values per
// thread.  The row is staged raw in shared memory by coalesced loads; each thread then owns V
// consecutive elements and runs stages 0 .. LOG_V-1 in registers.  The remaining stages run in
// phases of up to LOG_V-2 bits: the row is exchanged through shared memory (fp32, natural element
// order, float4 chunks XOR-swizzled so that both sides are conflict free) into a layout where a
// thread owns 2^b groups x C consecutive elements, the groups being the butterfly partners.
// Butterflies work on packed fp32 pairs (add/sub.f32x2), so a stage costs half an instruction per
// element; only the stride-1 stage is scalar.


__device__ __forceinline__ int swz4(int q) { return q ^ ((q >> 3) & 7); }      // float4-chunk swizzle

// Layout of a phase that butterflies bits [LO, LO+B): thread t owns groups j = 0 .. 2^B-1 of
// C = V >> B consecutive elements each.  The thread index supplies the other bits of the
// element index: its low LO-log2(C) bits sit below the group bits, the rest above them.
template <int LOG_V, int B, int LO>
struct PhaseLayout {
    static constexpr int LOG_C = LOG_V - B;
    static constexpr int C = 1 << LOG_C;
    static constexpr int G = 1 << B;
    static constexpr int BITS = B;
    static constexpr int LOW = LO;
    static_assert(LO >= LOG_C, "group bits must lie above the run bits");
    __device__ static __forceinline__ int elem(int t, int j) {
        constexpr int LOWT = LO - LOG_C;
        return ((t & ((1 << LOWT) - 1)) << LOG_C) + (j << LO) + ((t >> LOWT) << (LO + B));
    }
};

// Shared-memory exchange in natural element order, float4 chunks XOR-swizzled (swz4).  elem(t, j)
// is a bitwise OR of disjoint bit fields and swz4 is linear over XOR, so the swizzled byte offset of
// (t, j, k) is  offset(t) ^ offset(j, k)  with the second term a compile-time constant: one XOR per
// access instead of re-deriving the swizzle.  Runs of 2 use float2 accesses inside the chunk (the
// half-chunk select bit belongs to the thread term).
template <typename L>
__device__ __forceinline__ uint32_t exchange_thread_offset(int t) {
    const int e = L::elem(t, 0);
    uint32_t off = (uint32_t)swz4(e >> 2) << 4;
    if constexpr (L::C < 4) off |= (uint32_t)((e >> 1) & 1) << 3;
    return off;
}
template <typename L>
__device__ __forceinline__ constexpr uint32_t exchange_const_offset(int j, int k) {
    const int q = ((j << L::LOW) >> 2) + k;
    return (uint32_t)(q ^ ((q >> 3) & 7)) << 4;
}

// registers (layout L) -> shared memory
template <typename L, int V>
__device__ __forceinline__ void exchange_write(float* xch, const float (&v)[V], int t) {
    char* xb = reinterpret_cast<char*>(xch);
    const uint32_t tb = exchange_thread_offset<L>(t);
#pragma unroll
    for (int j = 0; j < L::G; ++j) {
        if constexpr (L::C >= 4) {
#pragma unroll
            for (int k = 0; k < L::C / 4; ++k)
                *reinterpret_cast<float4*>(xb + (tb ^ exchange_const_offset<L>(j, k))) =
                    make_float4(v[j * L::C + 4 * k], v[j * L::C + 4 * k + 1], v[j * L::C + 4 * k + 2], v[j * L::C + 4 * k + 3]);
        } else {
            *reinterpret_cast<float2*>(xb + (tb ^ exchange_const_offset<L>(j, 0))) = make_float2(v[j * 2], v[j * 2 + 1]);
        }
    }
}
template <typename L, int V>
__device__ __forceinline__ void exchange_read(const float* xch, float (&v)[V], int t) {
    const char* xb = reinterpret_cast<const char*>(xch);
    const uint32_t tb = exchange_thread_offset<L>(t);
#pragma unroll
    for (int j = 0; j < L::G; ++j) {
        if constexpr (L::C >= 4) {
#pragma unroll
            for (int k = 0; k < L::C / 4; ++k) {
                const float4 f = *reinterpret_cast<const float4*>(xb + (tb ^ exchange_const_offset<L>(j, k)));
                v[j * L::C + 4 * k] = f.x; v[j * L::C + 4 * k + 1] = f.y;
                v[j * L::C + 4 * k + 2] = f.z; v[j * L::C + 4 * k + 3] = f.w;
            }
        } else {
            const float2 f = *reinterpret_cast<const float2*>(xb + (tb ^ exchange_const_offset<L>(j, 0)));
            v[j * 2] = f.x; v[j * 2 + 1] = f.y;
        }
    }
}

// butterflies between groups (stride = whole groups of C >= 4 elements): all packed
template <typename L, int V>
__device__ __forceinline__ void butterfly_groups(float (&v)[V]) {
#pragma unroll
    for (int s = 0; s < L::BITS; ++s) {
        const int gs = 1 << s;
#pragma unroll
        for (int h = 0; h < L::G / 2; ++h) {
            const int lo = h & (gs - 1);
            const int j = ((h - lo) << 1) + lo;
#pragma unroll
            for (int c = 0; c < L::C; c += 2) {
                const float2 a = make_float2(v[j * L::C + c], v[j * L::C + c + 1]);
                const float2 b = make_float2(v[(j + gs) * L::C + c], v[(j + gs) * L::C + c + 1]);
                const float2 su = fadd2(a, b), di = fsub2(a, b);
                v[j * L::C + c] = su.x; v[j * L::C + c + 1] = su.y;
                v[(j + gs) * L::C + c] = di.x; v[(j + gs) * L::C + c + 1] = di.y;
            }
        }
    }
}

// stages 0 .. log2(V)-1 over V consecutive elements: stride 1 scalar, the rest packed
template <int V>
__device__ __forceinline__ void butterfly_consecutive(float (&v)[V]) {
#pragma unroll
    for (int i = 0; i < V; i += 2) {
        const float a = v[i], b = v[i + 1];
        v[i] = __fadd_rn(a, b);
        v[i + 1] = __fsub_rn(a, b);
    }
#pragma unroll
    for (int st = 2; st < V; st <<= 1) {
#pragma unroll
        for (int h = 0; h < V / 2; h += 2) {                   // h, h+1 index two adjacent butterflies
            const int lo = h & (st - 1);
            const int i = ((h - lo) << 1) + lo;
            const float2 a = make_float2(v[i], v[i + 1]);
            const float2 b = make_float2(v[i + st], v[i + st + 1]);
            const float2 su = fadd2(a, b), di = fsub2(a, b);
            v[i] = su.x; v[i + 1] = su.y;
            v[i + st] = di.x; v[i + st + 1] = di.y;
        }
    }
}

// Exact round-half-away-from-zero (C round()) of |y| < 2^22 with one add: adding the largest
// float below 0.5 with y's sign and truncating gives floor(|y| + 0.5) for every fp32 y, ties
// included (the sum of a tie k + 0.5 rounds up to k + 1, and 0.5 - 2^-25 stays below 1).
__device__ __forceinline__ int round_half_away_int(float y) {
    return __float2int_rz(__fadd_rn(y, copysignf(0.49999997f, y)));
}

template <typename Tq>
__device__ __forceinline__ uint8_t quantize_fast(float y) {
    if constexpr (std::is_same_v<Tq, int8_t>) return (uint8_t)(int8_t)round_half_away_int(y);
    else return float_to_e4m3_c10(y);
}

// Four quantised bytes from four fp32 values, lowest address first.  INT8: round half away from zero
// (one add + truncation each) and three byte permutes.  E4M3: two packed saturating conversions and
// one permute; the caller guarantees |y| <= 448 (1 + 2^-23) for finite rows (y = v * (448 / amax) with
// |v| <= amax), where the saturating cast and the c10 cast (overflow -> NaN beyond 464) agree, and a
// NaN stays a NaN in both.
template <typename Tq>
__device__ __forceinline__ uint32_t quantize_pack4(float y0, float y1, float y2, float y3) {
    if constexpr (std::is_same_v<Tq, int8_t>) {
        const uint32_t q0 = (uint32_t)round_half_away_int(y0), q1 = (uint32_t)round_half_away_int(y1);
        const uint32_t q2 = (uint32_t)round_half_away_int(y2), q3 = (uint32_t)round_half_away_int(y3);
        return __byte_perm(__byte_perm(q0, q1, 0x0040), __byte_perm(q2, q3, 0x0040), 0x5410);
    } else {
        return (uint32_t)float2_to_e4m3x2_sat(y0, y1) | ((uint32_t)float2_to_e4m3x2_sat(y2, y3) << 16);
    }
}

// NORM_MOD adds the block's pre-linear prologue in front of the transform, with the bf16 roundings
// of the separate ops it replaces: n = bf16(x * rsqrt(mean x^2)); u = bf16(bf16(n * bf16(1 + s)) + h)
// where s, h are the per-batch modulation rows (bf16 [rows / rows_per_mod, dim]).
// FULL: dim == 2^LOG_N, so no element of a row needs a bounds test.
template <typename Tin, typename Tout, int LOG_N, int LOG_V, int ROWS, Epilogue EPI, bool NORM_MOD = false, bool FULL = false>
__global__ void __launch_bounds__(ROWS << (LOG_N - LOG_V))
hadamard_row_kernel(const Tin* __restrict__ x, Tout* __restrict__ out, float* __restrict__ scales,
                    int64_t rows, int dim, int64_t x_row_stride, float scale,
                    const __nv_bfloat16* __restrict__ mod_scale = nullptr,
                    const __nv_bfloat16* __restrict__ mod_shift = nullptr, int64_t rows_per_mod = 1) {
    constexpr int N = 1 << LOG_N;
    constexpr int V = 1 << LOG_V;
    constexpr int T = N / V;                                   // threads per row
    constexpr int ITEMS = V / 8;                               // 8-element input items per thread
    constexpr int R = LOG_N - LOG_V;                           // bits left after the register phase
    // one exchange when the bits fit (runs of >= 2 consecutive elements), else two balanced ones so
    // that both keep runs of >= 4 (float4 accesses)
    constexpr int BMAX = LOG_V - 1;
    constexpr int B1 = R <= BMAX ? R : (R + 1) / 2;
    constexpr int B2 = R - B1;
    static_assert(B1 <= BMAX && B2 <= BMAX, "row too long for this values-per-thread choice");
    using L0 = PhaseLayout<LOG_V, 0, LOG_V>;                   // V consecutive elements
    using L1 = PhaseLayout<LOG_V, B1, LOG_V>;
    using L2 = PhaseLayout<LOG_V, B2, LOG_V + B1>;

    extern __shared__ __align__(16) float xch_all[];           // ROWS x N floats
    __shared__ float red[32];
    const int t = threadIdx.x % T;
    const int r_in_cta = threadIdx.x / T;
    const int64_t row = (int64_t)blockIdx.x * ROWS + r_in_cta;
    const bool row_ok = row < rows;
    float* xch = xch_all + r_in_cta * N;
    const Tin* xr = x + row * x_row_stride;

    // coalesced load of raw 8-element items into shared memory, then V consecutive elements per thread
    {
        using Item = typename Vec<8 * sizeof(Tin)>::type;
        Item* stage = reinterpret_cast<Item*>(xch);
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            const int item = t + k * T;
            Item val;
            if (row_ok && (FULL || item * 8 < dim)) val = *reinterpret_cast<const Item*>(xr + item * 8);
            else memset(&val, 0, sizeof(val));
            stage[item ^ ((item / ITEMS) & (ITEMS - 1))] = val;   // spread a thread's ITEMS reads over the banks
        }
    }
    __syncthreads();
    float v[V];
    {
        using Item = typename Vec<8 * sizeof(Tin)>::type;
        const Item* stage = reinterpret_cast<const Item*>(xch);
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            union { Item raw; Tin e[8]; } u;
            u.raw = stage[(t * ITEMS + (t & (ITEMS - 1))) ^ k];   // == (t * ITEMS + k) ^ (t % ITEMS)
#pragma unroll
            for (int j = 0; j < 8; ++j) v[k * 8 + j] = to_float<Tin>(u.e[j]);
        }
    }
    if constexpr (NORM_MOD) {
        static_assert(std::is_same_v<Tin, __nv_bfloat16>, "the norm + modulation prologue takes bf16 rows");
        __shared__ float red_ss[32];
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < V; ++i) ss = fmaf(v[i], v[i], ss);
#pragma unroll
        for (int m = 1; m < (T < 32 ? T : 32); m <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, m);
        if constexpr (T > 32) {
            constexpr int WPR = T / 32;
            if ((threadIdx.x & 31) == 0) red_ss[threadIdx.x >> 5] = ss;
            __syncthreads();
            ss = red_ss[r_in_cta * WPR];
#pragma unroll
            for (int k = 1; k < WPR; ++k) ss += red_ss[r_in_cta * WPR + k];
        }
        const float rr = rsqrtf(ss * (1.0f / (float)dim));
        const int64_t mrow = row_ok ? row / rows_per_mod : 0;
        const __nv_bfloat16* sc = mod_scale + mrow * dim + t * V;
        const __nv_bfloat16* sh = mod_shift + mrow * dim + t * V;
#pragma unroll
        for (int k = 0; k < ITEMS; ++k) {
            if (FULL || t * V + k * 8 < dim) {
                // packed bf16 arithmetic gives exactly the roundings of the separate ops: a product of two
                // bf16 values is exact in fp32, and a sum of two is either exact in fp32 or so lopsided that
                // both roundings return the larger operand; _rn keeps multiply and add from fusing
                const uint4 s8 = *reinterpret_cast<const uint4*>(sc + k * 8);
                const uint4 h8 = *reinterpret_cast<const uint4*>(sh + k * 8);
                const __nv_bfloat162 one2 = __floats2bfloat162_rn(1.0f, 1.0f);
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const uint32_t sw = j == 0 ? s8.x : (j == 2 ? s8.y : (j == 4 ? s8.z : s8.w));
                    const uint32_t hw = j == 0 ? h8.x : (j == 2 ? h8.y : (j == 4 ? h8.z : h8.w));
                    const float2 xr2 = fmul2(make_float2(v[k * 8 + j], v[k * 8 + j + 1]), make_float2(rr, rr));
                    const __nv_bfloat162 n = __floats2bfloat162_rn(xr2.x, xr2.y);
                    const __nv_bfloat162 m1 = __hadd2_rn(one2, *reinterpret_cast<const __nv_bfloat162*>(&sw));
                    const __nv_bfloat162 u = __hadd2_rn(__hmul2_rn(n, m1), *reinterpret_cast<const __nv_bfloat162*>(&hw));
                    const uint32_t uw = *reinterpret_cast<const uint32_t*>(&u);
                    v[k * 8 + j] = __uint_as_float(uw << 16);
                    v[k * 8 + j + 1] = __uint_as_float(uw & 0xffff0000u);
                }
            }
        }
    }
    butterfly_consecutive<V>(v);

    if constexpr (B1 > 0) {
        __syncthreads();                                       // everyone has read the raw staging area
        exchange_write<L0, V>(xch, v, t);
        __syncthreads();
        exchange_read<L1, V>(xch, v, t);
        butterfly_groups<L1, V>(v);
    }
    if constexpr (B2 > 0) {
        __syncthreads();
        exchange_write<L1, V>(xch, v, t);
        __syncthreads();
        exchange_read<L2, V>(xch, v, t);
        butterfly_groups<L2, V>(v);
    }
    using LF = std::conditional_t<(B2 > 0), L2, std::conditional_t<(B1 > 0), L1, L0>>;
    constexpr int C = LF::C;
    constexpr int PIECE = C < 8 ? C : 8;                       // elements per store; dim % 8 == 0 so a piece never straddles dim

    const float2 sc2 = make_float2(scale, scale);
#pragma unroll
    for (int i = 0; i < V; i += 2) {
        const float2 m = fmul2(make_float2(v[i], v[i + 1]), sc2);
        v[i] = m.x; v[i + 1] = m.y;
    }

    Tout* outr = out + row * (int64_t)dim;
    if constexpr (EPI == Epilogue::Cast) {
#pragma unroll
        for (int j = 0; j < LF::G; ++j) {
            const int e = LF::elem(t, j);
#pragma unroll
            for (int pc = 0; pc < C / PIECE; ++pc) {
                if (row_ok && (FULL || e + pc * PIECE < dim)) {
                    float o[PIECE];
#pragma unroll
                    for (int i = 0; i < PIECE; ++i) o[i] = v[j * C + pc * PIECE + i];
                    store_elems<Tout, PIECE>(outr + e + pc * PIECE, o);
                }
            }
        }
    } else {
        // round to the input dtype (what the unfused chain stores), then the row's absmax
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < LF::G; ++j) {
            const bool in = FULL || LF::elem(t, j) < dim;      // dim % 8 == 0: a run of <= 8 is all in or all out
            float m = 0.f;
#pragma unroll
            for (int i = 0; i < C; i += 2) {
                const float2 rt = round_through2<Tin>(v[j * C + i], v[j * C + i + 1]);
                v[j * C + i] = rt.x;
                v[j * C + i + 1] = rt.y;
                if (FULL || C <= 8 || LF::elem(t, j) + (i & ~7) < dim) m = fmaxf(m, fmaxf(fabsf(rt.x), fabsf(rt.y)));
            }
            if (C > 8 || in) amax = fmaxf(amax, m);
        }
        // reduce over the T threads of the row
#pragma unroll
        for (int m = 1; m < (T < 32 ? T : 32); m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
        if constexpr (T > 32) {
            constexpr int WPR = T / 32;                        // warps per row
            if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
            __syncthreads();
            amax = red[r_in_cta * WPR];
#pragma unroll
            for (int k = 1; k < WPR; ++k) amax = fmaxf(amax, red[r_in_cta * WPR + k]);
        }
        const float qmax = std::is_same_v<Tout, int8_t> ? 127.0f : 448.0f;
        const float qscale = __fdiv_rn(qmax, amax);
        if (row_ok && t == 0) scales[row] = __fdiv_rn(1.0f, qscale);
        const float qmul = amax == 0.f ? 0.f : qscale;         // an all-zero row quantises to zeros (0 * 0, not 0 * inf)
#pragma unroll
        for (int j = 0; j < LF::G; ++j) {
            const int e = LF::elem(t, j);
#pragma unroll
            for (int pc = 0; pc < C / PIECE; ++pc) {
                if (row_ok && (FULL || e + pc * PIECE < dim)) {
                    using BV = typename ByteVec<PIECE>::type;
                    union { BV vec; uint8_t b[PIECE]; uint32_t w[PIECE >= 4 ? PIECE / 4 : 1]; } u;
                    const float2 q2 = make_float2(qmul, qmul);
                    if constexpr (PIECE >= 4) {
#pragma unroll
                        for (int i = 0; i < PIECE; i += 4) {
                            const float2 y0 = fmul2(make_float2(v[j * C + pc * PIECE + i], v[j * C + pc * PIECE + i + 1]), q2);
                            const float2 y1 = fmul2(make_float2(v[j * C + pc * PIECE + i + 2], v[j * C + pc * PIECE + i + 3]), q2);
                            u.w[i / 4] = quantize_pack4<Tout>(y0.x, y0.y, y1.x, y1.y);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < PIECE; i += 2) {
                            const float2 y = fmul2(make_float2(v[j * C + pc * PIECE + i], v[j * C + pc * PIECE + i + 1]), q2);
                            u.b[i] = quantize_fast<Tout>(y.x);
                            u.b[i + 1] = quantize_fast<Tout>(y.y);
                        }
                    }
                    *reinterpret_cast<BV*>(reinterpret_cast<uint8_t*>(outr) + e + pc * PIECE) = u.vec;
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
        if (log_n > 14) { set_error_detail("%s: dim %d exceeds 16384", op, dim); return Q8K_ERR_UNSUPPORTED; }
#define Q8K_HR(LN, LV, NR)                                                                                \
    case LN: {                                                                                            \
        auto kern = dim == (1 << LN) ? hadamard_row_kernel<Tin, Tout, LN, LV, NR, EPI, false, true>       \
                                     : hadamard_row_kernel<Tin, Tout, LN, LV, NR, EPI, false, false>;     \
        constexpr int smem = NR * (1 << LN) * (int)sizeof(float);                                         \
        if (smem > 48 * 1024)                                                                             \
            Q8K_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));   \
        kern<<<(unsigned)((rows + NR - 1) / NR), NR << (LN - LV), smem, st>>>(xi, o, scales, rows, dim, stride, scale, nullptr, nullptr, 1); \
    } break
        // (row length, values per thread, rows per CTA), chosen by measurement: the plain transform
        // likes more values per thread (fewer exchanges), the fused quantizer more threads
        if constexpr (EPI == Epilogue::Cast) {
            switch (log_n) {
                Q8K_HR(9, 5, 8); Q8K_HR(10, 6, 8); Q8K_HR(11, 6, 4); Q8K_HR(12, 6, 2); Q8K_HR(13, 6, 1); Q8K_HR(14, 7, 1);
            }
        } else {
            switch (log_n) {
                Q8K_HR(9, 5, 8); Q8K_HR(10, 5, 4); Q8K_HR(11, 5, 2); Q8K_HR(12, 6, 2); Q8K_HR(13, 6, 1); Q8K_HR(14, 7, 1);
            }
        }
#undef Q8K_HR
    }
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

// fused RMSNorm + modulation + Hadamard + quantizer (bf16 rows of 512 .. 8192 elements)
template <typename Tout>
static int launch_norm_mod_quant(const void* x, const void* mod_scale, const void* mod_shift, void* q, float* scales,
                                 int64_t rows, int dim, int64_t rows_per_mod, float scale, cudaStream_t st) {
    int log_n = 9;
    while ((1 << log_n) < dim) ++log_n;
    const __nv_bfloat16* xi = (const __nv_bfloat16*)x;
    const __nv_bfloat16* ms = (const __nv_bfloat16*)mod_scale;
    const __nv_bfloat16* mh = (const __nv_bfloat16*)mod_shift;
    Tout* o = (Tout*)q;
#define Q8K_NM(LN, LV, NR)                                                                                \
    case LN: {                                                                                            \
        auto kern = dim == (1 << LN) ? hadamard_row_kernel<__nv_bfloat16, Tout, LN, LV, NR, Epilogue::Quant, true, true>  \
                                     : hadamard_row_kernel<__nv_bfloat16, Tout, LN, LV, NR, Epilogue::Quant, true, false>; \
        constexpr int smem = NR * (1 << LN) * (int)sizeof(float);                                         \
        if (smem > 48 * 1024)                                                                             \
            Q8K_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));   \
        kern<<<(unsigned)((rows + NR - 1) / NR), NR << (LN - LV), smem, st>>>(xi, o, scales, rows, dim, dim, scale, ms, mh, rows_per_mod); \
    } break
    switch (log_n) {
        Q8K_NM(9, 5, 8); Q8K_NM(10, 5, 4); Q8K_NM(11, 5, 2); Q8K_NM(12, 6, 2); Q8K_NM(13, 6, 1);
        default: set_error_detail("norm_modulate_quant: dim %d not in [512, 8192]", dim); return Q8K_ERR_UNSUPPORTED;
    }
#undef Q8K_NM
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

extern "C" int q8k_norm_modulate_quant(const void* x, const void* mod_scale, const void* mod_shift, void* q, int q_dtype,
                                       float* scales, int64_t rows, int dim, int64_t rows_per_mod, float scale,
                                       void* stream) {
    const char* op = "norm_modulate_quant";
    if (int rc = check_hadamard_args(op, x, Q8K_DT_BF16, q, rows, dim, dim)) return rc;
    if (rows == 0) return Q8K_OK;
    Q8K_REQUIRE(dim >= 257 && dim % 16 == 0, Q8K_ERR_UNSUPPORTED, "%s: dim %d must be a multiple of 16 above 256", op, dim);
    Q8K_REQUIRE(mod_scale && mod_shift && scales, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE(aligned16(mod_scale) && aligned16(mod_shift), Q8K_ERR_INVALID_ARG, "%s: modulation rows must be 16-byte aligned", op);
    Q8K_REQUIRE(rows_per_mod >= 1, Q8K_ERR_INVALID_ARG, "%s: rows_per_mod must be >= 1", op);
    cudaStream_t st = (cudaStream_t)stream;
    if (q_dtype == Q8K_DT_I8) return launch_norm_mod_quant<int8_t>(x, mod_scale, mod_shift, q, scales, rows, dim, rows_per_mod, scale, st);
    if (q_dtype == Q8K_DT_E4M3) return launch_norm_mod_quant<e4m3_t>(x, mod_scale, mod_shift, q, scales, rows, dim, rows_per_mod, scale, st);
    set_error_detail("%s: quantised dtype %d is not int8 or e4m3", op, q_dtype);
    return Q8K_ERR_UNSUPPORTED;
}
