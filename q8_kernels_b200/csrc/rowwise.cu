// HBM-bound row-wise kernels: per-token absmax quantizer, RMS norm, rotary
// embedding, mixed-precision FMA and tanh-GELU.
//
// Layout: every tensor is [rows, dim] with dim contiguous.  One CTA of T
// threads owns one row; a thread owns ITEMS "items" of 8 consecutive elements
// (item index t, t+T, ...), so every global access is a 16-byte (bf16), 8-byte
// (8-bit) or 32-byte (fp32) vector and a warp covers a contiguous segment.
// The row lives in registers between the reduction and the output pass, so HBM
// sees each element exactly once in and once out.
//
// No fast-math: the quantizer must reproduce IEEE division and C round().

#include <type_traits>
#include "common.cuh"

namespace q8k {

constexpr int kItem = 8;

template <int T>
__device__ __forceinline__ float block_reduce_max(float v, float* smem) {
    v = warp_max(v);
    if constexpr (T > 32) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) smem[warp] = v;
        __syncthreads();
        float r = smem[0];
#pragma unroll
        for (int w = 1; w < T / 32; ++w) r = fmaxf(r, smem[w]);
        __syncthreads();
        v = r;
    }
    return v;
}

template <int T>
__device__ __forceinline__ float block_reduce_sum(float v, float* smem) {
    v = warp_sum(v);
    if constexpr (T > 32) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) smem[warp] = v;
        __syncthreads();
        float r = smem[0];
#pragma unroll
        for (int w = 1; w < T / 32; ++w) r += smem[w];
        __syncthreads();
        v = r;
    }
    return v;
}

// ------------------------------------------------------------------ quantizer
// Semantics of tokenwise_quantization_kernel
// (csrc/quantizer/tokenwise_quant_cuda.cu:115-148) with IEEE arithmetic.
template <typename Tin, typename Tout, int ITEMS, int T>
__global__ void __launch_bounds__(T)
tokenwise_quant_kernel(const Tin* __restrict__ x, Tout* __restrict__ q, float* __restrict__ scales,
                       int dim, int64_t x_row_stride) {
    __shared__ float red[32];
    const int64_t row = blockIdx.x;
    const Tin* xr = x + row * x_row_stride;
    Tout* qr = q + row * (int64_t)dim;

    float v[ITEMS][kItem];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int e = (threadIdx.x + i * T) * kItem;
        if (e < dim) {
            load_vec<Tin, kItem>(xr + e, v[i]);
#pragma unroll
            for (int j = 0; j < kItem; ++j) amax = fmaxf(amax, fabsf(v[i][j]));
        }
    }
    amax = block_reduce_max<T>(amax, red);

    constexpr bool kInt8 = sizeof(Tout) == 1 && !__is_same(Tout, e4m3_t);
    const float qmax = kInt8 ? 127.0f : 448.0f;
    const float scale = __fdiv_rn(qmax, amax);            // +inf for an all-zero row
    const bool zero_row = amax == 0.f;

#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int e = (threadIdx.x + i * T) * kItem;
        if (e < dim) {
            union { uint2 v2; uint8_t b[kItem]; uint16_t h[kItem / 2]; } o;
            if constexpr (kInt8) {
#pragma unroll
                for (int j = 0; j < kItem; ++j) {
                    const float y = zero_row ? 0.f : __fmul_rn(v[i][j], scale);
                    // exact round half away from zero: truncate y + copysign(0.5 - 2^-25, y)
                    o.b[j] = (uint8_t)(int8_t)__float2int_rz(__fadd_rn(y, copysignf(0.49999997f, y)));
                }
            } else {
                // |x * scale| <= 448 (1 + 2^-23) for a finite row, far below the 464 where the c10 cast turns
                // into NaN, so the packed saturating conversion gives the same bytes; a NaN stays a NaN
#pragma unroll
                for (int j = 0; j < kItem; j += 2) {
                    const float y0 = zero_row ? 0.f : __fmul_rn(v[i][j], scale);
                    const float y1 = zero_row ? 0.f : __fmul_rn(v[i][j + 1], scale);
                    o.h[j / 2] = float2_to_e4m3x2_sat(y0, y1);
                }
            }
            *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(qr) + e) = o.v2;
        }
    }
    if (threadIdx.x == 0) scales[row] = __fdiv_rn(1.0f, scale);
}

// ------------------------------------------------------------------ RMS norm
// rms_norm_kernel (csrc/ops/rms_norm_cuda.cu:127-169): no eps, (x*r)*w.
template <typename Tin, typename Tout, int ITEMS, int T>
__global__ void __launch_bounds__(T)
rms_norm_kernel(const Tin* __restrict__ x, const float* __restrict__ w, Tout* __restrict__ out,
                float* __restrict__ rrms, int dim) {
    __shared__ float red[32];
    const int64_t row = blockIdx.x;
    const Tin* xr = x + row * (int64_t)dim;
    Tout* outr = out + row * (int64_t)dim;

    float v[ITEMS][kItem];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int e = (threadIdx.x + i * T) * kItem;
        if (e < dim) {
            load_vec<Tin, kItem>(xr + e, v[i]);
#pragma unroll
            for (int j = 0; j < kItem; ++j) ss = fmaf(v[i][j], v[i][j], ss);
        }
    }
    ss = block_reduce_sum<T>(ss, red);
    const float r = rsqrtf(ss * (1.0f / (float)dim));

#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int e = (threadIdx.x + i * T) * kItem;
        if (e < dim) {
            float o[kItem];
            if (w != nullptr) {
                float wv[kItem];
                load_vec<float, kItem>(w + e, wv);
#pragma unroll
                for (int j = 0; j < kItem; ++j) o[j] = __fmul_rn(__fmul_rn(v[i][j], r), wv[j]);
            } else {
#pragma unroll
                for (int j = 0; j < kItem; ++j) o[j] = __fmul_rn(v[i][j], r);
            }
            store_vec<Tout, kItem>(outr + e, o);
        }
    }
    if (rrms != nullptr && threadIdx.x == 0) rrms[row] = r;
}

// ------------------------------------------------------------------ element-wise rows
// These keep nothing between passes, so a CTA strides over a row in items and
// the grid is rows x ceil(items / T).

// rope_kernel (csrc/ops/rope_cuda.cu:99-103), products rounded before the add.
template <typename Tin, typename Tout, int T>
__global__ void __launch_bounds__(T)
rope_kernel(const Tin* __restrict__ x, const float* __restrict__ cosf_, const float* __restrict__ sinf_,
            Tout* __restrict__ out, int dim, int64_t freq_rows) {
    const int64_t row = blockIdx.x;
    const int e = (blockIdx.y * T + threadIdx.x) * kItem;
    if (e >= dim) return;
    const int64_t frow = freq_rows > 0 ? row % freq_rows : row;
    float xv[kItem], c[kItem], s[kItem], o[kItem];
    load_vec<Tin, kItem>(x + row * (int64_t)dim + e, xv);
    load_vec<float, kItem>(cosf_ + frow * (int64_t)dim + e, c);
    load_vec<float, kItem>(sinf_ + frow * (int64_t)dim + e, s);
#pragma unroll
    for (int j = 0; j < kItem; j += 2) {
        o[j]     = __fadd_rn(__fmul_rn(-xv[j + 1], s[j]), __fmul_rn(xv[j], c[j]));
        o[j + 1] = __fadd_rn(__fmul_rn(xv[j], s[j + 1]), __fmul_rn(xv[j + 1], c[j + 1]));
    }
    store_vec<Tout, kItem>(out + row * (int64_t)dim + e, o);
}

// fma_kernel (csrc/ops/fma_cuda.cu:92-95).  16 elements per thread (one 16-byte load of x and one store),
// e4m3 -> fp32 through the packed e4m3x2 -> f16x2 conversion, the c10 cast eight values at a time.
__device__ __forceinline__ void e4m3x4_to_float(uint32_t w, float (&o)[4]) {
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xffffu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
    const float2 a = __half22float2(__half2(lo)), c = __half22float2(__half2(hi));
    o[0] = a.x; o[1] = a.y; o[2] = c.x; o[3] = c.y;
}
template <typename Ty, typename Tz, int T>
__global__ void __launch_bounds__(T)
fma_kernel(const e4m3_t* __restrict__ x, const Ty* __restrict__ y, const Tz* __restrict__ z,
           e4m3_t* __restrict__ out, unsigned rows, int dim, unsigned y_every, unsigned z_every, float scale_add) {
    constexpr int E = 16;                                      // columns per thread
    constexpr int R = 4;                                       // rows per thread: y and z are widened once for all of them
    const unsigned row0 = blockIdx.x * R;                      // < 2^31 rows (checked by the caller)
    const int e = (blockIdx.y * T + threadIdx.x) * E;
    if (e >= dim) return;
    const unsigned nr = rows - row0 < (unsigned)R ? rows - row0 : (unsigned)R;
    // the common case: the rows of this thread share one y row and one z row (modulation rows broadcast over tokens)
    const bool shared_yz = row0 / y_every == (row0 + nr - 1) / y_every && row0 / z_every == (row0 + nr - 1) / z_every;
    float yv[E], zv[E];
    if (shared_yz) {
        load_vec<Ty, E>(y + (int64_t)(row0 / y_every) * dim + e, yv);
        load_vec<Tz, E>(z + (int64_t)(row0 / z_every) * dim + e, zv);
#pragma unroll
        for (int j = 0; j < E; ++j) yv[j] = __fadd_rn(yv[j], scale_add);
    }
    uint4 xw[R];
#pragma unroll
    for (int r = 0; r < R; ++r)
        if ((unsigned)r < nr) xw[r] = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(x) + (int64_t)(row0 + r) * dim + e);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if ((unsigned)r >= nr) break;
        const unsigned row = row0 + r;
        if (!shared_yz) {
            load_vec<Ty, E>(y + (int64_t)(row / y_every) * dim + e, yv);
            load_vec<Tz, E>(z + (int64_t)(row / z_every) * dim + e, zv);
#pragma unroll
            for (int j = 0; j < E; ++j) yv[j] = __fadd_rn(yv[j], scale_add);
        }
        float xv[E];
        {
            float t4[4];
            e4m3x4_to_float(xw[r].x, t4); xv[0] = t4[0]; xv[1] = t4[1]; xv[2] = t4[2]; xv[3] = t4[3];
            e4m3x4_to_float(xw[r].y, t4); xv[4] = t4[0]; xv[5] = t4[1]; xv[6] = t4[2]; xv[7] = t4[3];
            e4m3x4_to_float(xw[r].z, t4); xv[8] = t4[0]; xv[9] = t4[1]; xv[10] = t4[2]; xv[11] = t4[3];
            e4m3x4_to_float(xw[r].w, t4); xv[12] = t4[0]; xv[13] = t4[1]; xv[14] = t4[2]; xv[15] = t4[3];
        }
        uint4 ow;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {                   // packed fp32x2: each lane rounds like the scalar form
                const int i = h * 8 + j;
                const float2 v2 = fadd2(fmul2(make_float2(xv[i], xv[i + 1]), make_float2(yv[i], yv[i + 1])),
                                        make_float2(zv[i], zv[i + 1]));
                o[j] = v2.x;
                o[j + 1] = v2.y;
            }
            const uint2 w = pack8_e4m3_c10(o);
            if (h == 0) { ow.x = w.x; ow.y = w.y; } else { ow.z = w.x; ow.w = w.y; }
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(out) + (int64_t)row * dim + e) = ow;
    }
}

// gelu_forward_kernel (csrc/ops/gelu_forward_cuda.cu:12-16).
template <typename Tin, typename Tout, int T>
__global__ void __launch_bounds__(T)
gelu_kernel(const Tin* __restrict__ x, Tout* __restrict__ out, int dim) {
    const int64_t row = blockIdx.x;
    const int e = (blockIdx.y * T + threadIdx.x) * kItem;
    if (e >= dim) return;
    float xv[kItem], o[kItem];
    load_vec<Tin, kItem>(x + row * (int64_t)dim + e, xv);
    if constexpr (std::is_same_v<Tout, float>) {
#pragma unroll
        for (int j = 0; j < kItem; ++j) o[j] = gelu_tanh_precise(xv[j]);
    } else {
        // 0.5 (1 + tanh u) = 1 / (1 + e^(-2u)), so gelu(x) = x / (1 + 2^(-2 u log2 e)) with no cancellation anywhere:
        // a few fp32 ulps from the tanhf form, far below the 16-bit / 8-bit output step
        constexpr float kC0 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
        constexpr float kC1 = kC0 * 0.044715f;
#pragma unroll
        for (int j = 0; j < kItem; j += 2) {
            const float2 xx = make_float2(xv[j], xv[j + 1]);
            const float2 t = fmul2(ffma2(fmul2(xx, xx), make_float2(kC1, kC1), make_float2(kC0, kC0)), xx);
            float e0, e1, r0, r1;
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(t.x));
            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(t.y));
            const float2 d = fadd2(make_float2(e0, e1), make_float2(1.0f, 1.0f));
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(d.x));
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(d.y));
            const float2 y = fmul2(xx, make_float2(r0, r1));
            o[j] = y.x;
            o[j + 1] = y.y;
        }
    }
    store_vec<Tout, kItem>(out + row * (int64_t)dim + e, o);
}

// ------------------------------------------------------------------ training-side gradients
// gelu_backward_kernel (csrc/ops/gelu_backward_cuda.cu:88-100): d/dx of the tanh GELU times the
// incoming gradient, all in fp32, same association of the products as the reference.
template <typename Tx, typename Tg, typename Tout, int T>
__global__ void __launch_bounds__(T)
gelu_backward_kernel(const Tx* __restrict__ x, const Tg* __restrict__ grad, Tout* __restrict__ out, int dim) {
    const int64_t row = blockIdx.x;
    const int e = (blockIdx.y * T + threadIdx.x) * kItem;
    if (e >= dim) return;
    float xv[kItem], gv[kItem], o[kItem];
    load_vec<Tx, kItem>(x + row * (int64_t)dim + e, xv);
    load_vec<Tg, kItem>(grad + row * (int64_t)dim + e, gv);
    constexpr float k = 0.7978845608028654f, f = 0.044715f;
#pragma unroll
    for (int j = 0; j < kItem; ++j) {
        const float v = xv[j];
        const float tau = k * (v + f * v * v * v);
        const float phi = tanhf(tau);
        const float phi_prime = (1.0f - phi * phi) * (k * (1.0f + f * 3.0f * v * v));
        o[j] = gv[j] * (0.5f * (1.0f + phi) + 0.5f * v * phi_prime);
    }
    store_vec<Tout, kItem>(out + row * (int64_t)dim + e, o);
}

// rope_backward_kernel (csrc/ops/rope_backward_cuda.cu:101-110): the transposed rotation.
template <typename Tg, typename Tout, int T>
__global__ void __launch_bounds__(T)
rope_backward_kernel(const Tg* __restrict__ grad, const float* __restrict__ cosf_, const float* __restrict__ sinf_,
                     Tout* __restrict__ out, int dim, int64_t freq_rows) {
    const int64_t row = blockIdx.x;
    const int e = (blockIdx.y * T + threadIdx.x) * kItem;
    if (e >= dim) return;
    const int64_t frow = freq_rows > 0 ? row % freq_rows : row;
    float g[kItem], c[kItem], s[kItem], o[kItem];
    load_vec<Tg, kItem>(grad + row * (int64_t)dim + e, g);
    load_vec<float, kItem>(cosf_ + frow * (int64_t)dim + e, c);
    load_vec<float, kItem>(sinf_ + frow * (int64_t)dim + e, s);
#pragma unroll
    for (int j = 0; j < kItem; j += 2) {
        o[j]     = __fadd_rn(__fmul_rn(g[j], c[j]), __fmul_rn(g[j + 1], s[j + 1]));
        o[j + 1] = __fadd_rn(__fmul_rn(-g[j], s[j]), __fmul_rn(g[j + 1], c[j + 1]));
    }
    store_vec<Tout, kItem>(out + row * (int64_t)dim + e, o);
}

// rms_norm_backward_kernel (csrc/ops/rms_norm_backward_cuda.cu:135-160): with y the forward
// output (weights included), r the saved rsqrt(mean x^2) and g the incoming gradient,
//   dx_i = r / dim * (dim * g_i * w_i - y_i / w_i * sum_j g_j y_j).
template <typename Ty, typename Tg, typename Tout, int ITEMS, int T>
__global__ void __launch_bounds__(T)
rms_norm_backward_kernel(const Ty* __restrict__ y, const float* __restrict__ rrms, const Tg* __restrict__ grad,
                         const float* __restrict__ w, Tout* __restrict__ out, int dim) {
    __shared__ float red[32];
    const int64_t row = blockIdx.x;
    float yv[ITEMS][kItem], gv[ITEMS][kItem];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int e = (threadIdx.x + i * T) * kItem;
        if (e < dim) {
            load_vec<Ty, kItem>(y + row * (int64_t)dim + e, yv[i]);
            load_vec<Tg, kItem>(grad + row * (int64_t)dim + e, gv[i]);
#pragma unroll
            for (int j = 0; j < kItem; ++j) dot = fmaf(gv[i][j], yv[i][j], dot);
        }
    }
    dot = block_reduce_sum<T>(dot, red);
    const float fdim = (float)dim;
    const float r_over_dim = rrms[row] / fdim;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int e = (threadIdx.x + i * T) * kItem;
        if (e < dim) {
            float wv[kItem], o[kItem];
            if (w != nullptr) {
                load_vec<float, kItem>(w + e, wv);
            } else {
#pragma unroll
                for (int j = 0; j < kItem; ++j) wv[j] = 1.0f;
            }
#pragma unroll
            for (int j = 0; j < kItem; ++j)
                o[j] = r_over_dim * (fdim * gv[i][j] * wv[j] - yv[i][j] / wv[j] * dot);
            store_vec<Tout, kItem>(out + row * (int64_t)dim + e, o);
        }
    }
}

// ------------------------------------------------------------------ launch helpers
template <typename Tin, typename Tout>
static int launch_quant(const void* x, void* q, float* scales, int64_t rows, int dim,
                        int64_t stride, cudaStream_t st) {
    const int items = dim / kItem;
#define Q8K_Q_LAUNCH(ITEMS, T)                                                                  \
    tokenwise_quant_kernel<Tin, Tout, ITEMS, T><<<(unsigned)rows, T, 0, st>>>(                   \
        (const Tin*)x, (Tout*)q, scales, dim, stride)
    if (items <= 32)        Q8K_Q_LAUNCH(1, 32);
    else if (items <= 128)  Q8K_Q_LAUNCH(1, 128);
    else if (items <= 256)  Q8K_Q_LAUNCH(2, 128);
    else if (items <= 512)  Q8K_Q_LAUNCH(4, 128);
    else if (items <= 1024) Q8K_Q_LAUNCH(4, 256);
    else if (items <= 2048) Q8K_Q_LAUNCH(8, 256);
    else if (items <= 4096) Q8K_Q_LAUNCH(8, 512);
    else { set_error_detail("tokenwise_quant: dim %d exceeds 32768", dim); return Q8K_ERR_UNSUPPORTED; }
#undef Q8K_Q_LAUNCH
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

template <typename Tin, typename Tout>
static int launch_rms(const void* x, const float* w, void* out, float* rrms, int64_t rows, int dim,
                      cudaStream_t st) {
    const int items = dim / kItem;
#define Q8K_R_LAUNCH(ITEMS, T)                                                                  \
    rms_norm_kernel<Tin, Tout, ITEMS, T><<<(unsigned)rows, T, 0, st>>>(                          \
        (const Tin*)x, w, (Tout*)out, rrms, dim)
    if (items <= 32)        Q8K_R_LAUNCH(1, 32);
    else if (items <= 128)  Q8K_R_LAUNCH(1, 128);
    else if (items <= 256)  Q8K_R_LAUNCH(2, 128);
    else if (items <= 512)  Q8K_R_LAUNCH(4, 128);
    else if (items <= 1024) Q8K_R_LAUNCH(4, 256);
    else if (items <= 2048) Q8K_R_LAUNCH(8, 256);
    else if (items <= 4096) Q8K_R_LAUNCH(8, 512);
    else { set_error_detail("rms_norm: dim %d exceeds 32768", dim); return Q8K_ERR_UNSUPPORTED; }
#undef Q8K_R_LAUNCH
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

static int check_rows_dim(const char* op, int64_t rows, int dim, int multiple) {
    Q8K_REQUIRE(rows >= 0 && rows <= 0x7fffffffLL, Q8K_ERR_INVALID_ARG, "%s: rows %lld out of range", op, (long long)rows);
    Q8K_REQUIRE(dim > 0 && dim % multiple == 0, Q8K_ERR_INVALID_ARG,
                "%s: dim %d must be a positive multiple of %d", op, dim, multiple);
    return Q8K_OK;
}

}  // namespace q8k

using namespace q8k;

extern "C" int q8k_tokenwise_quant(const void* x, int x_dtype, void* q, int q_dtype, float* scales,
                                   int64_t rows, int dim, int64_t x_row_stride, void* stream) {
    if (int rc = check_rows_dim("tokenwise_quant", rows, dim, 16)) return rc;
    if (rows == 0) return Q8K_OK;
    Q8K_REQUIRE(x && q && scales, Q8K_ERR_INVALID_ARG, "tokenwise_quant: null pointer");
    Q8K_REQUIRE(aligned16(x) && aligned16(q), Q8K_ERR_INVALID_ARG, "tokenwise_quant: x and q must be 16-byte aligned");
    Q8K_REQUIRE(x_row_stride >= dim && (x_row_stride * dtype_size(x_dtype)) % 16 == 0, Q8K_ERR_INVALID_ARG,
                "tokenwise_quant: row stride %lld must be >= dim and a multiple of 16 bytes", (long long)x_row_stride);
    Q8K_REQUIRE(q_dtype == Q8K_DT_I8 || q_dtype == Q8K_DT_E4M3, Q8K_ERR_UNSUPPORTED,
                "tokenwise_quant: output dtype %d is not int8 or e4m3", q_dtype);
    cudaStream_t st = (cudaStream_t)stream;
#define Q8K_QD(TIN)                                                                              \
    return q_dtype == Q8K_DT_I8 ? launch_quant<TIN, int8_t>(x, q, scales, rows, dim, x_row_stride, st) \
                                : launch_quant<TIN, e4m3_t>(x, q, scales, rows, dim, x_row_stride, st)
    switch (x_dtype) {
        case Q8K_DT_F32:  Q8K_QD(float);
        case Q8K_DT_F16:  Q8K_QD(__half);
        case Q8K_DT_BF16: Q8K_QD(__nv_bfloat16);
        case Q8K_DT_E4M3: Q8K_QD(e4m3_t);
        default: break;
    }
#undef Q8K_QD
    set_error_detail("tokenwise_quant: input dtype %d not supported", x_dtype);
    return Q8K_ERR_UNSUPPORTED;
}

extern "C" int q8k_rms_norm(const void* x, int x_dtype, const float* weights, void* out, int out_dtype,
                            float* rrms, int64_t rows, int dim, void* stream) {
    if (int rc = check_rows_dim("rms_norm", rows, dim, 16)) return rc;
    if (rows == 0) return Q8K_OK;
    Q8K_REQUIRE(x && out, Q8K_ERR_INVALID_ARG, "rms_norm: null pointer");
    Q8K_REQUIRE(aligned16(x) && aligned16(out) && aligned16(weights), Q8K_ERR_INVALID_ARG,
                "rms_norm: pointers must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (x_dtype == Q8K_DT_BF16 && out_dtype == Q8K_DT_BF16) return launch_rms<__nv_bfloat16, __nv_bfloat16>(x, weights, out, rrms, rows, dim, st);
    if (x_dtype == Q8K_DT_BF16 && out_dtype == Q8K_DT_E4M3) return launch_rms<__nv_bfloat16, e4m3_t>(x, weights, out, rrms, rows, dim, st);
    if (x_dtype == Q8K_DT_E4M3 && out_dtype == Q8K_DT_BF16) return launch_rms<e4m3_t, __nv_bfloat16>(x, weights, out, rrms, rows, dim, st);
    if (x_dtype == Q8K_DT_E4M3 && out_dtype == Q8K_DT_E4M3) return launch_rms<e4m3_t, e4m3_t>(x, weights, out, rrms, rows, dim, st);
    set_error_detail("rms_norm: dtype pair (%d -> %d) not supported", x_dtype, out_dtype);
    return Q8K_ERR_UNSUPPORTED;
}

extern "C" int q8k_rope(const void* x, int x_dtype, const float* cos_freqs, const float* sin_freqs,
                        void* out, int out_dtype, int64_t rows, int dim, int64_t freq_rows, void* stream) {
    if (int rc = check_rows_dim("rope", rows, dim, 16)) return rc;
    if (rows == 0) return Q8K_OK;
    Q8K_REQUIRE(x && out && cos_freqs && sin_freqs, Q8K_ERR_INVALID_ARG, "rope: null pointer");
    Q8K_REQUIRE(aligned16(x) && aligned16(out) && aligned16(cos_freqs) && aligned16(sin_freqs),
                Q8K_ERR_INVALID_ARG, "rope: pointers must be 16-byte aligned");
    Q8K_REQUIRE(freq_rows >= 0, Q8K_ERR_INVALID_ARG, "rope: freq_rows must be >= 0");
    cudaStream_t st = (cudaStream_t)stream;
    constexpr int T = 128;
    dim3 grid((unsigned)rows, (unsigned)((dim / kItem + T - 1) / T));
#define Q8K_ROPE(TIN, TOUT) rope_kernel<TIN, TOUT, T><<<grid, T, 0, st>>>((const TIN*)x, cos_freqs, sin_freqs, (TOUT*)out, dim, freq_rows)
    if (x_dtype == Q8K_DT_BF16 && out_dtype == Q8K_DT_BF16) Q8K_ROPE(__nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == Q8K_DT_BF16 && out_dtype == Q8K_DT_E4M3) Q8K_ROPE(__nv_bfloat16, e4m3_t);
    else if (x_dtype == Q8K_DT_BF16 && out_dtype == Q8K_DT_F32) Q8K_ROPE(__nv_bfloat16, float);
    else if (x_dtype == Q8K_DT_E4M3 && out_dtype == Q8K_DT_BF16) Q8K_ROPE(e4m3_t, __nv_bfloat16);
    else if (x_dtype == Q8K_DT_E4M3 && out_dtype == Q8K_DT_E4M3) Q8K_ROPE(e4m3_t, e4m3_t);
    else { set_error_detail("rope: dtype pair (%d -> %d) not supported", x_dtype, out_dtype); return Q8K_ERR_UNSUPPORTED; }
#undef Q8K_ROPE
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

extern "C" int q8k_fma_8bit(const void* x, const void* y, int y_dtype, const void* z, int z_dtype, void* out,
                            int64_t rows, int dim, int64_t y_every, int64_t z_every, float scale_add,
                            void* stream) {
    if (int rc = check_rows_dim("fma_8bit", rows, dim, 16)) return rc;
    if (rows == 0) return Q8K_OK;
    Q8K_REQUIRE(x && y && z && out, Q8K_ERR_INVALID_ARG, "fma_8bit: null pointer");
    Q8K_REQUIRE(aligned16(x) && aligned16(y) && aligned16(z) && aligned16(out), Q8K_ERR_INVALID_ARG,
                "fma_8bit: pointers must be 16-byte aligned");
    Q8K_REQUIRE(y_every >= 1 && z_every >= 1, Q8K_ERR_INVALID_ARG, "fma_8bit: broadcast periods must be >= 1");
    cudaStream_t st = (cudaStream_t)stream;
    constexpr int T = 128;
    dim3 grid((unsigned)((rows + 3) / 4), (unsigned)((dim / 16 + T - 1) / T));
    const unsigned ye = (unsigned)(y_every > rows ? rows : y_every), ze = (unsigned)(z_every > rows ? rows : z_every);
#define Q8K_FMA(TY, TZ) fma_kernel<TY, TZ, T><<<grid, T, 0, st>>>((const e4m3_t*)x, (const TY*)y, (const TZ*)z, (e4m3_t*)out, (unsigned)rows, dim, ye, ze, scale_add)
    if (y_dtype == Q8K_DT_F32 && z_dtype == Q8K_DT_F32) Q8K_FMA(float, float);
    else if (y_dtype == Q8K_DT_F32 && z_dtype == Q8K_DT_E4M3) Q8K_FMA(float, e4m3_t);
    else if (y_dtype == Q8K_DT_BF16 && z_dtype == Q8K_DT_BF16) Q8K_FMA(__nv_bfloat16, __nv_bfloat16);
    else { set_error_detail("fma_8bit: (y,z) dtypes (%d,%d) not supported", y_dtype, z_dtype); return Q8K_ERR_UNSUPPORTED; }
#undef Q8K_FMA
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

extern "C" int q8k_gelu_forward(const void* x, int x_dtype, void* out, int out_dtype, int64_t rows, int dim,
                                void* stream) {
    if (int rc = check_rows_dim("gelu_forward", rows, dim, 16)) return rc;
    if (rows == 0) return Q8K_OK;
    Q8K_REQUIRE(x && out, Q8K_ERR_INVALID_ARG, "gelu_forward: null pointer");
    Q8K_REQUIRE(aligned16(x) && aligned16(out), Q8K_ERR_INVALID_ARG, "gelu_forward: pointers must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    constexpr int T = 128;
    dim3 grid((unsigned)rows, (unsigned)((dim / kItem + T - 1) / T));
#define Q8K_GELU(TIN, TOUT) gelu_kernel<TIN, TOUT, T><<<grid, T, 0, st>>>((const TIN*)x, (TOUT*)out, dim)
    if (x_dtype == Q8K_DT_BF16 && out_dtype == Q8K_DT_BF16) Q8K_GELU(__nv_bfloat16, __nv_bfloat16);
    else if (x_dtype == Q8K_DT_BF16 && out_dtype == Q8K_DT_E4M3) Q8K_GELU(__nv_bfloat16, e4m3_t);
    else if (x_dtype == Q8K_DT_E4M3 && out_dtype == Q8K_DT_BF16) Q8K_GELU(e4m3_t, __nv_bfloat16);
    else if (x_dtype == Q8K_DT_E4M3 && out_dtype == Q8K_DT_E4M3) Q8K_GELU(e4m3_t, e4m3_t);
    else { set_error_detail("gelu_forward: dtype pair (%d -> %d) not supported", x_dtype, out_dtype); return Q8K_ERR_UNSUPPORTED; }
#undef Q8K_GELU
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

// ------------------------------------------------------------------ gradients (training side)
namespace q8k {
template <typename F>
static int dispatch_8bit_pair(const char* op, int a_dtype, int b_dtype, F&& f) {
    // calls f(type tag of a, type tag of b) for a, b in {bf16, e4m3}
    if (a_dtype == Q8K_DT_BF16 && b_dtype == Q8K_DT_BF16) return f((__nv_bfloat16*)nullptr, (__nv_bfloat16*)nullptr);
    if (a_dtype == Q8K_DT_BF16 && b_dtype == Q8K_DT_E4M3) return f((__nv_bfloat16*)nullptr, (e4m3_t*)nullptr);
    if (a_dtype == Q8K_DT_E4M3 && b_dtype == Q8K_DT_BF16) return f((e4m3_t*)nullptr, (__nv_bfloat16*)nullptr);
    if (a_dtype == Q8K_DT_E4M3 && b_dtype == Q8K_DT_E4M3) return f((e4m3_t*)nullptr, (e4m3_t*)nullptr);
    set_error_detail("%s: dtype pair (%d, %d) not supported (bf16 / e4m3 only)", op, a_dtype, b_dtype);
    return Q8K_ERR_UNSUPPORTED;
}
}  // namespace q8k

extern "C" int q8k_gelu_backward(const void* x, int x_dtype, const void* grad_out, void* out, int out_dtype,
                                 int64_t rows, int dim, void* stream) {
    const char* op = "gelu_backward";
    if (int rc = check_rows_dim(op, rows, dim, 16)) return rc;
    if (rows == 0) return Q8K_OK;
    Q8K_REQUIRE(x && grad_out && out, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE(aligned16(x) && aligned16(grad_out) && aligned16(out), Q8K_ERR_INVALID_ARG,
                "%s: pointers must be 16-byte aligned", op);
    cudaStream_t st = (cudaStream_t)stream;
    constexpr int T = 128;
    dim3 grid((unsigned)rows, (unsigned)((dim / kItem + T - 1) / T));
    // the incoming gradient has the output's dtype (csrc/ops/gelu_backward_cuda.cu:83)
    int rc = dispatch_8bit_pair(op, x_dtype, out_dtype, [&](auto* tx, auto* to) {
        using Tx = std::remove_pointer_t<decltype(tx)>;
        using To = std::remove_pointer_t<decltype(to)>;
        gelu_backward_kernel<Tx, To, To, T><<<grid, T, 0, st>>>((const Tx*)x, (const To*)grad_out, (To*)out, dim);
        return Q8K_OK;
    });
    if (rc) return rc;
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

extern "C" int q8k_rope_backward(const void* grad_out, int grad_dtype, const float* cos_freqs, const float* sin_freqs,
                                 void* out, int out_dtype, int64_t rows, int dim, int64_t freq_rows, void* stream) {
    const char* op = "rope_backward";
    if (int rc = check_rows_dim(op, rows, dim, 16)) return rc;
    if (rows == 0) return Q8K_OK;
    Q8K_REQUIRE(grad_out && out && cos_freqs && sin_freqs, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE(aligned16(grad_out) && aligned16(out) && aligned16(cos_freqs) && aligned16(sin_freqs),
                Q8K_ERR_INVALID_ARG, "%s: pointers must be 16-byte aligned", op);
    Q8K_REQUIRE(freq_rows >= 0, Q8K_ERR_INVALID_ARG, "%s: freq_rows must be >= 0", op);
    cudaStream_t st = (cudaStream_t)stream;
    constexpr int T = 128;
    dim3 grid((unsigned)rows, (unsigned)((dim / kItem + T - 1) / T));
    int rc = dispatch_8bit_pair(op, grad_dtype, out_dtype, [&](auto* tg, auto* to) {
        using Tg = std::remove_pointer_t<decltype(tg)>;
        using To = std::remove_pointer_t<decltype(to)>;
        rope_backward_kernel<Tg, To, T><<<grid, T, 0, st>>>((const Tg*)grad_out, cos_freqs, sin_freqs, (To*)out, dim, freq_rows);
        return Q8K_OK;
    });
    if (rc) return rc;
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

extern "C" int q8k_rms_norm_backward(const void* x_normed, int x_dtype, const float* x_norms, const void* grad_out,
                                     const float* weights, void* out, int out_dtype, int64_t rows, int dim,
                                     void* stream) {
    const char* op = "rms_norm_backward";
    if (int rc = check_rows_dim(op, rows, dim, 16)) return rc;
    if (rows == 0) return Q8K_OK;
    Q8K_REQUIRE(x_normed && x_norms && grad_out && out, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE(aligned16(x_normed) && aligned16(grad_out) && aligned16(out) && aligned16(weights), Q8K_ERR_INVALID_ARG,
                "%s: pointers must be 16-byte aligned", op);
    cudaStream_t st = (cudaStream_t)stream;
    const int items = dim / kItem;
    if (items > 4096) { set_error_detail("%s: dim %d exceeds 32768", op, dim); return Q8K_ERR_UNSUPPORTED; }
    // the incoming gradient has the output's dtype (csrc/ops/rms_norm_backward_cuda.cu:117)
    int rc = dispatch_8bit_pair(op, x_dtype, out_dtype, [&](auto* ty, auto* to) {
        using Ty = std::remove_pointer_t<decltype(ty)>;
        using To = std::remove_pointer_t<decltype(to)>;
#define Q8K_RB_LAUNCH(ITEMS, T)                                                                   \
    rms_norm_backward_kernel<Ty, To, To, ITEMS, T><<<(unsigned)rows, T, 0, st>>>(                   \
        (const Ty*)x_normed, x_norms, (const To*)grad_out, weights, (To*)out, dim)
        if (items <= 32)        Q8K_RB_LAUNCH(1, 32);
        else if (items <= 128)  Q8K_RB_LAUNCH(1, 128);
        else if (items <= 256)  Q8K_RB_LAUNCH(2, 128);
        else if (items <= 512)  Q8K_RB_LAUNCH(4, 128);
        else if (items <= 1024) Q8K_RB_LAUNCH(4, 256);
        else if (items <= 2048) Q8K_RB_LAUNCH(8, 256);
        else                    Q8K_RB_LAUNCH(8, 512);
#undef Q8K_RB_LAUNCH
        return Q8K_OK;
    });
    if (rc) return rc;
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}
