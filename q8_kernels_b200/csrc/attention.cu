// FP8 flash-attention forward (head dim 64) on the sm_100a tensor cores, plus
// the pre-pass that turns bf16 q/k/v views into the e4m3 operands it consumes.
//
// Semantics follow csrc/flash_attention/flash_attention_cuda.cu:197-248,395-497
// and flash_attention_cuda_mask.cu:244,319 of the reference: all operands e4m3,
// fp32 scores, KV blocks of 64 keys visited from the LAST to the FIRST with an
// exact running max per block, P re-quantised to e4m3 (saturating) before P.V,
// the row sum taken over the fp32 P, columns >= N get -inf and (masked variant)
// columns >= key_lens[b] get -1e6.  The 64-key granularity of the running max
// is part of the numerics: e4m3(P) depends on which max P was scaled by, and a
// 128-key block moves the result by 3e-3..1e-2 (rel. Frobenius), so the block
// size is kept.  Blocks that lie entirely beyond key_lens[b] are skipped, which
// is numerically identical (their contribution is annihilated by the next
// block's rescale) except for key_lens[b] == 0, where every block is processed
// and the result is the mean of V, as in the reference.
//
// Structure: one CTA per 128 query rows of one (batch, head); 6 warps.
//   warp 0      TMA: Q tile once, then K (64 keys x 64 B) and V^T (64 x 64 keys)
//               tiles, all 64B-swizzled, through KS-deep mbarrier rings
//   warp 1      TMEM allocation; one thread issues S = Q.K^T (2 x tcgen05.mma
//               M128 N64 K32) into one of three S buffers (TMEM columns [0,192))
//               and O += P.V (2 x M128 N64 K32) into columns [192,256)
//   warps 2-5   softmax, one thread per query row: the scores of block i are loaded
//               from TMEM one block ahead (registers double buffered), max, rescale
//               O in TMEM when the max moved, exp2, write P as e4m3 into one of two
//               swizzled shared tiles (the A operand of P.V); at the end O / l ->
//               bf16 or e4m3 -> global
// S is triple and P double buffered, so Q.K^T of blocks i+1..i+3 and P.V of block
// i-1 run under the softmax of block i; two CTAs share an SM (TMEM 2 x 256 columns).

#include "common.cuh"
#include "tcgen05.cuh"
#include "tensormap.cuh"

namespace q8k {

constexpr int kAttnD = 64;
constexpr int kAttnBM = 128;
constexpr int kAttnBN = 64;
constexpr int kAttnKS = 8;                 // K and V ring depth
constexpr int kAttnThreads = 192;
constexpr int kAttnSBufs = 3;              // score buffers in TMEM
constexpr int kAttnTmemCols = 256;         // S0..S2: [0,192), O: [192,256)
constexpr uint32_t kAttnOCol = kAttnSBufs * kAttnBN;

struct AttnSmem {
    static constexpr int kQBytes = kAttnBM * kAttnD;               // 8 KB
    static constexpr int kKBytes = kAttnBN * kAttnD;               // 4 KB per stage
    static constexpr int kVBytes = kAttnD * kAttnBN;               // 4 KB per stage
    static constexpr int kPBytes = kAttnBM * kAttnBN;              // 8 KB per buffer
    static constexpr int kQOff = 0;
    static constexpr int kKOff = kQOff + kQBytes;
    static constexpr int kVOff = kKOff + kAttnKS * kKBytes;
    static constexpr int kPOff = kVOff + kAttnKS * kVBytes;
    static constexpr int kBarOff = kPOff + 2 * kPBytes;
    static constexpr int kNumBars = 1 + 4 * kAttnKS + 2 * kAttnSBufs + 4;
    static constexpr int kTmemPtrOff = kBarOff + kNumBars * 8;
    static constexpr int kAbortOff = kTmemPtrOff + 4;
    static constexpr int kTotal = kAbortOff + 4;
    static constexpr int kDynamic = kTotal + 1024;
};

struct AttnParams {
    void* out;
    const int* key_lens;
    int* status;
    int B, H, M, N;
    float scale_log2;                      // softmax_scale * log2(e)
    int out_e4m3;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// sm_100 packed fp32 pairs (one issue slot for two lanes of FMA-pipe work) and 3-input max
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(d)
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
          "l"(*reinterpret_cast<unsigned long long*>(&c)));
    return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;"
        : "=l"(d)
        : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
    return *reinterpret_cast<float2*>(&d);
}

__global__ void __launch_bounds__(kAttnThreads, 2)
flash_attn_fp8_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
    using L = AttnSmem;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t smem_base = ptx::smem_u32(smem);
    const uint32_t bar_base = smem_base + L::kBarOff;
    const uint32_t q_full = bar_base;
    auto k_full = [&](int s) { return bar_base + 8u * (1 + s); };
    auto k_empty = [&](int s) { return bar_base + 8u * (1 + kAttnKS + s); };
    auto v_full = [&](int s) { return bar_base + 8u * (1 + 2 * kAttnKS + s); };
    auto v_empty = [&](int s) { return bar_base + 8u * (1 + 3 * kAttnKS + s); };
    const uint32_t misc = bar_base + 8u * (1 + 4 * kAttnKS);
    auto s_full = [&](int b) { return misc + 8u * b; };                          // Q.K^T of a block landed in S[b]
    auto s_free = [&](int b) { return misc + 8u * (kAttnSBufs + b); };           // softmax holds S[b] in registers
    auto p_full = [&](int b) { return misc + 8u * (2 * kAttnSBufs + b); };       // softmax wrote P[b] (and rescaled O)
    auto p_free = [&](int b) { return misc + 8u * (2 * kAttnSBufs + 2 + b); };   // P.V that read P[b] retired
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOff);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

    // A launch that follows a failed one on the same status word does nothing.
    __shared__ int prior_failure;
    if (threadIdx.x == 0) prior_failure = p.status != nullptr ? *reinterpret_cast<volatile int*>(p.status) : 0;
    __syncthreads();
    if (prior_failure != 0) return;                            // uniform across the CTA

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int bh = blockIdx.y;
    const int m0 = blockIdx.x * kAttnBM;
    const int b = bh / p.H;

    // key range and block count for this batch entry
    int valid = p.N;                                           // columns >= valid get -1e6
    bool all_masked = false;
    if (p.key_lens != nullptr) {
        valid = p.key_lens[b];
        valid = valid < 0 ? 0 : (valid > p.N ? p.N : valid);
        all_masked = valid == 0;
    }
    const int k_range = all_masked ? p.N : valid;              // keys that are visited at all
    const int nblk = (k_range + kAttnBN - 1) / kAttnBN;

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full, 1);
        for (int s = 0; s < kAttnKS; ++s) {
            ptx::mbar_init(k_full(s), 1);
            ptx::mbar_init(k_empty(s), 1);
            ptx::mbar_init(v_full(s), 1);
            ptx::mbar_init(v_empty(s), 1);
        }
        for (int i = 0; i < kAttnSBufs; ++i) {
            ptx::mbar_init(s_full(i), 1);
            ptx::mbar_init(s_free(i), 128);
        }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(p_full(i), 128);
            ptx::mbar_init(p_free(i), 1);
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::prefetch_tensormap(&tmap_q);
        ptx::prefetch_tensormap(&tmap_k);
        ptx::prefetch_tensormap(&tmap_v);
    }
    if (warp == 1) {
        ptx::tmem_alloc<kAttnTmemCols>(ptx::smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)));
        ptx::tmem_relinquish_alloc_permit();
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            bool ok = true;
            ptx::mbar_arrive_expect_tx(q_full, L::kQBytes);
            ptx::tma_load_3d(smem_base + L::kQOff, &tmap_q, q_full, 0, m0, bh);
            int issued = 0;
            for (int i = 0; ok && i < nblk; ++i) {
                const int jb = nblk - 1 - i;
                const int s = i % kAttnKS;
                const uint32_t ph = (i / kAttnKS) & 1u;
                if (!ptx::mbar_wait(k_empty(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                ptx::mbar_arrive_expect_tx(k_full(s), L::kKBytes);
                ptx::tma_load_3d(smem_base + L::kKOff + s * L::kKBytes, &tmap_k, k_full(s), 0, jb * kAttnBN, bh);
                if (!ptx::mbar_wait(v_empty(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                ptx::mbar_arrive_expect_tx(v_full(s), L::kVBytes);
                ptx::tma_load_3d(smem_base + L::kVOff + s * L::kVBytes, &tmap_v, v_full(s), jb * kAttnBN, 0, bh);
                issued = i + 1;
            }
            if (!ok) {
                if (p.status != nullptr) atomicExch(p.status, Q8K_STATUS_TIMEOUT | (4 << 8));
                // bounded grace period for copies still in flight
                const int first = issued > kAttnKS ? issued - kAttnKS : 0;
                for (int i = first; i < issued; ++i) {
                    const unsigned long long t0 = ptx::globaltimer_ns();
                    while (!(ptx::mbar_try_wait(k_full(i % kAttnKS), (i / kAttnKS) & 1u) &&
                             ptx::mbar_try_wait(v_full(i % kAttnKS), (i / kAttnKS) & 1u)) &&
                           ptx::globaltimer_ns() - t0 < 100000000ull) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t IDESC = ptx::make_idesc_e4m3(kAttnBM, kAttnBN);   // both GEMMs are M128 N64
            const uint64_t q_desc = ptx::make_kmajor_desc(smem_base + L::kQOff, 64);
            const uint32_t o_tmem = tmem_base + kAttnOCol;
            bool ok = ptx::mbar_wait(q_full, 0, abort_flag);

            // S[i % 3] = Q . K(i)^T ; the buffer was last read by the softmax of block i-3
            auto issue_qk = [&](int i) -> bool {
                const int s = i % kAttnKS;
                const int sb = i % kAttnSBufs;
                if (!ptx::mbar_wait(k_full(s), (uint32_t)(i / kAttnKS) & 1u, abort_flag)) return false;
                if (i >= kAttnSBufs &&
                    !ptx::mbar_wait(s_free(sb), (uint32_t)((i - kAttnSBufs) / kAttnSBufs) & 1u, abort_flag))
                    return false;
                ptx::tcgen05_fence_after_sync();
                const uint64_t k_desc = ptx::make_kmajor_desc(smem_base + L::kKOff + s * L::kKBytes, 64);
#pragma unroll
                for (int k = 0; k < kAttnD / 32; ++k)
                    ptx::mma_f8f6f4(tmem_base + sb * kAttnBN, q_desc + 2 * k, k_desc + 2 * k, IDESC, k > 0 ? 1u : 0u);
                ptx::tcgen05_commit(k_empty(s));
                ptx::tcgen05_commit(s_full(sb));
                return true;
            };

            for (int i = 0; ok && i < kAttnSBufs && i < nblk; ++i) ok = issue_qk(i);
            for (int i = 0; ok && i < nblk; ++i) {
                const int s = i % kAttnKS;
                const int pb = i & 1;
                if (!ptx::mbar_wait(v_full(s), (uint32_t)(i / kAttnKS) & 1u, abort_flag)) { ok = false; break; }
                if (!ptx::mbar_wait(p_full(pb), (uint32_t)(i >> 1) & 1u, abort_flag)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                const uint64_t p_desc = ptx::make_kmajor_desc(smem_base + L::kPOff + pb * L::kPBytes, 64);
                const uint64_t v_desc = ptx::make_kmajor_desc(smem_base + L::kVOff + s * L::kVBytes, 64);
#pragma unroll
                for (int k = 0; k < kAttnBN / 32; ++k)
                    ptx::mma_f8f6f4(o_tmem, p_desc + 2 * k, v_desc + 2 * k, IDESC, (i > 0 || k > 0) ? 1u : 0u);
                ptx::tcgen05_commit(v_empty(s));
                ptx::tcgen05_commit(p_free(pb));
                if (i + kAttnSBufs < nblk) {
                    if (!issue_qk(i + kAttnSBufs)) { ok = false; break; }
                }
            }
            if (!ok && p.status != nullptr) atomicExch(p.status, Q8K_STATUS_TIMEOUT | (5 << 8));
        }
    } else {
        // ------------------------------------------------ softmax / correction / epilogue
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                      // row of the tile == TMEM lane
        const int row = m0 + r;
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const float c = p.scale_log2;
        const uint32_t swz = (uint32_t)((r >> 1) & 3);          // 64B swizzle: 16-byte chunk ^= bits [7,9) of the offset

        float m_run = -INFINITY;
        float l_run = 0.f;
        bool ok = true;

        // One 64-key block.  `cur` holds the scores of block i (its TMEM load was issued a step
        // earlier); the load of block i+1 into `nxt` is issued here and lands while the exps run.
        auto step = [&](int i, uint32_t (&cur)[2][32], uint32_t (&nxt)[2][32]) -> bool {
            const int jb = nblk - 1 - i;
            const int col0 = jb * kAttnBN;
            const int sb = i % kAttnSBufs;
            const int pb = i & 1;
            const bool need_mask = (col0 + kAttnBN > valid) || (col0 + kAttnBN > p.N);
            uint8_t* p_row = smem + L::kPOff + pb * L::kPBytes + r * kAttnBN;

            __syncwarp();
            ptx::tmem_wait_ld();                               // scores of block i are in registers
            ptx::tcgen05_fence_before_sync();
            ptx::mbar_arrive(s_free(sb));                      // S[sb] may be overwritten by Q.K^T of block i+3
            if (i + 1 < nblk) {
                const int nb = (i + 1) % kAttnSBufs;
                bool got = ptx::mbar_wait(s_full(nb), (uint32_t)((i + 1) / kAttnSBufs) & 1u, abort_flag);
                if (!__all_sync(0xffffffffu, got)) return false;
                ptx::tcgen05_fence_after_sync();
                ptx::tmem_ld_32x32b_x32(t_lane + nb * kAttnBN, nxt[0]);
                ptx::tmem_ld_32x32b_x32(t_lane + nb * kAttnBN + 32, nxt[1]);
            }

            // row max of the (masked) scores; four independent chains of 3-input max
            float m_blk = -INFINITY;
            if (need_mask) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int col = col0 + h * 32 + j;
                        float sv = __uint_as_float(cur[h][j]);
                        sv = col >= p.N ? -INFINITY : (col >= valid ? -1.0e6f : sv);
                        cur[h][j] = __float_as_uint(sv);
                        m_blk = fmaxf(m_blk, sv);
                    }
            } else {
                float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < 32; j += 8) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            mx[q] = fmax3(mx[q], __uint_as_float(cur[h][j + 2 * q]), __uint_as_float(cur[h][j + 2 * q + 1]));
                    }
                m_blk = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            }
            const float m_new = fmaxf(m_run, m_blk);
            const float m_scaled = m_new == -INFINITY ? 0.f : m_new * c;
            const float alpha = m_run == -INFINITY ? 0.f : fast_exp2((m_run - m_new) * c);

            if (i > 0 && __any_sync(0xffffffffu, m_new != m_run)) {
                // O is complete once P.V of the previous block has retired
                bool got = ptx::mbar_wait(p_free(pb ^ 1), (uint32_t)((i - 1) >> 1) & 1u, abort_flag);
                if (!__all_sync(0xffffffffu, got)) return false;
                ptx::tcgen05_fence_after_sync();
#pragma unroll 1
                for (int h = 0; h < kAttnD / 32; ++h) {
                    uint32_t orow[32];
                    __syncwarp();
                    ptx::tmem_ld_32x32b_x32(t_lane + kAttnOCol + h * 32, orow);
                    ptx::tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) orow[j] = __float_as_uint(__uint_as_float(orow[j]) * alpha);
                    ptx::tmem_st_32x32b_x32(t_lane + kAttnOCol + h * 32, orow);
                }
                ptx::tmem_wait_st();
            }
            if (i >= 2) {
                // P[pb] was the A operand of P.V of block i-2
                bool got = ptx::mbar_wait(p_free(pb), (uint32_t)((i - 2) >> 1) & 1u, abort_flag);
                if (!__all_sync(0xffffffffu, got)) return false;
            }

            // p = 2^(s*c - m*c), fp32 row sum, e4m3 P into the swizzled smem tile
            float row_sum = 0.f;
            if (need_mask) {
                // Masked scores are -1e6: there the product must be rounded before the subtraction
                // (as the unfused reference arithmetic does), or the fma's exact product leaves a
                // residual of up to half an ulp of 1.4e6 in the exponent.
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int g = 0; g < 2; ++g) {
                        uint32_t w[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            float pv[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float sv = __uint_as_float(cur[h][g * 16 + q * 4 + e]);
                                pv[e] = fast_exp2(__fsub_rn(__fmul_rn(sv, c), m_scaled));
                                row_sum += pv[e];
                            }
                            w[q] = (uint32_t)float2_to_e4m3x2_sat(pv[0], pv[1]) |
                                   ((uint32_t)float2_to_e4m3x2_sat(pv[2], pv[3]) << 16);
                        }
                        const uint32_t chunk = (uint32_t)(h * 2 + g) ^ swz;
                        *reinterpret_cast<uint4*>(p_row + chunk * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            } else {
                const float2 c2 = make_float2(c, c);
                const float2 nm2 = make_float2(-m_scaled, -m_scaled);
                float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int g = 0; g < 2; ++g) {
                        uint32_t w[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int j = g * 16 + q * 4;
                            const float2 e0 = ffma2(make_float2(__uint_as_float(cur[h][j]), __uint_as_float(cur[h][j + 1])), c2, nm2);
                            const float2 e1 = ffma2(make_float2(__uint_as_float(cur[h][j + 2]), __uint_as_float(cur[h][j + 3])), c2, nm2);
                            const float2 p0 = make_float2(fast_exp2(e0.x), fast_exp2(e0.y));
                            const float2 p1 = make_float2(fast_exp2(e1.x), fast_exp2(e1.y));
                            sum_a = fadd2(sum_a, p0);
                            sum_b = fadd2(sum_b, p1);
                            w[q] = (uint32_t)float2_to_e4m3x2_sat(p0.x, p0.y) |
                                   ((uint32_t)float2_to_e4m3x2_sat(p1.x, p1.y) << 16);
                        }
                        const uint32_t chunk = (uint32_t)(h * 2 + g) ^ swz;
                        *reinterpret_cast<uint4*>(p_row + chunk * 16) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
                row_sum = (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
            }
            l_run = l_run * alpha + row_sum;
            m_run = m_new;
            ptx::fence_proxy_async_smem();                     // P visible to the tensor core's smem reads
            ptx::tcgen05_fence_before_sync();                  // orders the O rescale before the signal
            ptx::mbar_arrive(p_full(pb));
            return true;
        };

        uint32_t s_a[2][32], s_b[2][32];
        if (nblk > 0) {
            ok = ptx::mbar_wait(s_full(0), 0, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                ptx::tcgen05_fence_after_sync();
                ptx::tmem_ld_32x32b_x32(t_lane, s_a[0]);
                ptx::tmem_ld_32x32b_x32(t_lane + 32, s_a[1]);
            }
        }
        for (int i = 0; ok && i < nblk; i += 2) {
            ok = step(i, s_a, s_b);
            if (ok && i + 1 < nblk) ok = step(i + 1, s_b, s_a);
        }

        // epilogue: O / l
        if (ok && nblk > 0) ok = ptx::mbar_wait(p_free((nblk - 1) & 1), (uint32_t)((nblk - 1) >> 1) & 1u, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            ptx::tcgen05_fence_after_sync();
            const float inv = (l_run == 0.f || l_run != l_run) ? 1.f : 1.f / l_run;
            const int64_t out_off = ((int64_t)bh * p.M + row) * kAttnD;
#pragma unroll 1
            for (int h = 0; h < kAttnD / 32; ++h) {
                uint32_t orow[32];
                __syncwarp();
                if (nblk > 0) {
                    ptx::tmem_ld_32x32b_x32(t_lane + kAttnOCol + h * 32, orow);
                    ptx::tmem_wait_ld();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) orow[j] = 0u;
                }
                if (row < p.M) {
                    float y[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) y[j] = __uint_as_float(orow[j]) * inv;
                    if (p.out_e4m3) {
                        uint8_t* o = reinterpret_cast<uint8_t*>(p.out) + out_off + h * 32;
#pragma unroll
                        for (int v4 = 0; v4 < 2; ++v4) {
                            uint32_t w[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const int j = v4 * 16 + q * 4;
                                w[q] = (uint32_t)float2_to_e4m3x2_sat(y[j], y[j + 1]) |
                                       ((uint32_t)float2_to_e4m3x2_sat(y[j + 2], y[j + 3]) << 16);
                            }
                            reinterpret_cast<uint4*>(o)[v4] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
                        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + out_off + h * 32;
#pragma unroll
                        for (int v4 = 0; v4 < 4; ++v4) {
                            uint32_t w[4];
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                const int j = v4 * 8 + q * 2;
                                __nv_bfloat162 b2 = __floats2bfloat162_rn(y[j], y[j + 1]);
                                w[q] = *reinterpret_cast<uint32_t*>(&b2);
                            }
                            reinterpret_cast<uint4*>(o)[v4] = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    }
                }
            }
        } else if (p.status != nullptr && threadIdx.x == 64) {
            atomicExch(p.status, Q8K_STATUS_TIMEOUT | (6 << 8));
        }
    }

    // ---------------------------------------------------- teardown
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc<kAttnTmemCols>(tmem_base);
    }
}

// ------------------------------------------------------------------ pre-pass kernels
// Q / K: one 64-element head row per group of 8 lanes; optional 64-point
// Hadamard (fp32 butterflies, ascending stride), times `scale`, cast c10-style
// to e4m3, written head-major [B,H,S,64].
__global__ void __launch_bounds__(128)
attn_prep_qk_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ out, int B, int H, int S,
                    int64_t stride_b, int64_t stride_s, int64_t stride_h, int apply_hadamard, float scale) {
    const int lane = threadIdx.x & 31;
    const int sub = lane & 7;
    const int64_t grp = (int64_t)blockIdx.x * 16 + (threadIdx.x >> 3);   // (b, s, h) flattened, h fastest
    const int64_t total = (int64_t)B * S * H;
    const bool row_ok = grp < total;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = 0.f;
    int h = 0, s = 0, b = 0;
    if (row_ok) {
        h = (int)(grp % H);
        s = (int)((grp / H) % S);
        b = (int)(grp / ((int64_t)H * S));
        load_vec<__nv_bfloat16, 8>(x + b * stride_b + s * stride_s + h * stride_h + sub * 8, v);
    }
    if (apply_hadamard) {
#pragma unroll
        for (int st = 1; st < 8; st <<= 1) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int lo = j & (st - 1);
                const int i = ((j - lo) << 1) + lo;
                const float a = v[i], bb = v[i + st];
                v[i] = __fadd_rn(a, bb);
                v[i + st] = __fsub_rn(a, bb);
            }
        }
#pragma unroll
        for (int mk = 1; mk < 8; mk <<= 1) {
            const bool upper = (lane & mk) != 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float other = __shfl_xor_sync(0xffffffffu, v[j], mk);
                v[j] = upper ? __fsub_rn(other, v[j]) : __fadd_rn(v[j], other);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = __fmul_rn(v[j], scale);
    }
    if (row_ok) {
        union { uint2 v2; uint8_t bts[8]; } o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.bts[j] = float_to_e4m3_c10(v[j]);
        *reinterpret_cast<uint2*>(out + (((int64_t)b * H + h) * S + s) * 64 + sub * 8) = o.v2;
    }
}

// V: [B,S,H,64] bf16 view -> vt [B,H,64,S_pad] e4m3, zero padded along S.
__global__ void __launch_bounds__(256)
attn_prep_v_kernel(const __nv_bfloat16* __restrict__ v, uint8_t* __restrict__ vt, int H, int S, int S_pad,
                   int64_t stride_b, int64_t stride_s, int64_t stride_h) {
    __shared__ __align__(16) uint8_t tile[64][80];                           // [d][s], padded row to spread banks
    const int bh = blockIdx.y;
    const int b = bh / H, h = bh % H;
    const int s0 = blockIdx.x * 64;
    const int sub = threadIdx.x & 7;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
        const int sl = pass * 32 + (threadIdx.x >> 3);
        const int s = s0 + sl;
        float x[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = 0.f;
        if (s < S) load_vec<__nv_bfloat16, 8>(v + b * stride_b + s * stride_s + h * stride_h + sub * 8, x);
#pragma unroll
        for (int j = 0; j < 8; ++j) tile[sub * 8 + j][sl] = s < S ? float_to_e4m3_c10(x[j]) : (uint8_t)0;
    }
    __syncthreads();
    const int d = threadIdx.x >> 2;
    const int sc = (threadIdx.x & 3) * 16;
    if (s0 + sc < S_pad) {
        const uint4 val = *reinterpret_cast<const uint4*>(&tile[d][sc]);
        *reinterpret_cast<uint4*>(vt + ((int64_t)bh * 64 + d) * S_pad + s0 + sc) = val;
    }
}

}  // namespace q8k

using namespace q8k;

extern "C" int q8k_flash_attention(const void* q, const void* k, const void* vt, void* out, int out_dtype,
                                   int B, int H, int M, int N, float softmax_scale, const int* key_lens,
                                   int* dev_status, void* stream) {
    const char* op = "flash_attention";
    Q8K_REQUIRE(q && k && vt && out, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE(B > 0 && H > 0 && M >= 0 && N > 0, Q8K_ERR_INVALID_ARG, "%s: bad shape B=%d H=%d M=%d N=%d", op, B, H, M, N);
    Q8K_REQUIRE(aligned16(q) && aligned16(k) && aligned16(vt) && aligned16(out), Q8K_ERR_INVALID_ARG,
                "%s: q, k, vt and out must be 16-byte aligned", op);
    Q8K_REQUIRE(out_dtype == Q8K_DT_E4M3 || out_dtype == Q8K_DT_BF16, Q8K_ERR_UNSUPPORTED,
                "%s: output dtype %d is not e4m3 or bf16", op, out_dtype);
    Q8K_REQUIRE((int64_t)B * H <= 65535, Q8K_ERR_TOO_LARGE, "%s: B*H = %lld exceeds 65535", op, (long long)B * H);
    if (M == 0) return Q8K_OK;
    const int n_pad = (N + 15) / 16 * 16;
    const uint64_t BH = (uint64_t)B * H;

    CUtensorMap tq, tk, tv;
    {
        const uint64_t dims[3] = {64, (uint64_t)M, BH};
        const uint64_t strides[2] = {64, (uint64_t)M * 64};
        const uint32_t box[3] = {64, (uint32_t)kAttnBM, 1};
        if (int rc = make_byte_tensor_map(&tq, q, 3, dims, strides, box, 64, op)) return rc;
    }
    {
        const uint64_t dims[3] = {64, (uint64_t)N, BH};
        const uint64_t strides[2] = {64, (uint64_t)N * 64};
        const uint32_t box[3] = {64, (uint32_t)kAttnBN, 1};
        if (int rc = make_byte_tensor_map(&tk, k, 3, dims, strides, box, 64, op)) return rc;
    }
    {
        const uint64_t dims[3] = {(uint64_t)n_pad, 64, BH};
        const uint64_t strides[2] = {(uint64_t)n_pad, (uint64_t)n_pad * 64};
        const uint32_t box[3] = {(uint32_t)kAttnBN, 64, 1};
        if (int rc = make_byte_tensor_map(&tv, vt, 3, dims, strides, box, 64, op)) return rc;
    }

    AttnParams p;
    p.out = out;
    p.key_lens = key_lens;
    p.status = dev_status;
    p.B = B; p.H = H; p.M = M; p.N = N;
    p.scale_log2 = (float)((double)softmax_scale * 1.4426950408889634);
    p.out_e4m3 = out_dtype == Q8K_DT_E4M3;

    Q8K_CUDA_OK(cudaFuncSetAttribute(flash_attn_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem::kDynamic));
    dim3 grid((unsigned)((M + kAttnBM - 1) / kAttnBM), (unsigned)BH);
    flash_attn_fp8_kernel<<<grid, kAttnThreads, AttnSmem::kDynamic, (cudaStream_t)stream>>>(tq, tk, tv, p);
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

extern "C" int q8k_attention_prep(const void* q, const void* k, const void* v, void* q8, void* k8, void* vt8,
                                  int B, int H, int S_q, int S_kv,
                                  int64_t q_stride_b, int64_t q_stride_s, int64_t q_stride_h,
                                  int64_t k_stride_b, int64_t k_stride_s, int64_t k_stride_h,
                                  int64_t v_stride_b, int64_t v_stride_s, int64_t v_stride_h,
                                  int apply_hadamard, float qk_scale, void* stream) {
    const char* op = "attention_prep";
    Q8K_REQUIRE(q && k && v && q8 && k8 && vt8, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE(B > 0 && H > 0 && S_q > 0 && S_kv > 0, Q8K_ERR_INVALID_ARG, "%s: bad shape", op);
    Q8K_REQUIRE((int64_t)B * H <= 65535, Q8K_ERR_TOO_LARGE, "%s: B*H exceeds 65535", op);
    const int64_t all_strides[9] = {q_stride_b, q_stride_s, q_stride_h, k_stride_b, k_stride_s, k_stride_h,
                                    v_stride_b, v_stride_s, v_stride_h};
    for (int i = 0; i < 9; ++i)
        Q8K_REQUIRE(all_strides[i] % 8 == 0, Q8K_ERR_INVALID_ARG, "%s: strides must be multiples of 8 elements", op);
    Q8K_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(q8) && aligned16(k8) && aligned16(vt8),
                Q8K_ERR_INVALID_ARG, "%s: pointers must be 16-byte aligned", op);
    cudaStream_t st = (cudaStream_t)stream;
    const int s_pad = (S_kv + 15) / 16 * 16;
    {
        const int64_t rows = (int64_t)B * S_q * H;
        attn_prep_qk_kernel<<<(unsigned)((rows + 15) / 16), 128, 0, st>>>(
            (const __nv_bfloat16*)q, (uint8_t*)q8, B, H, S_q, q_stride_b, q_stride_s, q_stride_h, apply_hadamard, qk_scale);
    }
    {
        const int64_t rows = (int64_t)B * S_kv * H;
        attn_prep_qk_kernel<<<(unsigned)((rows + 15) / 16), 128, 0, st>>>(
            (const __nv_bfloat16*)k, (uint8_t*)k8, B, H, S_kv, k_stride_b, k_stride_s, k_stride_h, apply_hadamard, qk_scale);
    }
    {
        dim3 grid((unsigned)((S_kv + 63) / 64), (unsigned)(B * H));
        attn_prep_v_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)v, (uint8_t*)vt8, H, S_kv, s_pad,
                                                 v_stride_b, v_stride_s, v_stride_h);
    }
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}
