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
// Structure: one CTA per 128 query rows of one (batch, head), two warpgroups
// whose register budgets are rebalanced with setmaxnreg (24 / 136 per thread),
// three CTAs per SM (registers; 3 x 128 TMEM columns).
//   warp 0      TMA: Q tile once, then K (64 keys x 64 B) and V (as 64 x 64 rows, or V^T as the
//               reference lays it out) tiles, all 64B-swizzled, into rings of three; one wait per block
//   warp 1      TMEM allocation; one thread issues O += P.V (2 x tcgen05.mma M128 N64 K32) into TMEM
//               columns [64,128)
//   warp 2      one thread issues S = Q.K^T (2 x M128 N64 K32) into columns [0,64); the two issuing
//               threads run side by side, one blocking wait per block each
//   warps 4-7   softmax, one thread per query row: the scores of block i sit in
//               registers (each half is refilled from TMEM with block i+1 as soon
//               as its exps are done), max, exp2, P as e4m3 into one of two
//               swizzled shared tiles (the A operand of P.V), then -- only when a
//               row max of the warp moved -- O *= alpha in TMEM through the
//               registers of the finished half; at the end O / l is parked in the warp's own
//               P rows and leaves through TMA stores (whole-row plain stores for several outputs)
// Three mbarriers carry the steady state: step_end (softmax -> MMA threads: P written, O
// rescaled, S read), s_full (one commit from each MMA thread -> softmax: next scores landed AND the
// previous P.V retired) and slot_free (MMA -> TMA).  Every wait is on consecutive phases
// of its barrier, no barrier can complete a second phase before its waiters have seen the first,
// so a parity is never ambiguous; and every wait is bounded.
// With at most three key blocks (cross-attention) a CTA keeps K/V and walks over several query
// tiles: see the MULTI template parameter.

#include <type_traits>

#include "common.cuh"
#include "tcgen05.cuh"
#include "tensormap.cuh"

namespace q8k {

constexpr int kAttnD = 64;
constexpr int kAttnBM = 128;
constexpr int kAttnBN = 64;
constexpr int kAttnKS = 3;                   // K and V ring depth
constexpr int kAttnThreads = 256;            // warpgroup 0: TMA + MMA, warpgroup 1: softmax
constexpr int kAttnRegsLaunch = 80;          // registers per thread at launch: 3 CTAs x 256 threads x 80 = 61440
constexpr int kAttnRegsIo = 24;              // after setmaxnreg: TMA / MMA warpgroup
constexpr int kAttnRegsSoftmax = 136;        //                    softmax warpgroup (2 * 80 = 24 + 136)
constexpr int kAttnTmemCols = 128;           // S: [0,64), O: [64,128)
constexpr uint32_t kAttnOCol = kAttnBN;

struct AttnSmem {
    static constexpr int kQBytes = kAttnBM * kAttnD;               // 8 KB
    static constexpr int kKBytes = kAttnBN * kAttnD;               // 4 KB per stage
    static constexpr int kVBytes = kAttnD * kAttnBN;               // 4 KB per stage
    static constexpr int kPBytes = kAttnBM * kAttnBN;              // 8 KB per buffer
    static constexpr int kQOff = 0;
    static constexpr int kKOff = kQOff + kQBytes;
    static constexpr int kVOff = kKOff + kAttnKS * kKBytes;
    static constexpr int kPOff = kVOff + kAttnKS * kVBytes;
    static constexpr int kQ2Off = kPOff + 2 * kPBytes;             // second Q buffer (several query tiles per CTA)
    static constexpr int kBarOff = kQ2Off + kQBytes;
    // q_full[2], k_full[3], v_full[3], slot_free, s_full, step_end, q_free[2]
    static constexpr int kNumBars = 2 + 2 * kAttnKS + 3 + 2;
    static constexpr int kTmemPtrOff = kBarOff + kNumBars * 8;
    static constexpr int kAbortOff = kTmemPtrOff + 4;
    static constexpr int kTotal = kAbortOff + 4;
    static constexpr int kDynamic = kTotal + 1024;
};

constexpr int kAttnMaxOut = 8;           // destinations of the output tile: this GPU's buffer and up to 7 peers'

struct AttnParams {
    void* outs[kAttnMaxOut];               // same layout and strides in every destination
    int n_out;
    const int* key_lens;
    int* status;
    int B, H, M, N;
    float scale_log2;                      // softmax_scale * log2(e)
    int out_e4m3;
    int tma_out;                           // 1: one destination, stored through tmap_o; 2: same, rows before heads in the map
    int64_t out_stride_b, out_stride_h, out_stride_s;   // output strides in elements (head dim contiguous)
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <int N> __device__ __forceinline__ void reg_dealloc() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N> __device__ __forceinline__ void reg_alloc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
// 2^x for two finite x <= 0 on the FMA pipe instead of the 16-lane exp2 unit, which is the busiest unit of this
// kernel: x is rounded to the nearest integer with the 1.5 * 2^23 trick, a quartic in the remainder f in [-0.5, 0.5]
// follows (max relative error 2.7e-6, far below half a step of the e4m3 rounding P goes through), and the integer is
// added into the exponent field.  x is clamped at -126 first (any finite or infinite input is safe).  The softmax
// step takes this path for one score in eight: more of them cost more issue slots than the exp2 unit gives back
// (measured: 1/8 -> -1.8 %, 1/4 -> -0.5 %, 1/2 -> +8 %).
__device__ __forceinline__ float2 exp2_poly2(float2 x) {
    // below -126 the result is 2^-126 (as good as the zero ex2.approx.ftz returns) and the shift below cannot wrap
    x = make_float2(fmaxf(x.x, -126.0f), fmaxf(x.y, -126.0f));
    const float2 magic = make_float2(12582912.0f, 12582912.0f);
    const float2 t = fadd2(x, magic);
    const float2 r = fadd2(t, make_float2(-12582912.0f, -12582912.0f));
    const float2 f = fadd2(x, make_float2(-r.x, -r.y));
    float2 p = ffma2(f, make_float2(0.009574017487466335f, 0.009574017487466335f),
                     make_float2(0.05591818317770958f, 0.05591818317770958f));
    p = ffma2(p, f, make_float2(0.2402464896440506f, 0.2402464896440506f));
    p = ffma2(p, f, make_float2(0.6931217312812805f, 0.6931217312812805f));
    p = ffma2(p, f, make_float2(0.9999992847442627f, 0.9999992847442627f));
    return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23)),
                       __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23)));
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint32_t pack4_e4m3(float a, float b, float c, float d) {
    uint32_t r;
    asm("{\n\t"
        ".reg .b16 lo, hi;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
        "mov.b32 %0, {lo, hi};\n\t"
        "}"
        : "=r"(r)
        : "f"(a), "f"(b), "f"(c), "f"(d));
    return r;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

// All waits of this kernel: see ptx::mbar_wait_bounded.  A wait that gave up returns like one
// that succeeded, so no control flow hangs off its result: the kernel runs to its end on garbage
// and reports the abort word through the status word.
__device__ __forceinline__ void bounded_wait(uint32_t bar, uint32_t parity, uint32_t abort_addr, uint32_t site) {
    ptx::mbar_wait_bounded(bar, parity, abort_addr, site, ptx::kSpinLimit);
}

// V_ROWS = false: V arrives transposed, [B,H,64,ceil16(N)] (the reference's layout), and is the K-major B
// operand of P.V.  V_ROWS = true: V arrives as rows, [B,H,N,64] like K, is loaded by the same kind of TMA
// box and read by the tensor core as an MN-major B operand, so no transpose pass is needed.
// MULTI = true (short key sequences, at most kAttnKS blocks: cross-attention): a CTA keeps K and V of its
// (batch, head) in shared memory and walks over several query tiles (blockIdx.x, + gridDim.x, ...), so that
// barrier set-up, TMEM allocation and the K/V loads are paid once per CTA instead of once per 128 rows.
template <bool V_ROWS, bool MULTI>
__global__ void __maxnreg__(kAttnRegsLaunch)
flash_attn_fp8_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
               const AttnParams p) {
    using L = AttnSmem;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t smem_base = ptx::smem_u32(smem);
    const uint32_t bar_base = smem_base + L::kBarOff;
    auto q_full = [&](int i) { return bar_base + 8u * i; };
    auto k_full = [&](int s) { return bar_base + 8u * (2 + s); };
    auto v_full = [&](int s) { return bar_base + 8u * (2 + kAttnKS + s); };
    // The three below complete their phases in a fixed order (per query tile: slot_free nblk, s_full nblk + 2,
    // step_end nblk + 1, or nblk + 2 with MULTI) and every waiter consumes them in that order.  No barrier can
    // be more than one completed phase ahead of a thread that still has to wait on it: the protocol makes
    // every producer depend on that waiter before it can complete a second one.
    const uint32_t slot_free = bar_base + 8u * (2 + 2 * kAttnKS);   // P.V(i) and Q.K^T(i+2) retired
    const uint32_t s_full = slot_free + 8u;                         // see the MMA issuer
    const uint32_t step_end = slot_free + 16u;                      // softmax: prologue, one per step, (MULTI) epilogue reached
    auto q_free = [&](int i) { return slot_free + 24u + 8u * i; };  // MULTI: all tensor-core reads of Q buffer i retired
    auto q_off = [&](int i) { return (uint32_t)(i ? L::kQ2Off : L::kQOff); };
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOff);
    const uint32_t abort_addr = smem_base + L::kAbortOff;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOff);

    __shared__ int prior_failure;
    if (threadIdx.x == 0) prior_failure = p.status != nullptr ? *reinterpret_cast<volatile int*>(p.status) : 0;
    __syncthreads();
    if (prior_failure != 0) return;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int bh = blockIdx.y;
    const int b = bh / p.H;
    // query tiles of this CTA: tile0, tile0 + tstride, ... (one tile unless MULTI)
    const int tile0 = blockIdx.x;
    const int tstride = MULTI ? (int)gridDim.x : 1;
    const int n_tiles = MULTI ? ((p.M + kAttnBM - 1) / kAttnBM - tile0 + tstride - 1) / tstride : 1;

    int valid = p.N;
    bool all_masked = false;
    if (p.key_lens != nullptr) {
        valid = p.key_lens[b];
        valid = valid < 0 ? 0 : (valid > p.N ? p.N : valid);
        all_masked = valid == 0;
    }
    const int k_range = all_masked ? p.N : valid;
    const int nblk = (k_range + kAttnBN - 1) / kAttnBN;          // >= 1

    if (threadIdx.x == 0) {
        ptx::mbar_init(q_full(0), 1);
        ptx::mbar_init(q_full(1), 1);
        for (int s = 0; s < kAttnKS; ++s) {
            ptx::mbar_init(k_full(s), 1);
            ptx::mbar_init(v_full(s), 1);
        }
        ptx::mbar_init(slot_free, 1);
        ptx::mbar_init(s_full, 2);                              // one commit from each of the two MMA-issuing threads
        ptx::mbar_init(step_end, 4);
        ptx::mbar_init(q_free(0), 1);
        ptx::mbar_init(q_free(1), 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::prefetch_tensormap(&tmap_q);
        ptx::prefetch_tensormap(&tmap_k);
        ptx::prefetch_tensormap(&tmap_v);
        if (p.tma_out) ptx::prefetch_tensormap(&tmap_o);
    }
    if (warp == 1) {
        ptx::tmem_alloc<kAttnTmemCols>(ptx::smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)));
        ptx::tmem_relinquish_alloc_permit();
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;

    auto teardown_barrier = [&]() {
        ptx::tcgen05_fence_before_sync();
        asm volatile("bar.sync 0, %0;" ::"n"(kAttnThreads) : "memory");
    };
    if (warp < 4) {
        reg_dealloc<kAttnRegsIo>();
        if (warp == 0) {
            // -------------------------------------------- TMA producer
            if (lane == 0) {
                auto load_q = [&](int t) {                      // query tile t of this CTA into Q buffer t & 1
                    ptx::mbar_arrive_expect_tx(q_full(t & 1), L::kQBytes);
                    ptx::tma_load_3d(smem_base + q_off(t & 1), &tmap_q, q_full(t & 1), 0, (tile0 + t * tstride) * kAttnBM, bh);
                };
                load_q(0);
                auto load_kv = [&](int j) {                     // block j (visit order) into slot j % 3
                    const int jb = nblk - 1 - j;
                    const int s = j % kAttnKS;
                    ptx::mbar_arrive_expect_tx(k_full(s), L::kKBytes);
                    ptx::tma_load_3d(smem_base + L::kKOff + s * L::kKBytes, &tmap_k, k_full(s), 0, jb * kAttnBN, bh);
                    ptx::mbar_arrive_expect_tx(v_full(s), L::kVBytes);
                    if (V_ROWS) ptx::tma_load_3d(smem_base + L::kVOff + s * L::kVBytes, &tmap_v, v_full(s), 0, jb * kAttnBN, bh);
                    else ptx::tma_load_3d(smem_base + L::kVOff + s * L::kVBytes, &tmap_v, v_full(s), jb * kAttnBN, 0, bh);
                };
                const int first = nblk < kAttnKS ? nblk : kAttnKS;
                for (int j = 0; j < first; ++j) load_kv(j);
                if constexpr (MULTI) {
                    // K and V stay where they are (nblk <= kAttnKS).  Q(t+2) goes into the buffer of tile t
                    // once all tensor-core work of tile t has retired.
                    if (n_tiles > 1) load_q(1);
                    for (int t = 0; t + 2 < n_tiles; ++t) {
                        bounded_wait(q_free(t & 1), (uint32_t)(t >> 1) & 1u, abort_addr, 4);
                        if (*abort_flag != 0) break;
                        load_q(t + 2);
                    }
                } else {
                    for (int i = 0; i + kAttnKS < nblk; ++i) {
                        // K(i) was consumed before step i, V(i) by P.V(i): both slots i % 3 are free
                        bounded_wait(slot_free, (uint32_t)i & 1u, abort_addr, 4);
                        if (*abort_flag != 0) break;            // a wait was abandoned: issue nothing more
                        load_kv(i + kAttnKS);
                    }
                }
                // (slot_free phases that are never waited on simply complete.)
                if (*abort_flag != 0) {
                    // grace period for copies still in flight: they land within microseconds
                    const unsigned long long t0 = ptx::globaltimer_ns();
                    while (ptx::globaltimer_ns() - t0 < 50000ull) {}
                }
            }
        } else if (warp == 1 || warp == 2) {
            // -------------------------------------------- MMA issuers: warp 1 issues O += P.V, warp 2 issues S = Q.K^T.
            // The two chains touch different accumulators and operands, and each issue costs the issuing thread
            // several hundred clocks (wait, descriptors, two MMAs, commit); side by side, the scores of block
            // i+2 are on their way half as long after step i ends as when one thread issued both.
            // s_full takes one commit from each thread per phase.  Phases of one tile: 0 = Q.K^T(0); 1 = Q.K^T(1)
            // (if any); i+2 = P.V(i) and Q.K^T(i+2) (if any).  So phase i+1, which the softmax warps wait for in
            // the middle of step i, says that the scores of block i+1 are in TMEM AND (i >= 1) that O holds P.V
            // up to block i-1; phase nblk+1 says that O is complete.
            if (lane == 0) {
                constexpr uint32_t IDESC = ptx::make_idesc_e4m3(kAttnBM, kAttnBN);
                // P.V with V as rows: B operand MN-major (bit 16); its 32-key K slices are 32 rows of 64 bytes apart
                constexpr uint32_t IDESC_PV = V_ROWS ? (IDESC | (1u << 16)) : IDESC;
                constexpr uint32_t V_KSTEP = V_ROWS ? (32 * 64) >> 4 : 2;
                const uint32_t s_tmem = tmem_base;
                const uint32_t o_tmem = tmem_base + kAttnOCol;
                const bool pv_thread = warp == 1;
                for (int t = 0; t < n_tiles; ++t) {
                    const uint32_t e_base = MULTI ? (uint32_t)t * (uint32_t)(nblk + 2) : 0u;   // step_end phases of earlier tiles
                    // The softmax warps must have seen the last s_full phase of the tile before (they then
                    // arrive once more) before this tile completes another one.
                    if (MULTI && t > 0) bounded_wait(step_end, (e_base - 1u) & 1u, abort_addr, 5);
                    if (pv_thread) {
                        ptx::tcgen05_commit(s_full);             // phases 0 and 1 carry no P.V: this thread's share is empty
                        bounded_wait(step_end, e_base & 1u, abort_addr, 5);
                        ptx::tcgen05_commit(s_full);
                        for (int i = 0; i < nblk; ++i) {
                            const int s = i % kAttnKS;
                            bounded_wait(step_end, (e_base + (uint32_t)i + 1u) & 1u, abort_addr, 5);   // P(i) written, O rescaled
                            bounded_wait(v_full(s), (uint32_t)(i / kAttnKS) & 1u, abort_addr, 5);
                            ptx::tcgen05_fence_after_sync();
                            const uint64_t p_desc = ptx::make_kmajor_desc(smem_base + L::kPOff + (i & 1) * L::kPBytes, 64);
                            const uint64_t v_desc = ptx::make_kmajor_desc(smem_base + L::kVOff + s * L::kVBytes, 64);
#pragma unroll
                            for (int k = 0; k < kAttnBN / 32; ++k)
                                ptx::mma_f8f6f4(o_tmem, p_desc + 2 * k, v_desc + V_KSTEP * k, IDESC_PV, (i > 0 || k > 0) ? 1u : 0u);
                            ptx::tcgen05_commit(s_full);
                            // K(i) was read by Q.K^T(i), whose scores the softmax warps have long consumed
                            ptx::tcgen05_commit(slot_free);
                        }
                        // (the last Q.K^T of the tile retired before the softmax warps could finish its block)
                        if (MULTI) ptx::tcgen05_commit(q_free(t & 1));
                    } else {
                        const uint64_t q_desc = ptx::make_kmajor_desc(smem_base + q_off(t & 1), 64);
                        auto issue_qk = [&](int j) {
                            const int s = j % kAttnKS;
                            bounded_wait(k_full(s), (uint32_t)(j / kAttnKS) & 1u, abort_addr, 5);
                            ptx::tcgen05_fence_after_sync();
                            const uint64_t k_desc = ptx::make_kmajor_desc(smem_base + L::kKOff + s * L::kKBytes, 64);
#pragma unroll
                            for (int k = 0; k < kAttnD / 32; ++k)
                                ptx::mma_f8f6f4(s_tmem, q_desc + 2 * k, k_desc + 2 * k, IDESC, k > 0 ? 1u : 0u);
                        };
                        bounded_wait(q_full(t & 1), (uint32_t)(t >> 1) & 1u, abort_addr, 5);
                        issue_qk(0);                             // (the score tile is free: S(last) of the tile before
                        ptx::tcgen05_commit(s_full);             //  went to registers before its last step ended)
                        bounded_wait(step_end, e_base & 1u, abort_addr, 5);      // S(0) is in registers
                        if (nblk > 1) issue_qk(1);
                        ptx::tcgen05_commit(s_full);
                        for (int i = 0; i < nblk; ++i) {
                            bounded_wait(step_end, (e_base + (uint32_t)i + 1u) & 1u, abort_addr, 5);   // S(i+1) is in registers
                            if (i + 2 < nblk) issue_qk(i + 2);
                            ptx::tcgen05_commit(s_full);
                        }
                    }
                }
            }
        }
        teardown_barrier();
        if (warp == 1) {
            __syncwarp();
            ptx::tcgen05_fence_after_sync();
            ptx::tmem_dealloc<kAttnTmemCols>(tmem_base);
        }
    } else {
        reg_alloc<kAttnRegsSoftmax>();
        // ------------------------------------------------ softmax / O rescale / epilogue
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        const uint32_t t_lane = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const float c = p.scale_log2;
        const uint32_t swz = (uint32_t)((r >> 1) & 3);
        // this row's 16-byte chunk ch of P buffer 0 sits at p_a0 ^ (ch << 4) (64B swizzle; the row starts 64-byte aligned)
        const uint32_t p_a0 = (smem_base + L::kPOff + (uint32_t)r * kAttnBN) | (swz << 4);

        uint32_t cur[2][32];
#pragma unroll 1
        for (int t = 0; t < n_tiles; ++t) {
        const int row = (tile0 + t * tstride) * kAttnBM + r;
        const uint32_t s_base = MULTI ? (uint32_t)t * (uint32_t)(nblk + 2) : 0u;   // s_full phases of earlier tiles
        float m_run = -INFINITY;
        float l_run = 0.f;

        bounded_wait(s_full, s_base & 1u, abort_addr, 6);
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_ld_32x32b_x32(t_lane, cur[0]);
        ptx::tmem_ld_32x32b_x32(t_lane + 32, cur[1]);
        ptx::tmem_wait_ld();
        ptx::tcgen05_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(step_end);

        // the output boxes of the tile before sit in this warp's P rows until TMA has read them out
        if (MULTI && t > 0 && p.tma_out) {
            if (lane == 0) ptx::bulk_wait_group_read<0>();
            __syncwarp();
        }

        // columns >= N get -inf, columns >= key_lens[b] the reference's mask value
        auto mask_scores = [&](int i) {
            const int col0 = (nblk - 1 - i) * kAttnBN;
            if (col0 + kAttnBN > valid || col0 + kAttnBN > p.N) {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int col = col0 + h * 32 + j;
                        const float sv = __uint_as_float(cur[h][j]);
                        cur[h][j] = __float_as_uint(col >= p.N ? -INFINITY : (col >= valid ? -1.0e6f : sv));
                    }
            }
        };

        // One step.  UNFUSED: products rounded before the subtraction (batch entries without a
        // single valid key, where every score is the mask value and 2^0 must come out exactly).
        auto step = [&](int i, auto unfused_tag, auto poly_tag, uint32_t pb_off) {
            constexpr bool UNFUSED = decltype(unfused_tag)::value;
            constexpr bool POLY = decltype(poly_tag)::value && !UNFUSED;     // exp2_poly2 for one score in eight
            if (UNFUSED) mask_scores(i);
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        mx[q] = fmax3(mx[q], __uint_as_float(cur[h][j + 2 * q]), __uint_as_float(cur[h][j + 2 * q + 1]));
                }
            const float m_new = fmaxf(fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])), m_run);   // finite: a block has a key < N
            const float m_scaled = m_new * c;
            const float alpha = fast_exp2((m_run - m_new) * c);     // first step: 2^-inf = 0
            const bool rescale = i > 0 && __any_sync(0xffffffffu, m_new != m_run);
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
                        float2 e0, e1;
                        if (UNFUSED) {
                            e0 = make_float2(__fsub_rn(__fmul_rn(__uint_as_float(cur[h][j]), c), m_scaled),
                                             __fsub_rn(__fmul_rn(__uint_as_float(cur[h][j + 1]), c), m_scaled));
                            e1 = make_float2(__fsub_rn(__fmul_rn(__uint_as_float(cur[h][j + 2]), c), m_scaled),
                                             __fsub_rn(__fmul_rn(__uint_as_float(cur[h][j + 3]), c), m_scaled));
                        } else {
                            e0 = ffma2(make_float2(__uint_as_float(cur[h][j]), __uint_as_float(cur[h][j + 1])), c2, nm2);
                            e1 = ffma2(make_float2(__uint_as_float(cur[h][j + 2]), __uint_as_float(cur[h][j + 3])), c2, nm2);
                        }
                        const float2 p0 = make_float2(fast_exp2(e0.x), fast_exp2(e0.y));
                        const float2 p1 = (POLY && (q == 3)) ? exp2_poly2(e1) : make_float2(fast_exp2(e1.x), fast_exp2(e1.y));
                        sum_a = fadd2(sum_a, p0);
                        sum_b = fadd2(sum_b, p1);
                        w[q] = pack4_e4m3(p0.x, p0.y, p1.x, p1.y);
                    }
                    st_shared_v4((p_a0 + pb_off) ^ ((uint32_t)(h * 2 + g) << 4), w[0], w[1], w[2], w[3]);
                }
                if (h == 0) {
                    // scores of block i+1 are in TMEM; for i >= 1 also: P.V(i-1) has retired
                    bounded_wait(s_full, (s_base + (uint32_t)i + 1u) & 1u, abort_addr, 6);
                    ptx::tcgen05_fence_after_sync();
                    if (i + 1 < nblk) ptx::tmem_ld_32x32b_x32(t_lane, cur[0]);
                }
            }
            l_run = l_run * alpha + ((sum_a.x + sum_a.y) + (sum_b.x + sum_b.y));
            m_run = m_new;
            if (rescale) {
                // O *= alpha, two 32-column halves through the registers of the dead second half
                const float2 al2 = make_float2(alpha, alpha);
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    ptx::tmem_ld_32x32b_x32(t_lane + kAttnOCol + hh * 32, cur[1]);
                    ptx::tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float2 m = fmul2(make_float2(__uint_as_float(cur[1][j]), __uint_as_float(cur[1][j + 1])), al2);
                        cur[1][j] = __float_as_uint(m.x);
                        cur[1][j + 1] = __float_as_uint(m.y);
                    }
                    ptx::tmem_st_32x32b_x32(t_lane + kAttnOCol + hh * 32, cur[1]);
                }
                ptx::tmem_wait_st();
            }
            if (i + 1 < nblk) ptx::tmem_ld_32x32b_x32(t_lane + 32, cur[1]);
            ptx::fence_proxy_async_smem();                      // P visible to the tensor core's smem reads
            ptx::tmem_wait_ld();                                // S is free once block i+1 sits in registers
            ptx::tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(step_end);
        };

        if (!all_masked) {
            mask_scores(0);                                     // only the block visited first can be partial
#pragma unroll 1
            // (the block visited first may hold -inf / mask values: every element of it goes to the exp2 unit)
            step(0, std::false_type{}, std::false_type{}, 0u);
            if (nblk > 1) step(1, std::false_type{}, std::true_type{}, (uint32_t)L::kPBytes);
#pragma unroll 1
            for (int i = 2; i < nblk; i += 2) {
                step(i, std::false_type{}, std::true_type{}, 0u);
                if (i + 1 < nblk) step(i + 1, std::false_type{}, std::true_type{}, (uint32_t)L::kPBytes);
            }
        } else {
#pragma unroll 1
            for (int i = 0; i < nblk; ++i) step(i, std::true_type{}, std::false_type{}, (uint32_t)(i & 1) * L::kPBytes);
        }

        // epilogue: O / l
        bounded_wait(s_full, (s_base + (uint32_t)nblk + 1u) & 1u, abort_addr, 7);
        ptx::tcgen05_fence_after_sync();
        if (MULTI) {                                            // the next tile's scores may now be produced
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(step_end);
        }
        {
            // O / l goes through shared memory so that the global stores are whole rows: every thread
            // converts its own row and parks it in the P rows of its warp (32 rows x 64 bytes in each of
            // the two P buffers, free now that every P.V has retired, and touched by no other warp), then
            // the warp writes the 32 rows out with 8 (bf16) or 4 (e4m3) lanes per row.
            const float inv = (l_run == 0.f || l_run != l_run) ? 1.f : 1.f / l_run;
            const uint32_t stage = smem_base + L::kPOff + (uint32_t)(quarter * 32) * kAttnBN;   // + kPBytes: second half
            // both halves of the O row come in at once, into the registers the scores lived in
            __syncwarp();
            ptx::tmem_ld_32x32b_x32(t_lane + kAttnOCol, cur[0]);
            ptx::tmem_ld_32x32b_x32(t_lane + kAttnOCol + 32, cur[1]);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int h = 0; h < kAttnD / 32; ++h) {
                const uint32_t (&orow)[32] = cur[h];
                const uint32_t half = stage + (uint32_t)h * L::kPBytes;
                if (p.out_e4m3) {                                // 32 bytes per row and half: 2 pieces, swizzled by row bit 2
#pragma unroll
                    for (int v4 = 0; v4 < 2; ++v4) {
                        uint32_t w[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int j = v4 * 16 + q * 4;
                            w[q] = pack4_e4m3(__uint_as_float(orow[j]) * inv, __uint_as_float(orow[j + 1]) * inv,
                                              __uint_as_float(orow[j + 2]) * inv, __uint_as_float(orow[j + 3]) * inv);
                        }
                        st_shared_v4(half + (uint32_t)lane * 32u + ((((uint32_t)v4) ^ (((uint32_t)lane >> 2) & 1u)) << 4),
                                     w[0], w[1], w[2], w[3]);
                    }
                } else {                                         // 64 bytes per row and half: 4 pieces, swizzled by row bits 1..2
#pragma unroll
                    for (int v4 = 0; v4 < 4; ++v4) {
                        uint32_t w[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int j = v4 * 8 + q * 2;
                            __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(orow[j]) * inv,
                                                                      __uint_as_float(orow[j + 1]) * inv);
                            w[q] = *reinterpret_cast<uint32_t*>(&b2);
                        }
                        st_shared_v4(half + (uint32_t)lane * 64u + ((((uint32_t)v4) ^ (((uint32_t)lane >> 1) & 3u)) << 4),
                                     w[0], w[1], w[2], w[3]);
                    }
                }
            }
            const int row_w0 = row - lane;                       // first row of this warp
            if (p.tma_out) {
                // one destination: the two staged boxes (32 rows x 32 columns each) go out as TMA stores, which
                // run while the warp is already at its next tile; rows beyond M are clipped by the map
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0 && row_w0 < p.M) {
                    const int head = bh - b * p.H;
                    const int c1 = p.tma_out == 2 ? row_w0 : head, c2 = p.tma_out == 2 ? head : row_w0;
                    const int xb = p.out_e4m3 ? 32 : 64;        // bytes per row of one box
                    ptx::tma_store_4d(&tmap_o, stage, 0, c1, c2, b);
                    ptx::tma_store_4d(&tmap_o, stage + L::kPBytes, xb, c1, c2, b);
                    ptx::bulk_commit_group();
                }
                continue;
            }
            __syncwarp();
            const int64_t head_off = (int64_t)b * p.out_stride_b + (int64_t)(bh - b * p.H) * p.out_stride_h;
            if (p.out_e4m3) {
                const int pc = lane & 3;                          // 16-byte piece of the 64-byte row
                const uint32_t src = stage + (uint32_t)(pc >> 1) * L::kPBytes;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int rr = (lane >> 2) + 8 * k;
                    uint4 val;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                                 : "r"(src + (uint32_t)rr * 32u + ((((uint32_t)pc & 1u) ^ (((uint32_t)rr >> 2) & 1u)) << 4))
                                 : "memory");
                    if (row_w0 + rr < p.M) {
                        const int64_t off = head_off + (int64_t)(row_w0 + rr) * p.out_stride_s + pc * 16;
                        for (int dst = 0; dst < p.n_out; ++dst)
                            *reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(p.outs[dst]) + off) = val;
                    }
                }
            } else {
                const int pc = lane & 7;                          // 16-byte piece of the 128-byte row
                const uint32_t src = stage + (uint32_t)(pc >> 2) * L::kPBytes;
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int rr = (lane >> 3) + 4 * k;
                    uint4 val;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(val.x), "=r"(val.y), "=r"(val.z), "=r"(val.w)
                                 : "r"(src + (uint32_t)rr * 64u + ((((uint32_t)pc & 3u) ^ (((uint32_t)rr >> 1) & 3u)) << 4))
                                 : "memory");
                    if (row_w0 + rr < p.M) {
                        const int64_t off = head_off + (int64_t)(row_w0 + rr) * p.out_stride_s + pc * 8;
                        for (int dst = 0; dst < p.n_out; ++dst)
                            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.outs[dst]) + off) = val;
                    }
                }
            }
            __syncwarp();                                       // the rows are read out before the next tile's P overwrites them
            if (p.n_out > 1) __threadfence_system();
        }
        }   // query tiles of this CTA
        if (p.tma_out && lane == 0) ptx::bulk_wait_group<0>();  // this warp's stores are performed before the CTA may exit
        teardown_barrier();
    }
    // an abandoned wait anywhere in the CTA is reported through the status word
    if (threadIdx.x == 0 && *abort_flag != 0 && p.status != nullptr)
        atomicExch(p.status, Q8K_STATUS_TIMEOUT | (*abort_flag << 8));
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
    if (row_ok) *reinterpret_cast<uint2*>(out + (((int64_t)b * H + h) * S + s) * 64 + sub * 8) = pack8_e4m3_c10(v);
}

// Q / K after their projection, fused: RMS norm over all H*64 channels with an fp32 weight (bf16
// result), optional rotary embedding with shared fp32 tables [S, H*64] (bf16 result), then per head
// the 64-point Hadamard times `scale` and the c10 e4m3 cast, written head-major [B,H,S,64].  One
// CTA per token row, 8 elements per thread (thread t owns channels 8t..8t+7, head t/8).  The
// roundings are those of the separate kernels (rms_norm_kernel, rope_kernel, attn_prep_qk_kernel);
// only the summation order of the mean square differs from rms_norm_kernel.
// MODE 0: one row per CTA.  MODE 1 (x2 / norm_w2 / out2: K next to Q, same shape and row stride): the CTA
// handles the Q row and the K row of its token, so the rotary table row is loaded once for both and the
// two chains interleave.  MODE 0 and 1 with x3 / out3 also cast the token's V row to e4m3 (no norm, no
// rotation), written head-major like the others.  MODE 2 (no rotary tables, an even number of rows): the CTA handles
// two consecutive rows of x for the same interleaving.
template <int MODE>
__global__ void __launch_bounds__(1024)
attn_qk_norm_rope_prep_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ x2,
                              const __nv_bfloat16* __restrict__ x3, int64_t x_row_stride,
                              const float* __restrict__ norm_w, const float* __restrict__ norm_w2,
                              const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                              uint8_t* __restrict__ out, uint8_t* __restrict__ out2, uint8_t* __restrict__ out3,
                              int H, int S, int apply_hadamard, float scale) {
    constexpr bool PAIR = MODE == 1;
    constexpr int NX = MODE == 0 ? 1 : 2;
    __shared__ float red[NX][32];
    const int t = threadIdx.x;
    const int lane = t & 31;
    const int dim = H * 64;
    const int64_t row = MODE == 2 ? (int64_t)blockIdx.x * 2 : (int64_t)blockIdx.x;   // b * S + s
    const int s_idx = (int)(row % S);
    const int64_t b = row / S;
    if (MODE == 2) { x2 = x + x_row_stride; norm_w2 = norm_w; }
    float v[NX][8];
    load_vec<__nv_bfloat16, 8>(x + row * x_row_stride + t * 8, v[0]);
    if (NX == 2) load_vec<__nv_bfloat16, 8>(x2 + row * x_row_stride + t * 8, v[NX - 1]);
    float v3[8];
    if (MODE != 2 && x3 != nullptr) load_vec<__nv_bfloat16, 8>(x3 + row * x_row_stride + t * 8, v3);
    // the weights and rotary rows do not depend on the reduction: fetch them under its latency; the
    // rotary row is the same for Q and K
    float wv[NX][8], c[8], sn[8];
    load_vec<float, 8>(norm_w + t * 8, wv[0]);
    if (NX == 2) load_vec<float, 8>(norm_w2 + t * 8, wv[NX - 1]);
    if (cos_t != nullptr) {
        load_vec<float, 8>(cos_t + (int64_t)s_idx * dim + t * 8, c);
        load_vec<float, 8>(sin_t + (int64_t)s_idx * dim + t * 8, sn);
    }

#pragma unroll
    for (int w = 0; w < NX; ++w) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) ss = fmaf(v[w][j], v[w][j], ss);
        ss = warp_sum(ss);
        if (lane == 0) red[w][t >> 5] = ss;
    }
    __syncthreads();

    const int h = t >> 3, sub = t & 7;
    if (MODE != 2 && x3 != nullptr)
        *reinterpret_cast<uint2*>(out3 + ((b * H + h) * S + s_idx) * 64 + sub * 8) = pack8_e4m3_c10(v3);
#pragma unroll
    for (int w = 0; w < NX; ++w) {
        float tot = red[w][0];
        for (int i = 1; i < (int)(blockDim.x >> 5); ++i) tot += red[w][i];
        const float r = rsqrtf(tot * (1.0f / (float)dim));
        float (&u)[8] = v[w];
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
            u[j] = __fmul_rn(__fmul_rn(u[j], r), wv[w][j]);
            u[j + 1] = __fmul_rn(__fmul_rn(u[j + 1], r), wv[w][j + 1]);
            round_through_bf16x2(u[j], u[j + 1]);
        }

        if (cos_t != nullptr) {
            float o[8];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                o[j]     = __fadd_rn(__fmul_rn(-u[j + 1], sn[j]), __fmul_rn(u[j], c[j]));
                o[j + 1] = __fadd_rn(__fmul_rn(u[j], sn[j + 1]), __fmul_rn(u[j + 1], c[j + 1]));
            }
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                u[j] = o[j];
                u[j + 1] = o[j + 1];
                round_through_bf16x2(u[j], u[j + 1]);
            }
        }

        if (apply_hadamard) {
#pragma unroll
            for (int st = 1; st < 8; st <<= 1) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int lo = j & (st - 1);
                    const int i = ((j - lo) << 1) + lo;
                    const float a = u[i], bb = u[i + st];
                    u[i] = __fadd_rn(a, bb);
                    u[i + st] = __fsub_rn(a, bb);
                }
            }
#pragma unroll
            for (int mk = 1; mk < 8; mk <<= 1) {
                const float sign = (lane & mk) ? -1.f : 1.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float other = __shfl_xor_sync(0xffffffffu, u[j], mk);
                    u[j] = __fmaf_rn(sign, u[j], other);       // other - u for the upper lane, u + other for the lower: exact
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) u[j] = __fmul_rn(u[j], scale);
        }
        if (MODE == 2) {                                        // second row: the next token (possibly of the next batch entry)
            const int64_t rw = row + w;
            *reinterpret_cast<uint2*>(out + (((rw / S) * H + h) * S + (rw % S)) * 64 + sub * 8) = pack8_e4m3_c10(u);
        } else {
            uint8_t* dst = w == 0 ? out : out2;
            *reinterpret_cast<uint2*>(dst + ((b * H + h) * S + s_idx) * 64 + sub * 8) = pack8_e4m3_c10(u);
        }
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

// Exercises the bounded wait and the status word without touching any tensor: one warp waits on
// an mbarrier that nothing ever arrives on, with a limit of `tries` tests.
__global__ void wait_selftest_kernel(int* status, uint32_t tries) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t abort_word;
    const uint32_t bar_addr = ptx::smem_u32(&bar);
    const uint32_t abort_addr = ptx::smem_u32(&abort_word);
    if (threadIdx.x == 0) {
        ptx::mbar_init(bar_addr, 1);
        abort_word = 0;
        ptx::fence_barrier_init();
    }
    __syncthreads();
    ptx::mbar_wait_bounded(bar_addr, 0, abort_addr, 9, tries);
    __syncthreads();
    if (threadIdx.x == 0 && abort_word != 0 && status != nullptr)
        atomicExch(status, (int)(Q8K_STATUS_TIMEOUT | (abort_word << 8)));
}

}  // namespace q8k

using namespace q8k;

extern "C" int q8k_flash_attention(const void* q, const void* k, const void* vt, void* out, int out_dtype,
                                   int B, int H, int M, int N, float softmax_scale, const int* key_lens,
                                   int* dev_status, void* stream) {
    return q8k_flash_attention_strided(q, k, vt, out, out_dtype, B, H, M, N, (int64_t)H * M * 64, (int64_t)M * 64, 64,
                                       softmax_scale, key_lens, dev_status, stream);
}

extern "C" int q8k_flash_attention_strided(const void* q, const void* k, const void* vt, void* out, int out_dtype,
                                           int B, int H, int M, int N, int64_t out_stride_b, int64_t out_stride_h,
                                           int64_t out_stride_s, float softmax_scale, const int* key_lens,
                                           int* dev_status, void* stream) {
    void* outs[1] = {out};
    return q8k_flash_attention_multi_out(q, k, vt, outs, 1, out_dtype, B, H, M, N, out_stride_b, out_stride_h,
                                         out_stride_s, softmax_scale, key_lens, dev_status, stream);
}

static int launch_flash_attention(bool v_rows, const void* q, const void* k, const void* vt, void* const* outs, int n_out,
                                  int out_dtype, int B, int H, int M, int N, int64_t out_stride_b,
                                  int64_t out_stride_h, int64_t out_stride_s, float softmax_scale,
                                  const int* key_lens, int* dev_status, void* stream);

extern "C" int q8k_flash_attention_multi_out(const void* q, const void* k, const void* vt, void* const* outs, int n_out,
                                             int out_dtype, int B, int H, int M, int N, int64_t out_stride_b,
                                             int64_t out_stride_h, int64_t out_stride_s, float softmax_scale,
                                             const int* key_lens, int* dev_status, void* stream) {
    return launch_flash_attention(false, q, k, vt, outs, n_out, out_dtype, B, H, M, N, out_stride_b, out_stride_h,
                                  out_stride_s, softmax_scale, key_lens, dev_status, stream);
}

extern "C" int q8k_flash_attention_v_rows(const void* q, const void* k, const void* v, void* const* outs, int n_out,
                                          int out_dtype, int B, int H, int M, int N, int64_t out_stride_b,
                                          int64_t out_stride_h, int64_t out_stride_s, float softmax_scale,
                                          const int* key_lens, int* dev_status, void* stream) {
    return launch_flash_attention(true, q, k, v, outs, n_out, out_dtype, B, H, M, N, out_stride_b, out_stride_h,
                                  out_stride_s, softmax_scale, key_lens, dev_status, stream);
}

static int launch_flash_attention(bool v_rows, const void* q, const void* k, const void* vt, void* const* outs, int n_out,
                                  int out_dtype, int B, int H, int M, int N, int64_t out_stride_b,
                                  int64_t out_stride_h, int64_t out_stride_s, float softmax_scale,
                                  const int* key_lens, int* dev_status, void* stream) {
    const char* op = "flash_attention";
    Q8K_REQUIRE(outs != nullptr && n_out >= 1 && n_out <= kAttnMaxOut, Q8K_ERR_INVALID_ARG,
                "%s: between 1 and %d output destinations", op, kAttnMaxOut);
    for (int i = 0; i < n_out; ++i)
        Q8K_REQUIRE(outs[i] != nullptr && aligned16(outs[i]), Q8K_ERR_INVALID_ARG,
                    "%s: output destination %d is null or not 16-byte aligned", op, i);
    void* out = outs[0];
    Q8K_REQUIRE(q && k && vt && out, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE(B > 0 && H > 0 && M >= 0 && N > 0, Q8K_ERR_INVALID_ARG, "%s: bad shape B=%d H=%d M=%d N=%d", op, B, H, M, N);
    Q8K_REQUIRE(aligned16(q) && aligned16(k) && aligned16(vt) && aligned16(out), Q8K_ERR_INVALID_ARG,
                "%s: q, k, vt and out must be 16-byte aligned", op);
    Q8K_REQUIRE(out_dtype == Q8K_DT_E4M3 || out_dtype == Q8K_DT_BF16, Q8K_ERR_UNSUPPORTED,
                "%s: output dtype %d is not e4m3 or bf16", op, out_dtype);
    Q8K_REQUIRE((int64_t)B * H <= 65535, Q8K_ERR_TOO_LARGE, "%s: B*H = %lld exceeds 65535", op, (long long)B * H);
    Q8K_REQUIRE(out_stride_b % 16 == 0 && out_stride_h % 16 == 0 && out_stride_s % 16 == 0 && out_stride_s >= 64,
                Q8K_ERR_INVALID_ARG, "%s: output strides must be multiples of 16 elements", op);
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
    if (v_rows) {                                              // V [B,H,N,64]: the same boxes as K
        const uint64_t dims[3] = {64, (uint64_t)N, BH};
        const uint64_t strides[2] = {64, (uint64_t)N * 64};
        const uint32_t box[3] = {64, (uint32_t)kAttnBN, 1};
        if (int rc = make_byte_tensor_map(&tv, vt, 3, dims, strides, box, 64, op)) return rc;
    } else {                                                   // V^T [B,H,64,ceil16(N)]
        const uint64_t dims[3] = {(uint64_t)n_pad, 64, BH};
        const uint64_t strides[2] = {(uint64_t)n_pad, (uint64_t)n_pad * 64};
        const uint32_t box[3] = {(uint32_t)kAttnBN, 64, 1};
        if (int rc = make_byte_tensor_map(&tv, vt, 3, dims, strides, box, 64, op)) return rc;
    }

    AttnParams p;
    for (int i = 0; i < kAttnMaxOut; ++i) p.outs[i] = i < n_out ? outs[i] : nullptr;
    p.n_out = n_out;
    p.key_lens = key_lens;
    p.status = dev_status;
    p.B = B; p.H = H; p.M = M; p.N = N;
    p.scale_log2 = (float)((double)softmax_scale * 1.4426950408889634);
    p.out_e4m3 = out_dtype == Q8K_DT_E4M3;
    p.out_stride_b = out_stride_b; p.out_stride_h = out_stride_h; p.out_stride_s = out_stride_s;

    // One destination: the epilogue stores through a 4-D map of the output (bytes of a head row; rows and
    // heads in the order of their strides; batch), 32-row boxes of half a head row, swizzled like the staging.
    CUtensorMap to = tq;
    p.tma_out = 0;
    if (n_out == 1) {
        const uint64_t esz = p.out_e4m3 ? 1 : 2;
        const bool rows_first = out_stride_s <= out_stride_h;
        const uint64_t s_lo = (uint64_t)(rows_first ? out_stride_s : out_stride_h) * esz;
        const uint64_t s_hi = (uint64_t)(rows_first ? out_stride_h : out_stride_s) * esz;
        const uint64_t s_b = (uint64_t)out_stride_b * esz;
        const bool nested = s_lo >= 64 * esz && s_hi % s_lo == 0 && (B == 1 || (s_b >= s_hi && s_b % s_hi == 0));
        if (nested) {
            const uint64_t dims[4] = {64 * esz, (uint64_t)(rows_first ? M : H), (uint64_t)(rows_first ? H : M), (uint64_t)B};
            const uint64_t strides[3] = {s_lo, s_hi, B == 1 ? s_hi * dims[2] : s_b};
            const uint32_t box[4] = {(uint32_t)(32 * esz), rows_first ? 32u : 1u, rows_first ? 1u : 32u, 1u};
            if (int rc = make_byte_tensor_map(&to, out, 4, dims, strides, box, (int)(32 * esz), op)) return rc;
            p.tma_out = rows_first ? 2 : 1;
        }
    }

    // The warpgroups re-budget registers with setmaxnreg; an increase blocks until the CTA's pool
    // has room, so the pool the kernel was compiled for must cover the three budgets.
    static_assert(2 * kAttnRegsLaunch == kAttnRegsIo + kAttnRegsSoftmax, "register budgets");
    // Short key sequences (all of K and V fit the ring): a CTA walks over several query tiles of its
    // (batch, head); as many CTAs per (batch, head) as fill the device once at three CTAs per SM.
    const int q_tiles = (M + kAttnBM - 1) / kAttnBM;
    const bool multi = (N + kAttnBN - 1) / kAttnBN <= kAttnKS && q_tiles > 1;
    int ctas_per_bh = q_tiles;
    if (multi) {
        static int num_sms = 0;
        if (num_sms == 0) {
            int dev = 0, n = 0;
            Q8K_CUDA_OK(cudaGetDevice(&dev));
            Q8K_CUDA_OK(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
            num_sms = n;
        }
        int g_max = (int)((uint64_t)(3 * num_sms) / BH);
        g_max = g_max < 1 ? 1 : (g_max > q_tiles ? q_tiles : g_max);
        const int tiles_per_cta = (q_tiles + g_max - 1) / g_max;
        ctas_per_bh = (q_tiles + tiles_per_cta - 1) / tiles_per_cta;
    }
    auto kern = v_rows ? (multi ? flash_attn_fp8_kernel<true, true> : flash_attn_fp8_kernel<true, false>)
                       : (multi ? flash_attn_fp8_kernel<false, true> : flash_attn_fp8_kernel<false, false>);
    cudaFuncAttributes fattr;
    Q8K_CUDA_OK(cudaFuncGetAttributes(&fattr, kern));
    Q8K_REQUIRE(fattr.numRegs >= kAttnRegsLaunch, Q8K_ERR_CUDA,
                "%s: kernel was built with %d registers per thread, %d needed for the warpgroup budgets", op,
                fattr.numRegs, kAttnRegsLaunch);
    Q8K_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem::kDynamic));
    dim3 grid((unsigned)ctas_per_bh, (unsigned)BH);
    kern<<<grid, kAttnThreads, AttnSmem::kDynamic, (cudaStream_t)stream>>>(tq, tk, tv, to, p);
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

extern "C" int q8k_attention_cast_rows(const void* x, void* out8, int B, int H, int S, int64_t stride_b, int64_t stride_s,
                                       int64_t stride_h, void* stream) {
    const char* op = "attention_cast_rows";
    Q8K_REQUIRE(x && out8, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE(B > 0 && H > 0 && S > 0, Q8K_ERR_INVALID_ARG, "%s: bad shape", op);
    Q8K_REQUIRE(stride_b % 8 == 0 && stride_s % 8 == 0 && stride_h % 8 == 0 && aligned16(x) && aligned16(out8),
                Q8K_ERR_INVALID_ARG, "%s: strides must be multiples of 8 elements and pointers 16-byte aligned", op);
    const int64_t rows = (int64_t)B * S * H;
    Q8K_REQUIRE((rows + 15) / 16 <= 0x7fffffffLL, Q8K_ERR_TOO_LARGE, "%s: too many rows", op);
    attn_prep_qk_kernel<<<(unsigned)((rows + 15) / 16), 128, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (uint8_t*)out8, B, H, S, stride_b, stride_s, stride_h, 0, 1.0f);
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

extern "C" int q8k_qk_norm_rope_prep(const void* x, int64_t x_row_stride, const float* norm_w, const float* cos_t,
                                     const float* sin_t, void* out8, int B, int S, int H, int apply_hadamard,
                                     float qk_scale, void* stream) {
    const char* op = "qk_norm_rope_prep";
    Q8K_REQUIRE(x && norm_w && out8, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), Q8K_ERR_INVALID_ARG, "%s: give both rotary tables or neither", op);
    Q8K_REQUIRE(B > 0 && S > 0 && H > 0 && H <= 128, Q8K_ERR_INVALID_ARG, "%s: bad shape B=%d S=%d H=%d (H <= 128)", op, B, S, H);
    Q8K_REQUIRE(H % 4 == 0, Q8K_ERR_UNSUPPORTED, "%s: H must be a multiple of 4", op);
    Q8K_REQUIRE(x_row_stride >= (int64_t)H * 64 && x_row_stride % 8 == 0, Q8K_ERR_INVALID_ARG,
                "%s: row stride must be >= H*64 and a multiple of 8 elements", op);
    Q8K_REQUIRE(aligned16(x) && aligned16(norm_w) && aligned16(cos_t) && aligned16(sin_t) && aligned16(out8),
                Q8K_ERR_INVALID_ARG, "%s: pointers must be 16-byte aligned", op);
    Q8K_REQUIRE((int64_t)B * S <= 0x7fffffffLL, Q8K_ERR_TOO_LARGE, "%s: too many rows", op);
    if (cos_t == nullptr && ((int64_t)B * S) % 2 == 0)
        attn_qk_norm_rope_prep_kernel<2><<<(unsigned)((int64_t)B * S / 2), H * 8, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)x, nullptr, nullptr, x_row_stride, norm_w, nullptr, nullptr, nullptr, (uint8_t*)out8,
            nullptr, nullptr, H, S, apply_hadamard, qk_scale);
    else
        attn_qk_norm_rope_prep_kernel<0><<<(unsigned)((int64_t)B * S), H * 8, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)x, nullptr, nullptr, x_row_stride, norm_w, nullptr, cos_t, sin_t, (uint8_t*)out8,
            nullptr, nullptr, H, S, apply_hadamard, qk_scale);
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

static int launch_qkv_prep(const char* op, const void* xq, const void* xk, const void* xv, int64_t x_row_stride,
                           const float* norm_wq, const float* norm_wk, const float* cos_t, const float* sin_t,
                           void* outq8, void* outk8, void* outv8, int B, int S, int H, int apply_hadamard,
                           float qk_scale, void* stream) {
    Q8K_REQUIRE(xk && norm_wk && outk8, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE((xq == nullptr) == (outq8 == nullptr) && (xq == nullptr) == (norm_wq == nullptr), Q8K_ERR_INVALID_ARG,
                "%s: give q, its norm weight and its output, or none of them", op);
    Q8K_REQUIRE((xv == nullptr) == (outv8 == nullptr), Q8K_ERR_INVALID_ARG, "%s: give both v and its output or neither", op);
    Q8K_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), Q8K_ERR_INVALID_ARG, "%s: give both rotary tables or neither", op);
    Q8K_REQUIRE(B > 0 && S > 0 && H > 0 && H <= 128, Q8K_ERR_INVALID_ARG, "%s: bad shape B=%d S=%d H=%d (H <= 128)", op, B, S, H);
    Q8K_REQUIRE(H % 4 == 0, Q8K_ERR_UNSUPPORTED, "%s: H must be a multiple of 4", op);
    Q8K_REQUIRE(x_row_stride >= (int64_t)H * 64 && x_row_stride % 8 == 0, Q8K_ERR_INVALID_ARG,
                "%s: row stride must be >= H*64 and a multiple of 8 elements", op);
    Q8K_REQUIRE(aligned16(xq) && aligned16(xk) && aligned16(xv) && aligned16(norm_wq) && aligned16(norm_wk) &&
                    aligned16(cos_t) && aligned16(sin_t) && aligned16(outq8) && aligned16(outk8) && aligned16(outv8),
                Q8K_ERR_INVALID_ARG, "%s: pointers must be 16-byte aligned", op);
    Q8K_REQUIRE((int64_t)B * S <= 0x7fffffffLL, Q8K_ERR_TOO_LARGE, "%s: too many rows", op);
    if (xq != nullptr)
        attn_qk_norm_rope_prep_kernel<1><<<(unsigned)((int64_t)B * S), H * 8, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)xq, (const __nv_bfloat16*)xk, (const __nv_bfloat16*)xv, x_row_stride, norm_wq, norm_wk, cos_t,
            sin_t, (uint8_t*)outq8, (uint8_t*)outk8, (uint8_t*)outv8, H, S, apply_hadamard, qk_scale);
    else                                                       // K and V only (cross-attention: Q comes from another tensor)
        attn_qk_norm_rope_prep_kernel<0><<<(unsigned)((int64_t)B * S), H * 8, 0, (cudaStream_t)stream>>>(
            (const __nv_bfloat16*)xk, nullptr, (const __nv_bfloat16*)xv, x_row_stride, norm_wk, nullptr, cos_t, sin_t,
            (uint8_t*)outk8, nullptr, (uint8_t*)outv8, H, S, apply_hadamard, qk_scale);
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

extern "C" int q8k_qk_norm_rope_prep_pair(const void* xq, const void* xk, int64_t x_row_stride, const float* norm_wq,
                                          const float* norm_wk, const float* cos_t, const float* sin_t, void* outq8,
                                          void* outk8, int B, int S, int H, int apply_hadamard, float qk_scale,
                                          void* stream) {
    Q8K_REQUIRE(xq != nullptr, Q8K_ERR_INVALID_ARG, "qk_norm_rope_prep_pair: null pointer");
    return launch_qkv_prep("qk_norm_rope_prep_pair", xq, xk, nullptr, x_row_stride, norm_wq, norm_wk, cos_t, sin_t, outq8,
                           outk8, nullptr, B, S, H, apply_hadamard, qk_scale, stream);
}

extern "C" int q8k_qkv_prep(const void* xq, const void* xk, const void* xv, int64_t x_row_stride, const float* norm_wq,
                            const float* norm_wk, const float* cos_t, const float* sin_t, void* outq8, void* outk8,
                            void* outv8, int B, int S, int H, int apply_hadamard, float qk_scale, void* stream) {
    Q8K_REQUIRE(xv != nullptr && outv8 != nullptr, Q8K_ERR_INVALID_ARG, "qkv_prep: null pointer");
    return launch_qkv_prep("qkv_prep", xq, xk, xv, x_row_stride, norm_wq, norm_wk, cos_t, sin_t, outq8, outk8, outv8, B, S,
                           H, apply_hadamard, qk_scale, stream);
}

extern "C" int q8k_attention_prep_v(const void* v, void* vt8, int B, int H, int S_kv, int64_t v_stride_b,
                                    int64_t v_stride_s, int64_t v_stride_h, void* stream) {
    const char* op = "attention_prep_v";
    Q8K_REQUIRE(v && vt8, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE(B > 0 && H > 0 && S_kv > 0 && (int64_t)B * H <= 65535, Q8K_ERR_INVALID_ARG, "%s: bad shape", op);
    Q8K_REQUIRE(v_stride_b % 8 == 0 && v_stride_s % 8 == 0 && v_stride_h % 8 == 0 && aligned16(v) && aligned16(vt8),
                Q8K_ERR_INVALID_ARG, "%s: strides must be multiples of 8 elements and pointers 16-byte aligned", op);
    const int s_pad = (S_kv + 15) / 16 * 16;
    dim3 grid((unsigned)((S_kv + 63) / 64), (unsigned)(B * H));
    attn_prep_v_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)v, (uint8_t*)vt8, H, S_kv, s_pad,
                                                              v_stride_b, v_stride_s, v_stride_h);
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

extern "C" int q8k_wait_selftest(int* dev_status, unsigned tries, void* stream) {
    const char* op = "wait_selftest";
    Q8K_REQUIRE(dev_status != nullptr, Q8K_ERR_INVALID_ARG, "%s: null status word", op);
    Q8K_REQUIRE(tries >= 1 && tries <= (1u << 16), Q8K_ERR_INVALID_ARG, "%s: tries must be in [1, 65536]", op);
    wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(dev_status, tries);
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}
