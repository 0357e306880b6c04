// CTA-pair variant of the 8-bit GEMM: a cluster of two CTAs on neighbouring SMs owns a 256 x 256
// output tile and runs ONE tcgen05.mma (cta_group::2, M = 256, N = 256, K = 32) per K slice.
//
// Why: in the single-CTA kernel every MMA streams a 128-row A slab and a 256-row B slab out of the
// CTA's shared memory, and TMA writes the same 48 KB per stage into it; shared memory bandwidth is
// what caps the main loop.  In a pair each CTA holds its own 128 rows of A and only HALF of the B
// rows (128 of 256), so both the TMA fill and the tensor-core reads per CTA drop by a third while
// the pair produces twice the output.
//
// Roles per CTA (10 warps, same as the single-CTA kernel):
//   warp 0     TMA producer: its A rows and its half of the B rows, 32 KB per stage, 6 stages; the
//              transaction bytes of BOTH CTAs are credited to the leader CTA's "full" barrier
//   warp 1     TMEM allocation (both CTAs); in the leader (even rank) one thread issues the MMAs
//              and commits to the "empty" / "accumulator full" barriers of both CTAs
//   warps 2-9  epilogue of the CTA's own 128 rows x 256 columns (identical arithmetic to the
//              single-CTA kernel); "accumulator free" arrivals of both CTAs go to the leader.
//              Output leaves through shared memory: each warp writes its 32 x 32 chunk into a
//              swizzled staging box and one lane hands it to a TMA store, so global memory sees
//              whole 32/64-byte row segments instead of 32 row-strided 16-byte stores per
//              instruction (which held the epilogue, and with it the K = 2048 shapes, back).
//              Outputs whose row pitch is not a multiple of 16 bytes keep the direct stores.
// No multicast loads are used: every CTA fetches its own operand tiles with plain TMA loads.

#include "gemm_common.cuh"

namespace q8k {

constexpr int kPairBN = 256;                 // tile columns (128 B rows from each CTA)
constexpr int kPairTmemCols = 512;           // two 256-column accumulators per CTA

// Shared memory of one CTA.  The gate/residual variant gives one of the six pipeline stages to residual
// staging: per epilogue warp two 32-row boxes that TMA fills one and two chunks ahead of their use.
template <bool RESID>
struct PairSmemT {
    static constexpr int kStages = RESID ? 5 : 6;
    static constexpr int kABytes = kGemmBM * kGemmBK;              // 16 KB: this CTA's 128 rows of A
    static constexpr int kBBytes = (kPairBN / 2) * kGemmBK;        // 16 KB: this CTA's 128 rows of B
    static constexpr int kStageBytes = kABytes + kBBytes;
    // output staging: per epilogue warp two 32-row boxes of 64 bytes per row (bf16) or 32 (e4m3)
    static constexpr int kStoreBoxBytes = 32 * 64;
    static constexpr int kStoreOffset = kStages * kStageBytes;
    static constexpr int kStoreBytes = (kGemmEpilogueThreads / 32) * 2 * kStoreBoxBytes;
    // residual staging (bf16 rows of 64 bytes), same box shape and swizzle as the output boxes
    static constexpr int kResidOffset = kStoreOffset + kStoreBytes;
    static constexpr int kResidBytes = RESID ? (kGemmEpilogueThreads / 32) * 2 * kStoreBoxBytes : 0;
    static constexpr int kBarOffset = kResidOffset + kResidBytes;
    static constexpr int kNumResidBars = RESID ? (kGemmEpilogueThreads / 32) * 2 : 0;
    static constexpr int kNumBars = 2 * kStages + 4 + kNumResidBars;
    static constexpr int kTmemPtrOffset = kBarOffset + kNumBars * 8;
    static constexpr int kAbortOffset = kTmemPtrOffset + 4;
    static constexpr int kPriorOffset = kAbortOffset + 4;
    static constexpr int kColScaleOffset = (kPriorOffset + 4 + 15) & ~15;
    static constexpr int kBiasOffset = kColScaleOffset + kPairBN * 4;
    static constexpr int kGateOffset = kBiasOffset + kPairBN * 4;  // bf16 gate row of the tile (gate/residual epilogue)
    static constexpr int kTotal = kGateOffset + kPairBN * 2;
    // No alignment slack: the kernel has no static shared memory, so the dynamic window starts on
    // a 1024-byte boundary; the kernel checks that and reports instead of running misaligned.
    static constexpr int kDynamic = kTotal;
    static_assert(kDynamic <= 227 * 1024, "pair GEMM shared memory");
};

struct PairParams {
    GemmParams g;
    int m_tiles2;                            // 256-row tiles per batch entry
    int n_tiles2;
    int total_tiles2;
    int tma_store;                           // 1: the epilogue stores through tmap_c
};

template <bool INT8, bool GELU, bool OUT_E4M3, bool RESID>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_8bit_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_r,
                      const PairParams pp) {
    using L = PairSmemT<RESID>;
    constexpr int kPairStages = L::kStages;
    const GemmParams& p = pp.g;
    constexpr uint32_t IDESC = INT8 ? ptx::make_idesc_s8(2 * kGemmBM, kPairBN) : ptx::make_idesc_e4m3(2 * kGemmBM, kPairBN);

    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t smem_base = ptx::smem_u32(smem);
    if (smem_base & 1023u) {                                   // same offset in both CTAs: both leave
        if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, Q8K_STATUS_TIMEOUT | (11 << 8));
        return;
    }
    const uint32_t bar_base = smem_base + L::kBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kPairStages + s); };
    auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kPairStages + a); };
    auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kPairStages + 2 + a); };
    auto resid_bar = [&](int w, int i) { return bar_base + 8u * (2 * kPairStages + 4 + 2 * w + i); };   // RESID only
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOffset);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOffset);
    float* col_scale_smem = reinterpret_cast<float*>(smem + L::kColScaleOffset);
    float* bias_smem = reinterpret_cast<float*>(smem + L::kBiasOffset);
    __nv_bfloat16* gate_smem = reinterpret_cast<__nv_bfloat16*>(smem + L::kGateOffset);

    const uint32_t rank = ptx::cluster_ctarank();              // 0 = leader, 1 = peer
    const bool leader = rank == 0;
    const int cluster_id = blockIdx.x >> 1;
    const int num_clusters = gridDim.x >> 1;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int k_iters = (p.K + kGemmBK - 1) / kGemmBK;

    // A launch that follows a failed one on the same status word does nothing.  The leader reads
    // the word and hands its decision to the peer, so the two CTAs of a pair always agree.
    volatile int* prior_failure = reinterpret_cast<volatile int*>(smem + L::kPriorOffset);
    if (threadIdx.x == 0 && leader) {
        const int v = p.status != nullptr ? *reinterpret_cast<volatile int*>(p.status) : 0;
        *prior_failure = v;
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(ptx::mapa_shared(smem_base + L::kPriorOffset, 1)), "r"(v)
                     : "memory");
    }
    ptx::cluster_sync_all();
    const bool skip = *prior_failure != 0;
    if (skip) return;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kPairStages; ++s) {
            ptx::mbar_init(full_bar(s), 2);                    // one arrive.expect_tx from each CTA's producer
            ptx::mbar_init(empty_bar(s), 1);                   // one commit from the leader's MMA thread
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(tmem_full_bar(a), 1);
            ptx::mbar_init(tmem_empty_bar(a), 2 * (kGemmEpilogueThreads / 32));   // every epilogue warp of both CTAs
        }
        if constexpr (RESID) {
            for (int w = 0; w < kGemmEpilogueThreads / 32; ++w) {
                ptx::mbar_init(resid_bar(w, 0), 1);
                ptx::mbar_init(resid_bar(w, 1), 1);
            }
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        if (pp.tma_store) ptx::prefetch_tensormap(&tmap_c);
        if (RESID && pp.tma_store) ptx::prefetch_tensormap(&tmap_r);
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair<kPairTmemCols>(ptx::smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)));
        ptx::tmem_relinquish_alloc_permit_pair();
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync_all();                                   // both CTAs' barriers exist before anyone signals across
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;

    // barriers of the leader CTA, as seen from this CTA
    auto leader_full_bar = [&](int s) { return ptx::mapa_shared(full_bar(s), 0); };
    auto leader_tmem_empty_bar = [&](int a) { return ptx::mapa_shared(tmem_empty_bar(a), 0); };

    if (warp == 0) {
        // ------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = cluster_id; ok && tile < pp.total_tiles2; tile += num_clusters) {
                const int n_blk = tile % pp.n_tiles2;
                const int m_blk = (tile / pp.n_tiles2) % pp.m_tiles2;
                const int batch = tile / (pp.n_tiles2 * pp.m_tiles2);
                const int a_row = (p.batch_a ? batch * p.M : 0) + m_blk * 2 * kGemmBM + (int)rank * kGemmBM;
                const int b_row = (p.batch_b ? batch * p.N : 0) + n_blk * kPairBN + (int)rank * (kPairBN / 2);
                for (int kb = 0; kb < k_iters; ++kb, ++it) {
                    const int s = it % kPairStages;
                    const uint32_t ph = (it / kPairStages) & 1u;
                    if (!ptx::mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t fb = leader_full_bar(s);
                    ptx::mbar_arrive_expect_tx_cluster(fb, L::kStageBytes);
                    const uint32_t a_dst = smem_base + s * L::kStageBytes;
                    ptx::tma_load_2d_pair(a_dst, &tmap_a, fb, kb * kGemmBK, a_row);
                    ptx::tma_load_2d_pair(a_dst + L::kABytes, &tmap_b, fb, kb * kGemmBK, b_row);
                }
            }
            if (!ok && p.status != nullptr) atomicExch(p.status, Q8K_STATUS_TIMEOUT | (8 << 8));
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && leader) {
            uint32_t it = 0;
            uint32_t tile_i = 0;
            bool ok = true;
            for (int tile = cluster_id; ok && tile < pp.total_tiles2; tile += num_clusters, ++tile_i) {
                const uint32_t acc = tile_i & 1u;
                const uint32_t acc_ph = (tile_i >> 1) & 1u;
                if (!ptx::mbar_wait(tmem_empty_bar(acc), acc_ph ^ 1u, abort_flag)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * kPairBN;
                for (int kb = 0; kb < k_iters; ++kb, ++it) {
                    const int s = it % kPairStages;
                    const uint32_t ph = (it / kPairStages) & 1u;
                    if (!ptx::mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
                    ptx::tcgen05_fence_after_sync();
                    const uint32_t a_addr = smem_base + s * L::kStageBytes;
                    const uint64_t a_desc = ptx::make_kmajor_desc(a_addr, 128);
                    const uint64_t b_desc = ptx::make_kmajor_desc(a_addr + L::kABytes, 128);
#pragma unroll
                    for (int k = 0; k < kGemmBK / 32; ++k) {
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        if constexpr (INT8) ptx::mma_i8_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, accumulate);
                        else ptx::mma_f8f6f4_pair(d_tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, accumulate);
                    }
                    // the stage is reusable in BOTH CTAs once these MMAs retire
                    ptx::tcgen05_commit_pair(ptx::mapa_shared(empty_bar(s), 0));
                    ptx::tcgen05_commit_pair(ptx::mapa_shared(empty_bar(s), 1));
                }
                if (ok) {
                    ptx::tcgen05_commit_pair(ptx::mapa_shared(tmem_full_bar(acc), 0));
                    ptx::tcgen05_commit_pair(ptx::mapa_shared(tmem_full_bar(acc), 1));
                }
            }
            if (!ok && p.status != nullptr) atomicExch(p.status, Q8K_STATUS_TIMEOUT | (9 << 8));
        }
    } else {
        // ------------------------------------------------ epilogue (warps 2..9) of this CTA's 128 rows
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int epi_tid = threadIdx.x - 64;
        constexpr int HALF_COLS = kPairBN / 2;
        constexpr int NCH = HALF_COLS / 32;
        const bool staged = pp.tma_store != 0;
        const uint32_t store_base = smem_base + L::kStoreOffset + (uint32_t)(warp - 2) * 2u * L::kStoreBoxBytes;
        uint32_t tile_i = 0;
        uint32_t store_i = 0;                                  // stores issued by this warp: picks the staging box
        uint32_t resid_i = 0, resid_c = 0;                     // residual boxes requested (lane 0) / consumed by this warp
        const uint32_t resid_base = smem_base + L::kResidOffset + (uint32_t)(warp - 2) * 2u * L::kStoreBoxBytes;
        bool ok = true;
        for (int tile = cluster_id; tile < pp.total_tiles2; tile += num_clusters, ++tile_i) {
            const int n_blk = tile % pp.n_tiles2;
            const int m_blk = (tile / pp.n_tiles2) % pp.m_tiles2;
            const int batch = tile / (pp.n_tiles2 * pp.m_tiles2);
            const int n0 = n_blk * kPairBN;
            const uint32_t acc = tile_i & 1u;
            const uint32_t acc_ph = (tile_i >> 1) & 1u;

            // gate row of this CTA's first row: the whole tile's, unless the tile straddles two gate rows
            int64_t gate_row_tile = 0;
            if constexpr (RESID)
                gate_row_tile = (((int64_t)batch * p.M + m_blk * 2 * kGemmBM + (int)rank * kGemmBM) / p.rows_per_gate) * p.N;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            for (int c = epi_tid; c < kPairBN; c += kGemmEpilogueThreads) {
                const int n = n0 + c;
                const bool in = n < p.N;
                col_scale_smem[c] = in ? p.b_scales[(p.batch_b ? (int64_t)batch * p.N : 0) + n] : 0.f;
                bias_smem[c] = (in && p.bias != nullptr) ? p.bias[n] : 0.f;
                if constexpr (RESID) {
                    if (p.gate != nullptr) gate_smem[c] = in ? p.gate[gate_row_tile + n] : __float2bfloat16(0.f);
                }
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");

            const int row = m_blk * 2 * kGemmBM + (int)rank * kGemmBM + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            const float sa = row_ok ? p.a_scales[(p.batch_a ? (int64_t)batch * p.M : 0) + row] : 0.f;
            const int64_t out_row = ((int64_t)batch * p.M + row) * p.N;
            const int64_t gate_row = RESID ? (((int64_t)batch * p.M + row) / p.rows_per_gate) * p.N : 0;
            const int col_base = half * HALF_COLS;
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * kPairBN + col_base;

            // Residual of this warp's 32 rows, one 32-column chunk per box (staged bf16 path): TMA loads it
            // into the warp's two residual boxes, the first two chunks before the accumulator is even
            // complete and chunk c+2 as soon as chunk c has been read out, so that the latency of the
            // residual is not paid inside the chunk that uses it.
            auto issue_resid = [&](int c) {                     // lane 0; chunks with columns inside N only
                const int nc = n0 + col_base + c * 32;
                if (nc < p.N) {
                    const uint32_t rb = resid_bar(warp - 2, (int)(resid_i & 1u));
                    ptx::mbar_arrive_expect_tx(rb, L::kStoreBoxBytes);
                    ptx::tma_load_3d(resid_base + (resid_i & 1u) * L::kStoreBoxBytes, &tmap_r, rb, nc * 2,
                                     m_blk * 2 * kGemmBM + (int)rank * kGemmBM + quarter * 32, batch);
                    ++resid_i;
                }
            };
            if constexpr (RESID && !OUT_E4M3) {
                if (staged && lane == 0) {
                    issue_resid(0);
                    issue_resid(1);
                }
            }

            if (ok) ok = ptx::mbar_wait(tmem_full_bar(acc), acc_ph, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) continue;
            ptx::tcgen05_fence_after_sync();

            uint32_t r[2][32];
            __syncwarp();
            ptx::tmem_ld_32x32b_x32(t_row, r[0]);
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                ptx::tmem_wait_ld();
                if (c + 1 < NCH) ptx::tmem_ld_32x32b_x32(t_row + (c + 1) * 32, r[(c + 1) & 1]);
                const int cl = col_base + c * 32;
                const int nc = n0 + cl;
                uint32_t rs_cur[16];
                if constexpr (RESID && !OUT_E4M3) {
                    if (staged && nc < p.N) {                  // warp-uniform
                        // this thread's row of the residual box (same swizzle as the output box)
                        const uint32_t rbox = resid_base + (resid_c & 1u) * L::kStoreBoxBytes;
                        if (!ptx::mbar_wait(resid_bar(warp - 2, (int)(resid_c & 1u)), (resid_c >> 1) & 1u, abort_flag)) ok = false;
                        ++resid_c;
                        const uint32_t rrow = rbox + (uint32_t)lane * 64u;
                        const uint32_t rsw = ((uint32_t)lane >> 1) & 3u;
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                         : "=r"(rs_cur[4 * q]), "=r"(rs_cur[4 * q + 1]), "=r"(rs_cur[4 * q + 2]), "=r"(rs_cur[4 * q + 3])
                                         : "r"(rrow + (((uint32_t)q ^ rsw) << 4))
                                         : "memory");
                        __syncwarp();
                        if (lane == 0 && c + 2 < NCH) {
                            ptx::fence_proxy_async_smem();
                            issue_resid(c + 2);
                        }
                    }
                }
                if (staged) {
                    if (nc < p.N) {                            // warp-uniform
                        const uint32_t(&rc)[32] = r[c & 1];
                        constexpr int ROW_BYTES = OUT_E4M3 ? 32 : 64;
                        const uint32_t box = store_base + (store_i & 1u) * L::kStoreBoxBytes;
                        ++store_i;
                        // the store that last used this box (two stores ago) must have read it out
                        if (lane == 0) ptx::bulk_wait_group_read<1>();
                        __syncwarp();
                        // row `lane` of the box, 16-byte pieces XOR-swizzled as the tensor map expects
                        // (SWIZZLE_64B: piece ^= (row >> 1) & 3; SWIZZLE_32B: piece ^= (row >> 2) & 1)
                        const uint32_t row_addr = box + (uint32_t)lane * ROW_BYTES;
                        const uint32_t sw = OUT_E4M3 ? ((uint32_t)lane >> 2) & 1u : ((uint32_t)lane >> 1) & 3u;
                        const float2 sa2 = make_float2(sa, sa);
#pragma unroll
                        for (int q = 0; q < ROW_BYTES / 16; ++q) {
                            uint32_t w[4];
                            if constexpr (OUT_E4M3) {
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const int j = q * 16 + e * 4;
                                    const float2 y0 = epilogue_pair<INT8, GELU>(rc[j], rc[j + 1], sa2, col_scale_smem + cl + j,
                                                                                bias_smem + cl + j);
                                    const float2 y1 = epilogue_pair<INT8, GELU>(rc[j + 2], rc[j + 3], sa2,
                                                                                col_scale_smem + cl + j + 2, bias_smem + cl + j + 2);
                                    w[e] = (uint32_t)float2_to_e4m3x2_sat(y0.x, y0.y) |
                                           ((uint32_t)float2_to_e4m3x2_sat(y1.x, y1.y) << 16);
                                }
                            } else {
                                uint4 gt = make_uint4(0, 0, 0, 0);
                                if constexpr (RESID) {
                                    if (p.gate != nullptr) {
                                        if (gate_row == gate_row_tile) gt = *reinterpret_cast<const uint4*>(gate_smem + cl + q * 8);
                                        else if (row_ok && nc + q * 8 < p.N)
                                            gt = *reinterpret_cast<const uint4*>(p.gate + gate_row + nc + q * 8);
                                    }
                                }
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const int j = q * 8 + e * 2;
                                    const float2 y0 = epilogue_pair<INT8, GELU>(rc[j], rc[j + 1], sa2, col_scale_smem + cl + j,
                                                                                bias_smem + cl + j);
                                    __nv_bfloat162 b2 = __floats2bfloat162_rn(y0.x, y0.y);
                                    if constexpr (RESID) {
                                        // out = bf16(bf16(gate * bf16(y)) + resid), the roundings of the separate torch
                                        // ops.  Packed bf16 arithmetic gives exactly those: a product of two bf16 values
                                        // is exact in fp32, and a sum of two is either exact in fp32 or so lopsided that
                                        // both roundings return the larger operand; _rn keeps the two from fusing.
                                        if (p.gate != nullptr) {
                                            const uint32_t gw = e == 0 ? gt.x : (e == 1 ? gt.y : (e == 2 ? gt.z : gt.w));
                                            b2 = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&gw), b2);
                                        }
                                        const uint32_t rw = rs_cur[4 * q + e];
                                        b2 = __hadd2_rn(b2, *reinterpret_cast<const __nv_bfloat162*>(&rw));
                                    }
                                    w[e] = *reinterpret_cast<uint32_t*>(&b2);
                                }
                            }
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(row_addr + (((uint32_t)q ^ sw) << 4)),
                                         "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3])
                                         : "memory");
                        }
                        ptx::fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            ptx::tma_store_3d(&tmap_c, box, nc * (OUT_E4M3 ? 1 : 2),
                                              m_blk * 2 * kGemmBM + (int)rank * kGemmBM + quarter * 32, batch);
                            ptx::bulk_commit_group();
                        }
                    }
                } else if (row_ok && nc < p.N) {
                    const uint32_t(&rc)[32] = r[c & 1];
                    float y[32];
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float2 v = epilogue_pair<INT8, GELU>(rc[j], rc[j + 1], make_float2(sa, sa),
                                                                   col_scale_smem + cl + j, bias_smem + cl + j);
                        y[j] = v.x;
                        y[j + 1] = v.y;
                    }
                    const int valid = min(32, p.N - nc);
                    if constexpr (OUT_E4M3) {
                        uint8_t* o = reinterpret_cast<uint8_t*>(p.out) + out_row + nc;
#pragma unroll
                        for (int v4 = 0; v4 < 2; ++v4) {
                            if (v4 * 16 < valid) {
                                uint32_t w[4];
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    const int j = v4 * 16 + q * 4;
                                    w[q] = (uint32_t)float2_to_e4m3x2_sat(y[j], y[j + 1]) |
                                           ((uint32_t)float2_to_e4m3x2_sat(y[j + 2], y[j + 3]) << 16);
                                }
                                reinterpret_cast<uint4*>(o)[v4] = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        }
                    } else {
                        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.out) + out_row + nc;
#pragma unroll
                        for (int v4 = 0; v4 < 4; ++v4) {
                            if (v4 * 8 < valid) {
                                uint32_t w[4];
                                uint4 rs = make_uint4(0, 0, 0, 0), gt = make_uint4(0, 0, 0, 0);
                                if constexpr (RESID) {
                                    rs = *reinterpret_cast<const uint4*>(p.resid + out_row + nc + v4 * 8);
                                    if (p.gate != nullptr)
                                        gt = *reinterpret_cast<const uint4*>(p.gate + gate_row + nc + v4 * 8);
                                }
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    const int j = v4 * 8 + q * 2;
                                    __nv_bfloat162 b2 = __floats2bfloat162_rn(y[j], y[j + 1]);
                                    if constexpr (RESID) {
                                        // out = bf16(bf16(gate * bf16(y)) + resid): the roundings of the separate
                                        // torch ops of blocks/ltx_transformer_block.py (gate*x, then + residual)
                                        float2 f = __bfloat1622float2(b2);
                                        if (p.gate != nullptr) {
                                            const uint32_t gw = (&gt.x)[q];
                                            const float2 g = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw));
                                            f = __bfloat1622float2(__floats2bfloat162_rn(g.x * f.x, g.y * f.y));
                                        }
                                        const uint32_t rw = (&rs.x)[q];
                                        const float2 r2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rw));
                                        b2 = __floats2bfloat162_rn(f.x + r2.x, f.y + r2.y);
                                    }
                                    w[q] = *reinterpret_cast<uint32_t*>(&b2);
                                }
                                reinterpret_cast<uint4*>(o)[v4] = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        }
                    }
                }
                __syncwarp();
            }
            ptx::tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(leader_tmem_empty_bar(acc));   // the leader's MMA thread waits for both CTAs
        }
        if (staged && lane == 0) ptx::bulk_wait_group<0>();     // this warp's stores are performed before the CTA may exit
        if (!ok && p.status != nullptr && epi_tid == 0) atomicExch(p.status, Q8K_STATUS_TIMEOUT | (10 << 8));
    }

    // ---------------------------------------------------- teardown: neither CTA may leave while the other can
    // still read its shared memory, signal its barriers or write its TMEM
    if (threadIdx.x == 0 && *abort_flag != 0) {
        // A wait was abandoned.  Copies issued before that may still be on their way into this CTA's
        // shared memory and towards its barriers: give them time to land (they take microseconds)
        // before the CTA gives both up.
        const unsigned long long t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 50000ull) {}
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::cluster_sync_all();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc_pair<kPairTmemCols>(tmem_base);
    }
}

// ------------------------------------------------------------------ host side
template <bool INT8, bool GELU, bool OUT_E4M3, bool RESID = false>
static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tr,
                       const PairParams& pp, cudaStream_t st) {
    using PairSmem = PairSmemT<RESID>;
    auto kern = gemm_8bit_pair_kernel<INT8, GELU, OUT_E4M3, RESID>;
    Q8K_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::kDynamic));
    // how many 2-CTA clusters can be resident at once (cached per kernel variant)
    static int max_clusters = -1;
    if (max_clusters < 0) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * gemm_num_sms());
        cfg.blockDim = dim3(kGemmThreads);
        cfg.dynamicSmemBytes = PairSmem::kDynamic;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); n = 0; }
        max_clusters = n;
    }
    if (max_clusters < 8) return Q8K_ERR_UNSUPPORTED;
    const int clusters = pp.total_tiles2 < max_clusters ? pp.total_tiles2 : max_clusters;
    kern<<<2 * clusters, kGemmThreads, PairSmem::kDynamic, st>>>(ta, tb, tc, tr, pp);
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

int launch_gemm_pair(bool int8, bool gelu, bool out_e4m3, bool resid, const void* a, const void* b, const GemmParams& p,
                     int bs_a, int bs_b, cudaStream_t st) {
    const char* op = int8 ? "q8_mm" : "fp8_mm";
    CUtensorMap ta, tb;
    {
        const uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)bs_a * (uint64_t)p.M};
        const uint64_t strides[1] = {(uint64_t)p.K};
        const uint32_t box[2] = {(uint32_t)kGemmBK, (uint32_t)kGemmBM};
        if (int rc = make_byte_tensor_map(&ta, a, 2, dims, strides, box, 128, op)) return rc;
    }
    {
        const uint64_t dims[2] = {(uint64_t)p.K, (uint64_t)bs_b * (uint64_t)p.N};
        const uint64_t strides[1] = {(uint64_t)p.K};
        const uint32_t box[2] = {(uint32_t)kGemmBK, (uint32_t)(kPairBN / 2)};
        if (int rc = make_byte_tensor_map(&tb, b, 2, dims, strides, box, 128, op)) return rc;
    }
    PairParams pp;
    pp.g = p;
    const int batch = bs_a > bs_b ? bs_a : bs_b;
    // output map for the staged epilogue: [batch, M, N] as bytes, 32-column boxes of 32 rows
    CUtensorMap tc = ta, tr = ta;
    const uint64_t esz = out_e4m3 ? 1 : 2;
    pp.tma_store = 0;
    if (((uint64_t)p.N * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(p.out) & 15) == 0) {
        const uint64_t dims[3] = {(uint64_t)p.N * esz, (uint64_t)p.M, (uint64_t)batch};
        const uint64_t strides[2] = {(uint64_t)p.N * esz, (uint64_t)p.M * (uint64_t)p.N * esz};
        const uint32_t box[3] = {(uint32_t)(32 * esz), 32u, 1u};
        if (int rc = make_byte_tensor_map(&tc, p.out, 3, dims, strides, box, (int)(32 * esz), op)) return rc;
        pp.tma_store = 1;
        // the residual has the output's shape: same boxes, read instead of written
        if (resid) {
            if ((reinterpret_cast<uintptr_t>(p.resid) & 15) != 0) pp.tma_store = 0;
            else if (int rc = make_byte_tensor_map(&tr, p.resid, 3, dims, strides, box, (int)(32 * esz), op)) return rc;
        }
    }
    pp.m_tiles2 = (p.M + 2 * kGemmBM - 1) / (2 * kGemmBM);
    pp.n_tiles2 = (p.N + kPairBN - 1) / kPairBN;
    const int64_t total = (int64_t)pp.m_tiles2 * pp.n_tiles2 * batch;
    if (total > 0x7fffffffLL) return Q8K_ERR_UNSUPPORTED;
    pp.total_tiles2 = (int)total;
#define Q8K_PAIR(I8)                                                                  \
    do {                                                                              \
        if (gelu) return out_e4m3 ? launch_pair<I8, true, true>(ta, tb, tc, tr, pp, st)       \
                                  : launch_pair<I8, true, false>(ta, tb, tc, tr, pp, st);     \
        return out_e4m3 ? launch_pair<I8, false, true>(ta, tb, tc, tr, pp, st)                \
                        : launch_pair<I8, false, false>(ta, tb, tc, tr, pp, st);              \
    } while (0)
    if (resid) {
        return int8 ? launch_pair<true, false, false, true>(ta, tb, tc, tr, pp, st)
                    : launch_pair<false, false, false, true>(ta, tb, tc, tr, pp, st);
    }
    if (int8) Q8K_PAIR(true);
    Q8K_PAIR(false);
#undef Q8K_PAIR
}

}  // namespace q8k
