// 8-bit GEMM with fused dequant + bias + tanh-GELU epilogue on the sm_100a
// tensor cores:  C[b] = act((A[b] . B[b]^T) * (sa[m] * sb[n]) + bias[n]).
//
//   A [bs_a, M, K], B [bs_b, N, K]  int8 (kind::i8, int32 accumulate) or
//   e4m3 (kind::f8f6f4, fp32 accumulate), both K-contiguous.
//
// Structure (one persistent CTA per SM, 10 warps):
//   warp 0      TMA producer: 128 x 128-byte A tile and BN x 128-byte B tile per
//               stage into 128B-swizzled shared memory, STAGES-deep mbarrier ring
//   warp 1      allocates TMEM; one thread issues tcgen05.mma (M=128, N=BN, K=32),
//               4 per stage, accumulating into one of two TMEM buffers
//   warps 2-9   epilogue: tcgen05.ld the finished accumulator (thread = one row of
//               one half of the columns, next chunk's load in flight), scale, bias,
//               GELU, cast, 16-byte global stores; runs while the MMA warp fills
//               the other TMEM buffer with the next tile
// Tiles are assigned statically: tile = blockIdx.x + i * gridDim.x, N fastest.
//
// Epilogue arithmetic follows csrc/gemm/q8_matmul_bias.cu:29-33,315-371 of the
// reference: float(acc) * (sa*sb) + bias, optional tanh-GELU, then bf16 (RNE)
// or e4m3 (saturating).

#include <stdlib.h>

#include "gemm_common.cuh"

namespace q8k {

template <int BN, int STAGES>
struct GemmSmem {
    static constexpr int kABytes = kGemmBM * kGemmBK;
    static constexpr int kBBytes = BN * kGemmBK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTileBytes = STAGES * kStageBytes;
    // after the tiles: barriers, TMEM base, abort flag, per-tile column scales and bias
    static constexpr int kBarOffset = kTileBytes;
    static constexpr int kNumBars = 2 * STAGES + 4;
    static constexpr int kTmemPtrOffset = kBarOffset + kNumBars * 8;
    static constexpr int kAbortOffset = kTmemPtrOffset + 4;
    static constexpr int kColScaleOffset = (kAbortOffset + 4 + 15) & ~15;
    static constexpr int kBiasOffset = kColScaleOffset + BN * 4;
    static constexpr int kTotal = kBiasOffset + BN * 4;
    static constexpr int kDynamic = kTotal + 1024;          // slack to align the base to 1024 B
};

template <bool INT8, int BN, int STAGES, bool GELU, bool OUT_E4M3, bool RESID>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_8bit_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p) {
    using L = GemmSmem<BN, STAGES>;
    constexpr int TMEM_COLS = 2 * BN;                         // two accumulators of BN fp32/int32 columns
    constexpr uint32_t IDESC = INT8 ? ptx::make_idesc_s8(kGemmBM, BN) : ptx::make_idesc_e4m3(kGemmBM, BN);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t smem_base = ptx::smem_u32(smem);
    const uint32_t bar_base = smem_base + L::kBarOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
    volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem + L::kTmemPtrOffset);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kAbortOffset);
    float* col_scale_smem = reinterpret_cast<float*>(smem + L::kColScaleOffset);
    float* bias_smem = reinterpret_cast<float*>(smem + L::kBiasOffset);

    // A launch that follows a failed one on the same status word does nothing, so a
    // protocol error costs one bounded wait instead of one per launch.
    __shared__ int prior_failure;
    if (threadIdx.x == 0) prior_failure = p.status != nullptr ? *reinterpret_cast<volatile int*>(p.status) : 0;
    __syncthreads();
    if (prior_failure != 0) return;                            // uniform across the CTA

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int k_iters = (p.K + kGemmBK - 1) / kGemmBK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(tmem_full_bar(a), 1);
            ptx::mbar_init(tmem_empty_bar(a), kGemmEpilogueThreads / 32);   // one arrival per epilogue warp
        }
        *abort_flag = 0;
        ptx::fence_barrier_init();
        ptx::fence_proxy_async_smem();
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc<TMEM_COLS>(ptx::smem_u32(const_cast<uint32_t*>(tmem_ptr_smem)));
        ptx::tmem_relinquish_alloc_permit();
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    ptx::tcgen05_fence_after_sync();
    const uint32_t tmem_base = *tmem_ptr_smem;

    if (warp == 0) {
        // ------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x) {
                const int n_blk = tile % p.n_tiles;
                const int m_blk = (tile / p.n_tiles) % p.m_tiles;
                const int batch = tile / (p.n_tiles * p.m_tiles);
                const int a_row = (p.batch_a ? batch * p.M : 0) + m_blk * kGemmBM;
                const int b_row = (p.batch_b ? batch * p.N : 0) + n_blk * BN;
                for (int kb = 0; kb < k_iters; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!ptx::mbar_wait(empty_bar(s), ph ^ 1u, abort_flag)) { ok = false; break; }
                    ptx::mbar_arrive_expect_tx(full_bar(s), L::kStageBytes);
                    const uint32_t a_dst = smem_base + s * L::kStageBytes;
                    ptx::tma_load_2d(a_dst, &tmap_a, full_bar(s), kb * kGemmBK, a_row);
                    ptx::tma_load_2d(a_dst + L::kABytes, &tmap_b, full_bar(s), kb * kGemmBK, b_row);
                }
            }
            if (!ok) {
                // Give copies that are still in flight a bounded chance to land before the CTA retires.
                if (p.status != nullptr) atomicExch(p.status, Q8K_STATUS_TIMEOUT | (1 << 8));
                const uint32_t issued = it < (uint32_t)STAGES ? it : (uint32_t)STAGES;
                for (uint32_t j = 0; j < issued; ++j) {
                    const uint32_t i2 = it - 1 - j;
                    const unsigned long long t0 = ptx::globaltimer_ns();
                    while (!ptx::mbar_try_wait(full_bar(i2 % STAGES), (i2 / STAGES) & 1u) &&
                           ptx::globaltimer_ns() - t0 < 100000000ull) {}
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------ MMA issuer
        if (lane == 0) {
            uint32_t it = 0;
            uint32_t tile_i = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.total_tiles; tile += gridDim.x, ++tile_i) {
                const uint32_t acc = tile_i & 1u;
                const uint32_t acc_ph = (tile_i >> 1) & 1u;
                if (!ptx::mbar_wait(tmem_empty_bar(acc), acc_ph ^ 1u, abort_flag)) { ok = false; break; }
                ptx::tcgen05_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < k_iters; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    if (!ptx::mbar_wait(full_bar(s), ph, abort_flag)) { ok = false; break; }
                    ptx::tcgen05_fence_after_sync();
                    const uint32_t a_addr = smem_base + s * L::kStageBytes;
                    const uint64_t a_desc = ptx::make_kmajor_desc(a_addr, 128);
                    const uint64_t b_desc = ptx::make_kmajor_desc(a_addr + L::kABytes, 128);
#pragma unroll
                    for (int k = 0; k < kGemmBK / 32; ++k) {
                        // advancing 32 bytes along K inside the 128-byte swizzle row: +2 in the >>4 address field
                        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
                        if constexpr (INT8) ptx::mma_i8(d_tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, accumulate);
                        else ptx::mma_f8f6f4(d_tmem, a_desc + 2 * k, b_desc + 2 * k, IDESC, accumulate);
                    }
                    ptx::tcgen05_commit(empty_bar(s));          // stage reusable once these MMAs retire
                }
                if (ok) ptx::tcgen05_commit(tmem_full_bar(acc));
            }
            if (!ok && p.status != nullptr) atomicExch(p.status, Q8K_STATUS_TIMEOUT | (2 << 8));
        }
    } else {
        // ------------------------------------------------ epilogue (warps 2..9, 256 threads)
        // Warp w may touch TMEM lanes [32*(w%4), +32).  Warps 2-5 take the left half of the
        // tile's columns, warps 6-9 the right half; a thread owns one output row of its half.
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        const int epi_tid = threadIdx.x - 64;
        constexpr int HALF_COLS = BN / 2;
        constexpr int NCH = HALF_COLS / 32;                    // 32-column chunks per thread and tile
        uint32_t tile_i = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x, ++tile_i) {
            const int n_blk = tile % p.n_tiles;
            const int m_blk = (tile / p.n_tiles) % p.m_tiles;
            const int batch = tile / (p.n_tiles * p.m_tiles);
            const int n0 = n_blk * BN;
            const uint32_t acc = tile_i & 1u;
            const uint32_t acc_ph = (tile_i >> 1) & 1u;

            asm volatile("bar.sync 1, 256;" ::: "memory");     // everyone is done with the previous tile's column data
            for (int c = epi_tid; c < BN; c += kGemmEpilogueThreads) {
                const int n = n0 + c;
                const bool in = n < p.N;
                col_scale_smem[c] = in ? p.b_scales[(p.batch_b ? (int64_t)batch * p.N : 0) + n] : 0.f;
                bias_smem[c] = (in && p.bias != nullptr) ? p.bias[n] : 0.f;
            }
            asm volatile("bar.sync 1, 256;" ::: "memory");

            if (ok) ok = ptx::mbar_wait(tmem_full_bar(acc), acc_ph, abort_flag);
            ok = __all_sync(0xffffffffu, ok);                  // keep the warp convergent for tcgen05.ld
            if (!ok) continue;                                 // still take part in the named barriers
            ptx::tcgen05_fence_after_sync();

            const int row = m_blk * kGemmBM + quarter * 32 + lane;
            const bool row_ok = row < p.M;
            const float sa = row_ok ? p.a_scales[(p.batch_a ? (int64_t)batch * p.M : 0) + row] : 0.f;
            const int64_t out_row = ((int64_t)batch * p.M + row) * p.N;
            const int64_t gate_row = RESID ? (((int64_t)batch * p.M + row) / p.rows_per_gate) * p.N : 0;
            const int col_base = half * HALF_COLS;
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + col_base;

            // The load of chunk c+1 is in flight while chunk c is scaled, activated and stored.
            uint32_t r[2][32];
            __syncwarp();
            ptx::tmem_ld_32x32b_x32(t_row, r[0]);
#pragma unroll
            for (int c = 0; c < NCH; ++c) {
                ptx::tmem_wait_ld();
                if (c + 1 < NCH) ptx::tmem_ld_32x32b_x32(t_row + (c + 1) * 32, r[(c + 1) & 1]);
                const int cl = col_base + c * 32;              // column inside the tile
                const int nc = n0 + cl;
                if (row_ok && nc < p.N) {
                    const uint32_t(&rc)[32] = r[c & 1];
                    float y[32];
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float2 v = epilogue_pair<INT8, GELU>(rc[j], rc[j + 1], make_float2(sa, sa),
                                                                   col_scale_smem + cl + j, bias_smem + cl + j);
                        y[j] = v.x;
                        y[j + 1] = v.y;
                    }
                    const int valid = min(32, p.N - nc);       // N % 16 == 0, so valid is 16 or 32
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
                __syncwarp();                                  // reconverge before the next warp-collective TMEM op
            }
            ptx::tcgen05_fence_before_sync();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(tmem_empty_bar(acc));
        }
        if (!ok && p.status != nullptr && epi_tid == 0) atomicExch(p.status, Q8K_STATUS_TIMEOUT | (3 << 8));
    }

    // ---------------------------------------------------- teardown
    if (threadIdx.x == 0 && *abort_flag != 0) {
        // A wait was abandoned.  Copies issued before that may still be on their way into this CTA's
        // shared memory and towards its barriers: give them time to land (they take microseconds)
        // before the CTA gives both up.
        const unsigned long long t0 = ptx::globaltimer_ns();
        while (ptx::globaltimer_ns() - t0 < 50000ull) {}
    }
    ptx::tcgen05_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        ptx::tcgen05_fence_after_sync();
        ptx::tmem_dealloc<TMEM_COLS>(tmem_base);
    }
}

// ------------------------------------------------------------------ host side
static int g_num_sms = 0;

int gemm_num_sms() {
    if (g_num_sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 148;
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
        g_num_sms = n;
    }
    return g_num_sms;
}

template <bool INT8, int BN, int STAGES, bool GELU, bool OUT_E4M3, bool RESID = false>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p, cudaStream_t st) {
    using L = GemmSmem<BN, STAGES>;
    auto kern = gemm_8bit_kernel<INT8, BN, STAGES, GELU, OUT_E4M3, RESID>;
    Q8K_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic));
    const int grid = p.total_tiles < gemm_num_sms() ? p.total_tiles : gemm_num_sms();
    kern<<<grid, kGemmThreads, L::kDynamic, st>>>(ta, tb, p);
    Q8K_CUDA_OK(cudaGetLastError());
    return Q8K_OK;
}

static int gemm_8bit(bool int8, const void* a, const void* b, const float* bias, const float* a_scales,
                     const float* b_scales, void* out, int out_dtype, int bs_a, int bs_b, int M, int N, int K,
                     int fuse_gelu, int* dev_status, void* stream, const void* resid = nullptr,
                     const void* gate = nullptr, int64_t rows_per_gate = 1) {
    const char* op = int8 ? "q8_mm" : "fp8_mm";
    Q8K_REQUIRE(a && b && a_scales && b_scales && out, Q8K_ERR_INVALID_ARG, "%s: null pointer", op);
    Q8K_REQUIRE(bs_a >= 1 && bs_b >= 1 && (bs_a == bs_b || bs_a == 1 || bs_b == 1), Q8K_ERR_INVALID_ARG,
                "%s: batch mismatch (%d vs %d)", op, bs_a, bs_b);
    Q8K_REQUIRE(M >= 0 && N > 0 && K > 0, Q8K_ERR_INVALID_ARG, "%s: bad shape M=%d N=%d K=%d", op, M, N, K);
    Q8K_REQUIRE(N % 16 == 0 && K % 16 == 0, Q8K_ERR_INVALID_ARG, "%s: N=%d and K=%d must be multiples of 16", op, N, K);
    Q8K_REQUIRE(aligned16(a) && aligned16(b) && aligned16(out), Q8K_ERR_INVALID_ARG,
                "%s: a, b and out must be 16-byte aligned", op);
    Q8K_REQUIRE(out_dtype == Q8K_DT_BF16 || out_dtype == Q8K_DT_E4M3, Q8K_ERR_UNSUPPORTED,
                "%s: output dtype %d is not bf16 or e4m3", op, out_dtype);
    const int batch = bs_a > bs_b ? bs_a : bs_b;
    Q8K_REQUIRE((int64_t)bs_a * M <= 0x7fffffffLL && (int64_t)bs_b * N <= 0x7fffffffLL, Q8K_ERR_TOO_LARGE,
                "%s: batch * rows exceeds 2^31", op);
    if (M == 0) return Q8K_OK;

    // 256-column tiles unless they would leave most of the device idle (e.g. the 128-token K/V projection
    // of a cross-attention): then twice as many 128-column tiles, each streaming half as much of B
    const int64_t tiles256 = (int64_t)((M + kGemmBM - 1) / kGemmBM) * ((N + 255) / 256) * batch;
    const bool bn256 = N > 128 && tiles256 >= gemm_num_sms() / 2;
    const int bn = bn256 ? 256 : 128;

    CUtensorMap ta, tb;
    {
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)bs_a * (uint64_t)M};
        const uint64_t strides[1] = {(uint64_t)K};
        const uint32_t box[2] = {(uint32_t)kGemmBK, (uint32_t)kGemmBM};
        if (int rc = make_byte_tensor_map(&ta, a, 2, dims, strides, box, 128, op)) return rc;
    }
    {
        const uint64_t dims[2] = {(uint64_t)K, (uint64_t)bs_b * (uint64_t)N};
        const uint64_t strides[1] = {(uint64_t)K};
        const uint32_t box[2] = {(uint32_t)kGemmBK, (uint32_t)bn};
        if (int rc = make_byte_tensor_map(&tb, b, 2, dims, strides, box, 128, op)) return rc;
    }

    GemmParams p;
    p.a_scales = a_scales;
    p.b_scales = b_scales;
    p.bias = bias;
    p.out = out;
    p.status = dev_status;
    p.resid = reinterpret_cast<const __nv_bfloat16*>(resid);
    p.gate = reinterpret_cast<const __nv_bfloat16*>(gate);
    p.rows_per_gate = rows_per_gate > 0 ? rows_per_gate : 1;
    p.M = M; p.N = N; p.K = K;
    p.batch_a = bs_a > 1; p.batch_b = bs_b > 1;
    p.m_tiles = (M + kGemmBM - 1) / kGemmBM;
    p.n_tiles = (N + bn - 1) / bn;
    const int64_t total = (int64_t)p.m_tiles * p.n_tiles * batch;
    Q8K_REQUIRE(total <= 0x7fffffffLL, Q8K_ERR_TOO_LARGE, "%s: too many tiles", op);
    p.total_tiles = (int)total;
    cudaStream_t st = (cudaStream_t)stream;
    const bool gelu = fuse_gelu != 0;
    const bool e4m3 = out_dtype == Q8K_DT_E4M3;

    // Large problems run on 256 x 256 tiles owned by CTA pairs (half the B-operand shared-memory
    // traffic per CTA); small ones, or devices that cannot co-schedule the pairs, on 128 x 256 tiles.
    static const bool pair_disabled = getenv("Q8K_GEMM_NO_PAIR") != nullptr;
    const bool fuse_resid = resid != nullptr;
    if (fuse_resid) {
        Q8K_REQUIRE(!gelu && !e4m3, Q8K_ERR_UNSUPPORTED, "%s: the gate/residual tail needs a bf16 output without GELU", op);
        Q8K_REQUIRE(aligned16(resid) && aligned16(gate), Q8K_ERR_INVALID_ARG, "%s: gate and residual must be 16-byte aligned", op);
    }
    if (!pair_disabled && M > kGemmBM && N > 128) {
        const int rc = launch_gemm_pair(int8, gelu, e4m3, fuse_resid, a, b, p, bs_a, bs_b, st);
        if (rc != Q8K_ERR_UNSUPPORTED) return rc;
    }
#define Q8K_GEMM_DISPATCH(I8, BNV, ST)                                                        \
    do {                                                                                      \
        if (gelu) return e4m3 ? launch_gemm<I8, BNV, ST, true, true>(ta, tb, p, st)           \
                              : launch_gemm<I8, BNV, ST, true, false>(ta, tb, p, st);         \
        return e4m3 ? launch_gemm<I8, BNV, ST, false, true>(ta, tb, p, st)                    \
                    : launch_gemm<I8, BNV, ST, false, false>(ta, tb, p, st);                  \
    } while (0)
    if (fuse_resid) {
        if (int8) return bn256 ? launch_gemm<true, 256, 4, false, false, true>(ta, tb, p, st)
                               : launch_gemm<true, 128, 6, false, false, true>(ta, tb, p, st);
        return bn256 ? launch_gemm<false, 256, 4, false, false, true>(ta, tb, p, st)
                     : launch_gemm<false, 128, 6, false, false, true>(ta, tb, p, st);
    }
    if (int8) {
        if (bn256) Q8K_GEMM_DISPATCH(true, 256, 4);
        Q8K_GEMM_DISPATCH(true, 128, 6);
    }
    if (bn256) Q8K_GEMM_DISPATCH(false, 256, 4);
    Q8K_GEMM_DISPATCH(false, 128, 6);
#undef Q8K_GEMM_DISPATCH
}

}  // namespace q8k

extern "C" int q8k_q8_mm(const void* a, const void* b, const float* bias, const float* a_scales,
                         const float* b_scales, void* out, int out_dtype, int bs_a, int bs_b, int M, int N,
                         int K, int fuse_gelu, int* dev_status, void* stream) {
    return q8k::gemm_8bit(true, a, b, bias, a_scales, b_scales, out, out_dtype, bs_a, bs_b, M, N, K, fuse_gelu,
                          dev_status, stream);
}

extern "C" int q8k_mm_gate_residual(int int8, const void* a, const void* b, const float* bias, const float* a_scales,
                                    const float* b_scales, const void* gate, const void* resid, int64_t rows_per_gate,
                                    void* out, int bs_a, int bs_b, int M, int N, int K, int* dev_status, void* stream) {
    if (resid == nullptr) {
        q8k::set_error_detail("mm_gate_residual: null residual");
        return Q8K_ERR_INVALID_ARG;
    }
    return q8k::gemm_8bit(int8 != 0, a, b, bias, a_scales, b_scales, out, Q8K_DT_BF16, bs_a, bs_b, M, N, K, 0, dev_status,
                          stream, resid, gate, rows_per_gate);
}

extern "C" int q8k_fp8_mm(const void* a, const void* b, const float* bias, const float* a_scales,
                          const float* b_scales, void* out, int out_dtype, int bs_a, int bs_b, int M, int N,
                          int K, int fuse_gelu, int* dev_status, void* stream) {
    return q8k::gemm_8bit(false, a, b, bias, a_scales, b_scales, out, out_dtype, bs_a, bs_b, M, N, K, fuse_gelu,
                          dev_status, stream);
}
