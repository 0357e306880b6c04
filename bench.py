#!/usr/bin/env python
"""Benchmark of the 8-bit DiT inference hot path on B200.

Headline (``value``): FP8 GEMM throughput at the LTX-Video DiT linear shapes.  One
"step" is one pass of the FP8 GEMM sweep: tokens M = 6144*B for B in {1, 4},
(K, N) in {(2048,2048), (2048,6144), (2048,8192), (8192,2048)}, each with and
without the fused bias + tanh-GELU epilogue, bf16 output -- 16 launches of the
tcgen05 kernel.  Inputs are seeded synthetic tensors (activations ~N(0,1) with
0.1 % outlier channels x20 quantised per token, weights ~N(0,0.02) per channel),
resident in HBM when the timed region starts.  ``e2e`` is the same sweep through
the public ``fp8_linear`` call with pinned HOST activations and results (H2D,
fused quantizer, GEMM, D2H inside the timed region).

``detail`` (always present, compact) carries the rest of the metric: FP8
Hadamard self-attention and masked cross-attention, the INT8 sweep, a same-run
cuBLASLt FP8 (``torch._scaled_mm``) sweep, the row-wise kernels in GB/s, one DiT
block and the 28-block stack (eager and as one CUDA graph).  ``--full`` adds the
per-shape tables.

With N > 1 GPUs (one process per GPU under torchrun) each rank runs the sweep on
its own token shard (sharding by video: no data-path collective); the time is
the max over ranks, the value the sum of all ranks' FLOPs over that time.
``detail`` then also holds the 28-block stack sharded by video (one video per
rank, the final ``all_gather_into_tensor`` inside the timed region) and one
block with its attention cores sharded by head.

``--impl reference`` times the reference's algorithm on the host CPU cores
instead (torch-CPU restatement in oracle/, all threads) on a bounded sample of
the same workload.

``--case NAME`` runs ONE kernel on one synthetic case a few times and prints its
CUDA-event time: the small, self-ending program to put under ``ncu``::

  python bench.py --case gemm_fp8 --m 6144 --k 2048 --n 2048 --gelu --iters 3
  python bench.py --case attention --b 1 --h 37 --s 4096 --iters 2
  python bench.py --case hadamard_quant --rows 24576 --dim 2048
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

E4M3 = torch.float8_e4m3fn
SHAPES_KN = [(2048, 2048), (2048, 6144), (2048, 8192), (8192, 2048)]
BATCHES = [1, 4]
TOKENS = 6144
CPU_SAMPLE_ROWS = 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NOMINAL_FP8_TFLOPS = 4500.0
QK_SCALE = math.sqrt(1 / 64) * math.sqrt(64 ** -0.5)     # Hadamard normalisation with sqrt(softmax scale) folded in
CASES = ["gemm_fp8", "gemm_int8", "attention", "cross_attention", "quantizer", "quantizer_fp8", "hadamard",
         "hadamard_quant", "norm_modulate_quant", "rms_norm", "rope", "fma", "gelu", "qk_prep", "prep_v", "dit_block"]


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.lines = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- workload
def sweep_cases():
    """(M, K, N, with_bias_gelu) for one step, in launch order."""
    cases = []
    for b in BATCHES:
        for (k, n) in SHAPES_KN:
            for fused in (False, True):
                cases.append((TOKENS * b, k, n, fused))
    return cases


# DRAM traffic of the GEMM kernel per FLOP, from one ncu capture of the M6144 K2048 N8192 bias+GELU
# launch (29.6 MB read + 53.6 MB written for 206.158 GFLOP).
NCU_DRAM_BYTES_PER_FLOP = (29.59e6 + 53.60e6) / 206.158e9


def sweep_flops():
    return sum(2.0 * m * k * n for (m, k, n, _) in sweep_cases())


def make_device_operands(dev, kind: str, seed: int):
    """Quantised operands for every distinct (M,K) activation and (N,K) weight of the sweep,
    generated on the device from a seeded generator: activations ~N(0,1) with 0.1 % of the channels
    scaled x20, weights ~N(0,0.02)."""
    import q8_kernels_b200 as q8
    g = torch.Generator(device=dev).manual_seed(seed)
    qd = E4M3 if kind == "fp8" else torch.int8
    acts, wts = {}, {}
    for b in BATCHES:
        for (k, n) in SHAPES_KN:
            m = TOKENS * b
            if (m, k) not in acts:
                x = torch.randn(m, k, generator=g, device=dev, dtype=torch.float32)
                idx = torch.randperm(k, generator=g, device=dev)[: max(1, math.ceil(0.001 * k))]
                x[:, idx] *= 20.0
                xq, xs = q8.native.tokenwise_quant(x.to(torch.bfloat16), qd)
                acts[(m, k)] = (xq, xs, x.to(torch.bfloat16))
                del x
            if (n, k) not in wts:
                w = (torch.randn(n, k, generator=g, device=dev, dtype=torch.float32) * 0.02).to(torch.bfloat16)
                wq, ws = q8.native.tokenwise_quant(w, qd)
                bias = torch.randn(n, generator=g, device=dev, dtype=torch.float32) * 0.02
                wts[(n, k)] = (wq, ws, bias)
    return acts, wts


def run_sweep(q8, acts, wts, kind: str):
    mm = (q8.native.fp8_mm, q8.native.fp8_mm_bias) if kind == "fp8" else (q8.native.q8_mm, q8.native.q8_mm_bias)
    launches = 0
    for (m, k, n, fused) in sweep_cases():
        xq, xs, _ = acts[(m, k)]
        wq, ws, bias = wts[(n, k)]
        if fused:
            mm[1](xq, wq, bias, xs, ws, True, torch.bfloat16)
        else:
            mm[0](xq, wq, xs, ws, False, torch.bfloat16)
        launches += 1
    return launches


def time_region(fn, steps: int, warmup: int, barrier=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record()
    launches = 0
    for _ in range(steps):
        launches += fn() or 0
    end.record()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    return start.elapsed_time(end), launches


def timed(fn, iters, warm=3, graph=True):
    """Average device time of one call.  The `iters` calls are captured into one CUDA graph and the replay is
    timed, so that a kernel of a few tens of microseconds is not measured at the rate at which Python can
    launch it (callables that rotate over buffers keep doing so: each captured call has its own operands)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        try:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                keep = [fn() for _ in range(iters)]            # outputs live in the graph's pool
            g.replay()
            torch.cuda.synchronize()
            s.record()
            g.replay()
            e.record()
            torch.cuda.synchronize()
            ms = s.elapsed_time(e) / iters
            del keep, g
            return ms
        except RuntimeError:
            torch.cuda.synchronize()
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / iters


def bench_config(world: int, cpu_sample: bool = False):
    cfg = {"workload": "config2_fp8_gemm_sweep", "tokens": [TOKENS * b for b in BATCHES], "shapes_KN": SHAPES_KN,
           "epilogues": ["scales", "scales+bias+tanh_gelu"], "out": "bf16", "launches_per_step": len(sweep_cases()),
           "parallelism": f"dp{world} (by video, no collective)",
           "l2": "operands + outputs of one step are ~3.7 GB, far beyond the 126 MB L2"}
    if cpu_sample:
        cfg["cpu_sample"] = f"each step = first {CPU_SAMPLE_ROWS} token rows of every (K,N) shape, bias+GELU epilogue"
    return cfg


# ----------------------------------------------------------------------------- CPU arm
def cpu_sample_cases():
    """Bounded sample of the sweep for the CPU: the first 1024 token rows of every (K,N)
    shape with the fused bias+GELU epilogue (FP8 per-token / per-channel, fp32 accumulate)."""
    return [(CPU_SAMPLE_ROWS, k, n) for (k, n) in SHAPES_KN]


def cpu_run_once(ops):
    from oracle import q8_oracle as O
    for (x, wq, ws, bias) in ops:
        xq, xs = O.tokenwise_quant(x, E4M3)
        O.fp8_mm(xq, wq, xs, ws, True, torch.bfloat16, bias=bias)


def cpu_make_ops(seed=1234):
    from oracle import q8_oracle as O
    import helpers as Hp
    ops = []
    for i, (m, k, n) in enumerate(cpu_sample_cases()):
        x = Hp.activations(m, k, seed + i)
        w = Hp.weights(n, k, seed + 100 + i)
        wq, ws = O.tokenwise_quant(w, E4M3)
        ops.append((x, wq, ws, Hp.bias_vec(n, seed + 200 + i)))
    return ops


def cpu_flops():
    return sum(2.0 * m * k * n for (m, k, n) in cpu_sample_cases())


def cpu_baseline(max_seconds: float = 12.0, steps: int = None, warmup: int = 1):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    ops = cpu_make_ops()
    for _ in range(warmup):
        cpu_run_once(ops)
    times = []
    t_all = time.perf_counter()
    n = 0
    while True:
        t0 = time.perf_counter()
        cpu_run_once(ops)
        times.append(time.perf_counter() - t0)
        n += 1
        if steps is not None:
            if n >= steps:
                break
        elif time.perf_counter() - t_all > max_seconds or n >= 50:
            break
    sec = sum(times) / len(times)
    return {"value": cpu_flops() / sec / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": "first 1024 token rows of each (K,N) sweep shape, per-token e4m3 quantizer + fp32 matmul + "
                      "bias + tanh-GELU (oracle/q8_oracle.py, torch CPU)",
            "ms_per_step": sec * 1e3, "steps": n}


def run_reference_arm(args, rank: int):
    if rank != 0:
        return
    cb = cpu_baseline(steps=max(1, args.steps), warmup=max(1, min(args.warmup, 2)))
    line = {
        "impl": "reference", "metric": "fp8_gemm_tflops", "value": cb["value"], "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": cb["steps"], "warmup": args.warmup, "ms_per_step": cb["ms_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": bench_config(args.gpus, cpu_sample=True),
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- detail
def detail_gemm_tables(q8, dev, acts, wts, kind):
    """Per-shape TFLOP/s of one kind (``--full``)."""
    nat = q8.native
    per = {}
    mm = (nat.fp8_mm, nat.fp8_mm_bias) if kind == "fp8" else (nat.q8_mm, nat.q8_mm_bias)
    for (m, k, n, fused) in sweep_cases():
        xq, xs, _ = acts[(m, k)]
        wq, ws, bias = wts[(n, k)]
        f = (lambda: mm[1](xq, wq, bias, xs, ws, True, torch.bfloat16)) if fused else \
            (lambda: mm[0](xq, wq, xs, ws, False, torch.bfloat16))
        ms = timed(f, 20)
        per[f"M{m}_K{k}_N{n}{'_bias_gelu' if fused else ''}"] = round(2.0 * m * k * n / ms / 1e9, 1)
    return per


def detail_scaled_mm(dev, acts, wts, steps):
    """The same FP8 sweep through cuBLASLt (``torch._scaled_mm`` with per-row / per-column scales,
    bf16 output; bias + GELU cases run without the GELU, which it cannot fuse): a same-run, same-box
    library number to set the hand-written kernel against.  It runs as many steps as the headline loop,
    so that both numbers are taken in the same power state (a long loop sits at the power cap)."""
    try:
        def step():
            for (m, k, n, fused) in sweep_cases():
                xq, xs, _ = acts[(m, k)]
                wq, ws, bias = wts[(n, k)]
                torch._scaled_mm(xq, wq.t(), scale_a=xs.view(m, 1), scale_b=ws.view(1, n),
                                 bias=bias.to(torch.bfloat16) if fused else None, out_dtype=torch.bfloat16)
        ms = timed(step, steps, warm=3, graph=False)
        return {"tflops": round(sweep_flops() / ms / 1e9, 1), "ms_per_step": round(ms, 4), "steps": steps,
                "what": "torch._scaled_mm, e4m3 x e4m3, row-wise scales, bf16 out, same 16 launches (no GELU)"}
    except Exception as exc:                                   # noqa: BLE001  (library path: report, do not fail the bench)
        return {"tflops": None, "unavailable": f"{type(exc).__name__}: {str(exc)[:160]}"}


def detail_attention(q8, dev, peaks):
    """Self-attention B=2 H=32 S=6144 D=64 (Hadamard-rotated e4m3 Q/K, bf16 out) and cross-attention
    on 128 keys with per-batch valid lengths; CUDA-event times of the kernel and of the public call
    that includes the bf16 -> e4m3 pre-pass."""
    nat = q8.native
    g = torch.Generator(device=dev).manual_seed(3)
    B, H, S, D = 2, 32, 6144, 64
    qkv = [torch.randn(B, S, H * D, generator=g, device=dev).to(torch.bfloat16).view(B, S, H, D).transpose(1, 2)
           for _ in range(3)]
    F = q8.functional.flash_attention.flash_attn_func
    q8_, k8_, vt_ = nat.attention_prep(qkv[0], qkv[1], qkv[2], True, QK_SCALE)
    ms_core = timed(lambda: nat.flash_attention(q8_, k8_, vt_, 1.0, None, torch.bfloat16), 10)
    ms_full = timed(lambda: F(qkv[0], qkv[1], qkv[2], apply_qk_hadamard=True, out_dtype=torch.bfloat16), 10)
    fl = 4.0 * B * H * S * S * D
    sm_mhz = float(peaks.get("sm_max_mhz") or 1965.0)
    exp_floor_ms = B * H * S * S / (148 * 16 * sm_mhz * 1e6) * 1e3      # 16 exp2 per clock per SM
    out = {"self_attention": {
        "shape_BHSD": [B, H, S, D], "kernel_ms": round(ms_core, 4), "kernel_tflops": round(fl / ms_core / 1e9, 1),
        "frac_of_nominal_4500": round(fl / ms_core / 1e9 / NOMINAL_FP8_TFLOPS, 4),
        "exp2_floor_ms": round(exp_floor_ms, 4), "frac_of_exp2_floor": round(exp_floor_ms / ms_core, 4),
        "with_prepass_ms": round(ms_full, 4), "with_prepass_tflops": round(fl / ms_full / 1e9, 1)}}
    kx = [torch.randn(B, 128, H * D, generator=g, device=dev).to(torch.bfloat16).view(B, 128, H, D).transpose(1, 2)
          for _ in range(2)]
    lens = torch.randint(16, 129, (B,), generator=g, device=dev, dtype=torch.int32)
    q8c, k8c, vtc = nat.attention_prep(qkv[0], kx[0], kx[1], True, QK_SCALE)
    ms_x = timed(lambda: nat.flash_attention(q8c, k8c, vtc, 1.0, lens, torch.bfloat16), 20)
    bytes_x = B * H * S * D * (1 + 2) + 2 * B * H * 128 * D
    gbs = bytes_x / ms_x / 1e6
    out["cross_attention"] = {"shape": "Q [2,32,6144,64] x K/V [2,32,128,64], key lengths " + str(lens.tolist()),
                              "kernel_ms": round(ms_x, 4), "gbs_e4m3_in_bf16_out": round(gbs, 1),
                              "frac_of_measured_hbm": round(gbs / peaks["hbm_gbs"], 3),
                              "tflops_dense": round(4.0 * B * H * S * 128 * D / ms_x / 1e9, 1)}
    return out


def rowwise_cases(q8, dev, rows, dim, g):
    """name -> (callable over rotating inputs, algorithmic bytes per call)."""
    nat = q8.native
    nset = max(2, int(math.ceil(400e6 / (rows * dim * 2))))     # rotate over > 3 x L2 of inputs
    xs = [torch.randn(rows, dim, generator=g, device=dev).to(torch.bfloat16) for _ in range(nset)]
    x8 = [x.to(E4M3) for x in xs[:2]]
    cos = torch.randn(1, rows, dim, generator=g, device=dev)
    sin = torch.randn(1, rows, dim, generator=g, device=dev)
    mod = [(torch.randn(1, 1, dim, generator=g, device=dev) * 0.1).to(torch.bfloat16) for _ in range(2)]
    state = {"i": 0}

    def rot():
        state["i"] = (state["i"] + 1) % nset
        return xs[state["i"]]
    sq = 1 / math.sqrt(dim)
    return {
        "quantizer_int8": (lambda: nat.tokenwise_quant(rot(), None), rows * (3 * dim + 4)),
        "quantizer_fp8": (lambda: nat.tokenwise_quant(rot(), E4M3), rows * (3 * dim + 4)),
        "hadamard_bf16": (lambda: nat.fast_hadamard_transform(rot(), sq, None), rows * 4 * dim),
        "hadamard_quant_int8": (lambda: nat.hadamard_quant(rot(), sq, torch.int8), rows * (3 * dim + 4)),
        "norm_modulate_quant_int8": (lambda: nat.norm_modulate_quant(rot().view(1, rows, dim), mod[0], mod[1]),
                                     rows * (3 * dim + 4)),
        "rms_norm": (lambda: nat.rms_norm(rot(), None, None), rows * (4 * dim + 4)),
        # x in, x out, and one fp32 cos and one fp32 sin value per element (batch 1: nothing is shared)
        "rope_bf16": (lambda: nat.rope(rot().view(1, rows, dim), cos, sin, torch.bfloat16), rows * (4 + 8) * dim),
        "fma_e4m3": (lambda: nat.fma_8bit(x8[state["i"] & 1].view(1, rows, dim), mod[0], mod[1], 1.0), rows * 2 * dim),
        "gelu": (lambda: nat.gelu_forward(rot(), None), rows * 4 * dim),
    }


def detail_rowwise(q8, dev, peaks, full):
    g = torch.Generator(device=dev).manual_seed(5)
    out = {}
    hbm = peaks["hbm_gbs"]
    for rows, dim in [(24576, 2048), (24576, 8192)]:
        cases = rowwise_cases(q8, dev, rows, dim, g)
        for name, (fn, nbytes) in cases.items():
            if not full and name in ("fma_e4m3",) and dim == 8192:
                continue
            ms = timed(fn, 20)
            gbs = nbytes / ms / 1e6
            out[f"{name}_{rows}x{dim}"] = {"ms": round(ms, 4), "gbs": round(gbs, 1),
                                           "frac_of_measured_hbm": round(gbs / hbm, 3)}
        del cases
        torch.cuda.empty_cache()
    return out


def dit_inputs(q8, dev, seed, caption=True):
    cfg = q8.blocks.LTXStackConfig()
    g = torch.Generator(device="cpu").manual_seed(seed)
    S, T = 6144, 128
    x = torch.randn(1, S, cfg.inner_dim, generator=g).to(torch.bfloat16).to(dev)
    text = torch.randn(1, T, cfg.caption_channels if caption else cfg.inner_dim, generator=g).to(torch.bfloat16).to(dev)
    ts = (torch.randn(1, 1, 6 * cfg.inner_dim, generator=g) * 0.1).to(torch.bfloat16).to(dev)
    grid = q8.blocks.latent_grid(16, 16, 24, device=dev)
    lens = torch.tensor([97], dtype=torch.int32, device=dev)
    return cfg, x, text, ts, grid, lens


DIT_BLOCK_FLOP = (2.0 * 6144 * (6 * 2048 ** 2 + 2 * 2048 * 8192) + 2.0 * 128 * 2 * 2048 ** 2
                  + 4.0 * 32 * 6144 * 6144 * 64 + 4.0 * 32 * 6144 * 128 * 64)


def detail_dit(q8, dev, rank, world):
    """One video (16x16x24 latent grid = 6144 tokens, 128 text tokens) through one block and through the
    28-block stack: INT8 linears, FP8 Hadamard attention, random-init weights.  With several ranks every
    rank runs its own video (same weights, different inputs) and the final hidden states are
    all-gathered inside the timed region; times are the max over ranks."""
    import torch.distributed as dist
    from q8_kernels_b200 import sharding
    cfg, x, text, ts, grid, lens = dit_inputs(q8, dev, seed=100 + rank)
    stack = q8.blocks.random_init_(q8.blocks.LTXStack(cfg), seed=11, device=dev)
    barrier = dist.barrier if world > 1 else None

    def reduce_max(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    with torch.no_grad():
        freqs = stack.freqs_cis(grid)
        tproj = stack.caption_projection(text)
        blk = stack.transformer_blocks[0]
        ms_blk = reduce_max(timed(lambda: blk(x, freqs, None, tproj, lens, ts), 10))

        def run_eager():
            y = stack(x, grid, text, lens, ts)
            if world > 1:
                y = sharding.gather_videos(y, [1] * world)
            return 1
        steps = 3
        ms, _ = time_region(run_eager, steps, 2, barrier)
        ms_stack = reduce_max(ms / steps)

        # the same stack replayed from one CUDA graph (no host work between its kernels); the gather follows the replay
        side = torch.cuda.Stream(dev)
        with torch.cuda.stream(side):
            stack(x, grid, text, lens, ts)
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y_static = stack(x, grid, text, lens, ts)

        def run_graph():
            graph.replay()
            if world > 1:
                sharding.gather_videos(y_static, [1] * world)
            return 1
        ms, _ = time_region(run_graph, steps, 2, barrier)
        ms_graph = reduce_max(ms / steps)
        finite = bool(torch.isfinite(y_static.float()).all())
        del graph, y_static
    q8._lib.check_status(dev)
    out = {"tokens": 6144, "text_tokens": 128, "linears": "int8", "attention": "fp8 hadamard", "videos": world,
           "block_ms": round(ms_blk, 4), "block_tflops": round(DIT_BLOCK_FLOP / ms_blk / 1e9, 1),
           "stack28_ms": round(ms_stack, 3), "stack28_cuda_graph_ms": round(ms_graph, 3),
           "stack28_videos_per_s": round(world / (ms_graph / 1e3), 2),
           "stack28_tflops_all_gpus": round(world * 28 * DIT_BLOCK_FLOP / ms_graph / 1e9, 1),
           "output_finite": finite}
    if world > 1:
        out["sharding"] = ("by video: one video per rank, weights replicated, no collective inside the stack; "
                           "all_gather_into_tensor of the final [1,6144,2048] bf16 hidden states inside the timed region")
    del stack
    torch.cuda.empty_cache()
    # the same block built from FP8 linears (per-token e4m3 activations, e4m3 weights), one block only
    ms_fp8 = float("nan")
    try:
        cfg8 = q8.blocks.LTXStackConfig(num_layers=1, linear="fp8")
        stack8 = q8.blocks.random_init_(q8.blocks.LTXStack(cfg8), seed=11, device=dev)
        with torch.no_grad():
            tproj8 = stack8.caption_projection(text)
            blk8 = stack8.transformer_blocks[0]
            ms_fp8 = timed(lambda: blk8(x, freqs, None, tproj8, lens, ts), 10)
        del stack8, blk8
    except Exception as exc:                                   # noqa: BLE001  (an extra figure: report, do not fail the bench)
        out["block_fp8_linears_unavailable"] = f"{type(exc).__name__}: {str(exc)[:120]}"
    ms_fp8 = reduce_max(ms_fp8)
    if ms_fp8 == ms_fp8:
        out["block_ms_fp8_linears"] = round(ms_fp8, 4)
    q8._lib.check_status(dev)
    torch.cuda.empty_cache()
    return out


def detail_head_sharded_block(q8, dev, rank, world):
    """One DiT block on 6144 tokens with the self- and cross-attention cores sharded by head over the
    ranks (H / world heads each); linears, norms and RoPE replicated.  Two ways to reassemble the
    channel dim before the output projection: an NCCL all-gather, or the attention kernel storing its
    heads into every rank's buffer (up to the 8 destinations one launch can store to).  Every
    variant is compared bit for bit with the replicated block.  Max over ranks of the CUDA-event time."""
    import torch.distributed as dist
    from q8_kernels_b200 import sharding
    cfg, x, text, ts, grid, lens = dit_inputs(q8, dev, seed=99, caption=False)
    cfg = q8.blocks.LTXStackConfig(num_layers=1)
    stack = q8.blocks.random_init_(q8.blocks.LTXStack(cfg), seed=11, device=dev)        # same seed: replicated weights
    blk = stack.transformer_blocks[0]
    freqs = stack.freqs_cis(grid)
    hs = sharding.head_shard(cfg.num_attention_heads, rank, world)
    use_peers = world <= sharding.PeerBuffers.MAX_WORLD
    peers = sharding.PeerBuffers(6144 * cfg.inner_dim, dev) if use_peers else None

    def run(sharded):
        with torch.no_grad():
            if sharded == "nccl":
                return blk(x, freqs, None, text, lens, ts, head_shard=hs, gather_heads=sharding.gather_heads)
            if sharded == "peer":
                return blk(x, freqs, None, text, lens, ts, head_shard=hs, peer_buffers=peers)
            return blk(x, freqs, None, text, lens, ts)

    ref = run(None)
    checks = {}
    for name in ("replicated_again", "nccl") + (("peer", "peer_again") if use_peers else ()):
        got = run({"replicated_again": None, "peer_again": "peer"}.get(name, name))
        checks[name] = int((got != ref).sum())
    t = torch.tensor([checks[k] for k in sorted(checks)], device=dev, dtype=torch.int64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)                  # worst rank
    mismatches = dict(zip(sorted(checks), (int(v) for v in t)))
    out = {"world": world, "heads_per_rank": cfg.num_attention_heads // world, "tokens": 6144,
           "mismatching_elements_vs_replicated_max_over_ranks": mismatches,
           "bit_identical_to_replicated": not any(mismatches.values())}
    for name, sharded in (("replicated_ms", None), ("head_sharded_nccl_gather_ms", "nccl")) + \
            ((("head_sharded_peer_store_ms", "peer"),) if use_peers else ()):
        ms, _ = time_region(lambda: run(sharded) is None or 1, 20, 3, dist.barrier)
        t = torch.tensor([ms / 20], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out[name] = round(float(t[0]), 4)
    q8._lib.check_status(dev)
    if peers is not None:
        peers.close()
    return out


# ----------------------------------------------------------------------------- one kernel, one case
def run_case(a):
    """``--case``: one kernel on one synthetic case, ``--iters`` launches after ``--case-warmup``."""
    import q8_kernels_b200 as q8
    nat = q8.native
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    work, unit = 0.0, "TFLOP/s"

    if a.case in ("gemm_fp8", "gemm_int8"):
        qd = E4M3 if a.case == "gemm_fp8" else torch.int8
        x = torch.randn(a.m, a.k, generator=g, device=dev).to(torch.bfloat16)
        w = (torch.randn(a.n, a.k, generator=g, device=dev) * 0.02).to(torch.bfloat16)
        xq, xs = nat.tokenwise_quant(x, qd)
        wq, ws = nat.tokenwise_quant(w, qd)
        bias = torch.randn(a.n, generator=g, device=dev) * 0.02
        mm, mmb = (nat.fp8_mm, nat.fp8_mm_bias) if qd == E4M3 else (nat.q8_mm, nat.q8_mm_bias)
        fn = (lambda: mmb(xq, wq, bias, xs, ws, True, torch.bfloat16)) if a.gelu else \
             (lambda: mm(xq, wq, xs, ws, False, torch.bfloat16))
        if a.resid:                                       # the block's "gate * linear + residual" epilogue
            gate = torch.randn(1, 1, a.n, generator=g, device=dev).to(torch.bfloat16)
            resid = torch.randn(1, a.m, a.n, generator=g, device=dev).to(torch.bfloat16)
            fn = lambda: nat.mm_gate_residual(xq, wq, bias, xs, ws, gate, resid)                       # noqa: E731
        work = 2.0 * a.m * a.k * a.n / 1e12
    elif a.case in ("attention", "cross_attention", "qk_prep", "prep_v"):
        skv = a.skv if a.skv > 0 else (a.s if a.case != "cross_attention" else 128)
        mk = lambda s: torch.randn(a.b, s, a.h * 64, generator=g, device=dev).to(torch.bfloat16)   # noqa: E731
        qf, kf, vf = mk(a.s), mk(skv), mk(skv)
        hv = lambda t: t.view(a.b, t.shape[1], a.h, 64).transpose(1, 2)                               # noqa: E731
        if a.case == "qk_prep":
            wq = torch.ones(a.h * 64, device=dev)
            cs = torch.randn(1, a.s, a.h * 64, generator=g, device=dev)
            fn = lambda: nat.qk_norm_rope_prep_pair(qf, kf, wq, wq, (cs, cs), a.h, True, QK_SCALE)   # noqa: E731
            work, unit = a.b * a.s * a.h * 64 * (2 * 3 + 8) / 1e9, "GB/s"
        elif a.case == "prep_v":
            fn = lambda: nat.attention_prep_v(hv(vf))                                                 # noqa: E731
            work, unit = a.b * skv * a.h * 64 * 3 / 1e9, "GB/s"
        else:
            q8_, k8_, vt_ = nat.attention_prep(hv(qf), hv(kf), hv(vf), True, QK_SCALE)
            lens = None
            if a.case == "cross_attention":
                lens = torch.randint(16, 129, (a.b,), generator=g, device=dev, dtype=torch.int32)
            fn = lambda: nat.flash_attention(q8_, k8_, vt_, 1.0, lens, torch.bfloat16)              # noqa: E731
            work = 4.0 * a.b * a.h * a.s * skv * 64 / 1e12
    elif a.case == "dit_block":
        cfg = q8.blocks.LTXStackConfig(num_layers=1)
        stack = q8.blocks.random_init_(q8.blocks.LTXStack(cfg), seed=1, device=dev)
        blk = stack.transformer_blocks[0]
        S, T = a.s, 128
        x = torch.randn(a.b, S, cfg.inner_dim, generator=g, device=dev).to(torch.bfloat16)
        text = torch.randn(a.b, T, cfg.inner_dim, generator=g, device=dev).to(torch.bfloat16)
        ts = (torch.randn(a.b, 1, 6 * cfg.inner_dim, generator=g, device=dev) * 0.1).to(torch.bfloat16)
        freqs = stack.freqs_cis(q8.blocks.latent_grid(S // 384, 16, 24, device=dev))
        lens = torch.full((a.b,), 97, dtype=torch.int32, device=dev)

        def fn():
            with torch.no_grad():
                return blk(x, freqs, None, text, lens, ts)
        work = a.b * (2.0 * S * (6 * 2048 ** 2 + 2 * 2048 * 8192) + 4.0 * 2048 ** 2 * T + 4.0 * 32 * S * (S + T) * 64) / 1e12
    else:
        unit = "GB/s"
        name = {"quantizer": "quantizer_int8", "hadamard": "hadamard_bf16", "hadamard_quant": "hadamard_quant_int8",
                "norm_modulate_quant": "norm_modulate_quant_int8", "rope": "rope_bf16", "fma": "fma_e4m3"}.get(a.case, a.case)
        fn, nbytes = rowwise_cases(q8, dev, a.rows, a.dim, g)[name]
        work = nbytes / 1e9

    for _ in range(a.case_warmup):
        fn()
    torch.cuda.synchronize()
    if a.graph:
        side = torch.cuda.Stream(dev)
        with torch.cuda.stream(side):                     # first calls outside capture: lazy set-up, allocator warm-up
            fn()
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            keep = fn()                                   # noqa: F841  (outputs live in the graph's pool)
        fn = graph.replay
        fn()
        torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(a.iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    q8._lib.check_status(dev)
    ms = s.elapsed_time(e) / a.iters
    print(f"{a.case}: {ms:.4f} ms/launch, {work / (ms / 1e3):.1f} {unit}")


# ----------------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--full", action="store_true", help="add per-shape GEMM tables and every row-wise case")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-detail", action="store_true", help="headline only")
    ap.add_argument("--case", choices=CASES, help="run one kernel on one case and print its time")
    ap.add_argument("--m", type=int, default=6144)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--gelu", action="store_true", help="GEMM case with bias + tanh-GELU epilogue")
    ap.add_argument("--resid", action="store_true", help="GEMM case with the gate * y + residual epilogue")
    ap.add_argument("--b", type=int, default=1)
    ap.add_argument("--h", type=int, default=8)
    ap.add_argument("--s", type=int, default=4096)
    ap.add_argument("--skv", type=int, default=0, help="key/value length (default: --s, or 128 for cross_attention)")
    ap.add_argument("--rows", type=int, default=24576)
    ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--case-warmup", type=int, default=1)
    ap.add_argument("--graph", action="store_true", help="--case: capture into a CUDA graph and time its replays")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    if args.case:
        run_case(args)
        return
    args.warmup = max(args.warmup, 3)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import q8_kernels_b200 as q8

    barrier = None
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        barrier = dist.barrier
    peaks = load_peaks()

    # ---- device-resident sweep (value)
    acts, wts = make_device_operands(dev, "fp8", seed=1234 + rank)
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_total, launches = time_region(lambda: run_sweep(q8, acts, wts, "fp8"), args.steps, args.warmup, barrier)
    clocks = sampler.stop()
    q8._lib.check_status(dev)

    # ---- end to end through the public API with host buffers
    pinned_in, pinned_out = {}, {}
    for (m, k, n, fused) in sweep_cases():
        if (m, k) not in pinned_in:
            pinned_in[(m, k)] = acts[(m, k)][2].cpu().pin_memory()
        pinned_out[(m, n)] = torch.empty(1, m, n, dtype=torch.bfloat16).pin_memory()
    h2d = sum(pinned_in[(m, k)].numel() * 2 for (m, k, n, f) in sweep_cases())
    d2h = sum(m * n * 2 for (m, k, n, f) in sweep_cases())
    fp8_linear = q8.functional.linear.fp8_linear

    # Three streams, as a serving loop would run it: uploads, compute (the current stream) and
    # downloads overlap across calls; PCIe is full duplex, so the step costs about the larger of
    # the two copy directions instead of their sum.  The step ends when the last download has.
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

    def e2e_step():
        cur = torch.cuda.current_stream(dev)
        s_in.wait_stream(cur)
        for (m, k, n, fused) in sweep_cases():
            with torch.cuda.stream(s_in):
                x = pinned_in[(m, k)].to(dev, non_blocking=True)
                uploaded = s_in.record_event()
            cur.wait_event(uploaded)
            x.record_stream(cur)
            wq, ws, bias = wts[(n, k)]
            y = fp8_linear(x, wq, bias if fused else None, None, ws, False, torch.bfloat16)
            computed = cur.record_event()
            s_out.wait_event(computed)
            with torch.cuda.stream(s_out):
                pinned_out[(m, n)].copy_(y, non_blocking=True)
            y.record_stream(s_out)
        cur.wait_stream(s_out)
        return len(sweep_cases()) * 2          # quantizer + GEMM kernel per call

    e2e_steps = max(2, min(args.steps, 5))
    ms_e2e, _ = time_region(e2e_step, e2e_steps, 1, barrier)
    del pinned_in, pinned_out

    # ---- reduce over ranks
    ms_step = ms_total / args.steps
    ms_e2e_step = ms_e2e / e2e_steps
    if world > 1:
        t = torch.tensor([ms_step, ms_e2e_step], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, ms_e2e_step = float(t[0]), float(t[1])
    flops = sweep_flops()
    value = world * flops / ms_step / 1e9
    e2e_value = world * flops / ms_e2e_step / 1e9

    line = None
    if rank == 0:
        # A timed region of well under a second runs at burst clocks (the sampled SM clock says so);
        # a long one settles under the power cap.  The denominator follows the regime that was measured.
        sm, smax = clocks.get("sm_mhz"), clocks.get("sm_max_mhz")
        if sm and smax:
            burst = sm >= 0.93 * smax
        else:
            burst = ms_total < 1000.0
        bf16 = peaks["bf16_tflops"] if burst else peaks["bf16_tflops_sustained"]
        peak = 2.0 * bf16
        per_gpu = flops / ms_step / 1e9
        line = {
            "metric": "fp8_gemm_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
            "config": bench_config(world),
            "clocks": clocks,
            "e2e": {"value": round(e2e_value, 2), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": round(ms_e2e_step, 3),
                    "api": "q8_kernels_b200.functional.linear.fp8_linear(bf16 pinned host activations) -> pinned host bf16; uploads, compute and downloads on three streams"},
            "gpu_launches": launches,
            "roofline": {"bound": "tensor", "achieved": round(per_gpu, 2), "peak": round(peak, 1), "unit": "TFLOP/s",
                         "frac": round(per_gpu / peak, 4),
                         "traffic": round(NCU_DRAM_BYTES_PER_FLOP * flops / len(sweep_cases())),
                         "traffic_basis": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the "
                                          "M6144 K2048 N8192 bias+GELU launch (83.2 MB for 206.2 GFLOP), scaled by "
                                          "FLOPs to the sweep's average launch",
                         "peak_kind": "burst" if burst else "sustained",
                         "peak_basis": f"2 x {peaks['_source']} {'burst' if burst else 'sustained'} dense bf16 cuBLAS "
                                       f"rate ({bf16} TFLOP/s): FP8 issues at twice the bf16 rate; the timed region "
                                       f"lasted {ms_total:.0f} ms at a median SM clock of {sm} MHz",
                         "frac_of_nominal_4500": round(per_gpu / NOMINAL_FP8_TFLOPS, 4),
                         "kernel": "gemm_8bit_pair_kernel<fp8> (cta_group::2, 256x256 tiles, 6 stages, TMA-store epilogue)",
                         "flops_per_launch_avg": flops / len(sweep_cases()),
                         "avg_launch_ms": round(ms_step / len(sweep_cases()), 5)},
        }
        if not args.no_cpu_baseline and world == 1:
            cb = cpu_baseline()
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
            line["cpu_baseline"]["value"] = round(cb["value"], 4)

    # ---- the rest of the metric
    if not args.no_detail:
        detail = {}
        if rank == 0:
            sm_ref = detail_scaled_mm(dev, acts, wts, args.steps)
            detail["fp8_sweep_cublaslt_scaled_mm"] = sm_ref
            if sm_ref.get("tflops"):
                line["roofline"]["frac_vs_scaled_mm"] = round(flops / ms_step / 1e9 / sm_ref["tflops"], 4)
            if args.full:
                detail["fp8_gemm_tflops_per_shape"] = detail_gemm_tables(q8, dev, acts, wts, "fp8")
        del acts, wts
        torch.cuda.empty_cache()
        if rank == 0:
            acts8, wts8 = make_device_operands(dev, "int8", seed=7)
            ms8, _ = time_region(lambda: run_sweep(q8, acts8, wts8, "int8"), 5, 3)
            detail["int8_gemm_sweep"] = {"tflops": round(flops / (ms8 / 5) / 1e9, 1), "ms_per_step": round(ms8 / 5, 4),
                                         "frac_of_nominal_4500": round(flops / (ms8 / 5) / 1e9 / NOMINAL_FP8_TFLOPS, 4)}
            if args.full:
                detail["int8_gemm_tflops_per_shape"] = detail_gemm_tables(q8, dev, acts8, wts8, "int8")
            del acts8, wts8
            torch.cuda.empty_cache()
            detail.update(detail_attention(q8, dev, peaks))
            torch.cuda.empty_cache()
            detail["rowwise"] = detail_rowwise(q8, dev, peaks, args.full)
            q8._lib.check_status(dev)
        if world > 1:
            dist.barrier()
        dit = detail_dit(q8, dev, rank, world)                # collective inside when world > 1: every rank runs it
        if rank == 0:
            detail["dit"] = dit
        if world > 1:
            sharded = detail_head_sharded_block(q8, dev, rank, world)
            if rank == 0:
                detail["dit_block_head_sharded"] = sharded
        if rank == 0:
            line["detail"] = detail
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
