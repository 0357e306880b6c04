"""Run one kernel on one synthetic case a few times -- the small, self-ending
program to put under ``ncu`` (or a timer) when looking at a single kernel.

  python -m q8_kernels_b200.run_case gemm_fp8 --m 6144 --k 2048 --n 2048 --gelu --iters 3
  python -m q8_kernels_b200.run_case attention --b 1 --h 8 --s 4096 --iters 2
  python -m q8_kernels_b200.run_case hadamard_quant --rows 24576 --dim 2048

Prints the mean CUDA-event time per launch and the derived TFLOP/s or GB/s.
"""
from __future__ import annotations

import argparse
import math

import torch


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=["gemm_fp8", "gemm_int8", "attention", "cross_attention", "quantizer", "hadamard",
                                     "hadamard_quant", "rms_norm", "rope", "gelu", "dit_block"])
    ap.add_argument("--m", type=int, default=6144)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--n", type=int, default=2048)
    ap.add_argument("--gelu", action="store_true", help="GEMM with bias + tanh-GELU epilogue")
    ap.add_argument("--b", type=int, default=1)
    ap.add_argument("--h", type=int, default=8)
    ap.add_argument("--s", type=int, default=4096)
    ap.add_argument("--skv", type=int, default=0, help="key/value length (default: --s, or 128 for cross_attention)")
    ap.add_argument("--rows", type=int, default=24576)
    ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--graph", action="store_true", help="capture the case into a CUDA graph and time its replays")
    a = ap.parse_args()

    import q8_kernels_b200 as q8
    nat = q8.native
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    E4M3 = torch.float8_e4m3fn
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
        work = 2.0 * a.m * a.k * a.n / 1e12
    elif a.case in ("attention", "cross_attention"):
        skv = a.skv if a.skv > 0 else (a.s if a.case == "attention" else 128)
        q = torch.randn(a.b, a.s, a.h * 64, generator=g, device=dev).to(torch.bfloat16).view(a.b, a.s, a.h, 64).transpose(1, 2)
        k = torch.randn(a.b, skv, a.h * 64, generator=g, device=dev).to(torch.bfloat16).view(a.b, skv, a.h, 64).transpose(1, 2)
        v = torch.randn(a.b, skv, a.h * 64, generator=g, device=dev).to(torch.bfloat16).view(a.b, skv, a.h, 64).transpose(1, 2)
        q8_, k8_, vt_ = nat.attention_prep(q, k, v, True, math.sqrt(1 / 64) * math.sqrt(64 ** -0.5))
        lens = None
        if a.case == "cross_attention":
            lens = torch.randint(16, 129, (a.b,), generator=g, device=dev, dtype=torch.int32)
        fn = lambda: nat.flash_attention(q8_, k8_, vt_, 1.0, lens, torch.bfloat16)  # noqa: E731
        work = 4.0 * a.b * a.h * a.s * skv * 64 / 1e12
    elif a.case == "dit_block":
        # one LTX-Video block (hidden 2048, 32 x 64 heads, FFN 8192) on --s tokens and 128 text tokens
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
                return blk(x, freqs, None, text, lens, ts, attn_type="q8_kernels")
        work = a.b * (2.0 * S * (6 * 2048 ** 2 + 2 * 2048 * 8192) + 4.0 * 2048 ** 2 * T + 4.0 * 32 * S * (S + T) * 64) / 1e12
    else:
        x = torch.randn(a.rows, a.dim, generator=g, device=dev).to(torch.bfloat16)
        unit = "GB/s"
        if a.case == "quantizer":
            fn, nbytes = (lambda: nat.tokenwise_quant(x, None)), a.rows * (3 * a.dim + 4)
        elif a.case == "hadamard":
            fn, nbytes = (lambda: nat.fast_hadamard_transform(x, 1 / math.sqrt(a.dim), None)), a.rows * 4 * a.dim
        elif a.case == "hadamard_quant":
            fn, nbytes = (lambda: nat.hadamard_quant(x, 1 / math.sqrt(a.dim), torch.int8)), a.rows * (3 * a.dim + 4)
        elif a.case == "rms_norm":
            fn, nbytes = (lambda: nat.rms_norm(x, None, None)), a.rows * (4 * a.dim + 4)
        elif a.case == "rope":
            cs = torch.randn(1, a.rows, a.dim, generator=g, device=dev)
            x3 = x.view(1, a.rows, a.dim)
            fn, nbytes = (lambda: nat.rope(x3, cs, cs, torch.bfloat16)), a.rows * 12 * a.dim
        else:
            fn, nbytes = (lambda: nat.gelu_forward(x, None)), a.rows * 4 * a.dim
        work = nbytes / 1e9

    for _ in range(a.warmup):
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


if __name__ == "__main__":
    main()
