"""The allocation-free linear entry point (q8k_linear_static), called through the C ABI.

Some hosts of this library cannot hand it device scratch: a plugin inside a runtime that has
reserved all device memory for itself gets input and output pointers and nothing else, and a
latency-critical thread may not be allowed to call cudaMalloc at all.  For them the library
carries a fixed scratch array of its own.  This test checks that the entry point produces exactly
what q8k_linear (caller-provided workspace) produces, twice in a row with different problems so
that the second call runs over the first call's leftovers, and that oversized problems are
refused.  It allocates its tensors with torch, but the call under test receives only pointers.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import pytest
import torch

import helpers as Hp

pytestmark = pytest.mark.gpu
E4M3 = torch.float8_e4m3fn


def _call_both(lib, _lib, dev, M, K, N, w_dtype, use_hadamard, gelu, seed):
    from q8_kernels_b200 import native
    x = Hp.activations(M, K, seed).to(dev)
    w = Hp.weights(N, K, seed + 1).to(dev)
    bias = Hp.bias_vec(N, seed + 2).to(dev)
    if w_dtype == torch.int8:
        wq, ws = native.hadamard_quant(w, K ** -0.5, torch.int8)
    else:
        wq, ws = native.tokenwise_quant(w, E4M3)
    status = _lib.status_word(dev)
    stream = _lib.stream_ptr(dev)
    out_ws = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    out_static = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
    need = lib.q8k_linear_workspace_bytes(M, K)
    ws_buf = torch.empty(need, dtype=torch.uint8, device=dev)
    args = (x.data_ptr(), _lib.DT_BF16, wq.data_ptr(), _lib.dt(wq.dtype), ws.data_ptr(), bias.data_ptr())
    tail = (_lib.DT_BF16, M, N, K, int(use_hadamard), int(gelu))
    rc = lib.q8k_linear(*args, out_ws.data_ptr(), *tail, ws_buf.data_ptr(), need, status.data_ptr(), stream)
    assert rc == 0, lib.q8k_last_error_detail()
    rc = lib.q8k_linear_static(*args, out_static.data_ptr(), *tail, status.data_ptr(), stream)
    assert rc == 0, lib.q8k_last_error_detail()
    torch.cuda.synchronize(dev)
    return out_ws, out_static, (x, wq, ws, bias)


def test_linear_static_matches_workspace_variant_twice(cuda_device):
    from q8_kernels_b200 import _lib
    lib = _lib.lib
    # first call: INT8 weights, Hadamard-rotated activations, bias + GELU
    from oracle import q8_oracle as O
    a, b, (x, wq, ws, bias) = _call_both(lib, _lib, cuda_device, 300, 2048, 512, torch.int8, True, True, seed=71)
    assert not torch.isnan(b.float()).any()
    assert torch.equal(a, b)                                   # same kernels, same inputs: identical bits
    assert Hp.rel_fro(b.float(), a.float()) <= 2e-3
    # and against the CPU oracle of the same chain (Hadamard, per-token INT8, GEMM, bias, tanh-GELU)
    want = O.q8_linear(x.cpu(), wq.cpu(), bias.cpu(), None, ws.cpu(), True, torch.bfloat16)[0]
    assert Hp.rel_fro(b.float(), want.float()) <= 2e-3
    # second call straight after, smaller and of the other kind: it runs over what the first left behind
    a2, b2, (x2, wq2, ws2, bias2) = _call_both(lib, _lib, cuda_device, 96, 256, 128, E4M3, False, False, seed=81)
    assert not torch.isnan(b2.float()).any()
    assert torch.equal(a2, b2)
    assert Hp.rel_fro(b2.float(), a2.float()) <= 2e-3
    want2 = O.fp8_linear(x2.cpu(), wq2.cpu(), bias2.cpu(), None, ws2.cpu(), False, torch.bfloat16)[0]
    assert Hp.rel_fro(b2.float(), want2.float()) <= 2e-3
    _lib.check_status(cuda_device)


@pytest.mark.parametrize("M,K,N", [(8192, 2048, 128), (65536, 64, 128)])
def test_linear_static_at_the_edge_of_its_capacity(cuda_device, M, K, N):
    """M*K equal to the scratch size (the quantised rows end exactly where the scale region begins)
    and M equal to the row limit (the scale region is full): same bits as the workspace variant."""
    from q8_kernels_b200 import _lib
    a, b, _ = _call_both(_lib.lib, _lib, cuda_device, M, K, N, torch.int8, True, False, seed=91)
    assert not torch.isnan(b.float()).any()
    assert torch.equal(a, b)
    _lib.check_status(cuda_device)


def test_linear_static_rejects_oversized_problems(cuda_device):
    from q8_kernels_b200 import _lib
    lib = _lib.lib
    buf = torch.zeros(4096, dtype=torch.uint8, device=cuda_device).data_ptr()
    # M*K beyond the built-in scratch: refused before anything is launched
    rc = lib.q8k_linear_static(buf, _lib.DT_BF16, buf, _lib.DT_I8, buf, None, buf, _lib.DT_BF16,
                               16384, 128, 2048, 1, 0, None, None)
    assert rc == -5
    assert b"built-in scratch" in lib.q8k_last_error_detail()
    # too many rows for the scale region
    rc = lib.q8k_linear_static(buf, _lib.DT_BF16, buf, _lib.DT_I8, buf, None, buf, _lib.DT_BF16,
                               70000, 128, 64, 1, 0, None, None)
    assert rc == -5
