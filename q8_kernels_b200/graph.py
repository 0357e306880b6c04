"""CUDA-graph replay of inference callables (reference: q8_kernels/graph/graph.py:384-401,461-510,
the auto-graph wrapper it applies to the transformer).

``graphed(fn)`` returns a callable with ``fn``'s signature.  The first call with a new input
signature (device / dtype / shape of every tensor argument, value of every other argument) runs
``fn`` eagerly on a side stream (lazy set-up, allocator warm-up), captures one more run into a CUDA
graph over static copies of the tensor arguments, and replays it; later calls with that signature
copy their tensors into the static buffers and replay.  Everything this package launches is
capturable: no allocation from the driver, no synchronisation, no host-side reads inside the ops.

Outputs are the graph's own static tensors: they are overwritten by the next call with the same
signature, exactly as with the reference's wrapper -- clone what must outlive the next call.
"""
from __future__ import annotations

import dataclasses
import functools
import threading
from typing import Any, Callable, Dict, Tuple

import torch


def hash_arg(arg) -> Any:
    """Hashable signature of one argument (q8_kernels/graph/graph.py:384-401): tensors by device,
    dtype and shape (one-element CPU tensors also by value), containers element-wise, scalars by
    value, anything else by type."""
    if isinstance(arg, torch.Tensor):
        dev = arg.device
        return (dev.type, dev.index, arg.dtype, tuple(arg.shape),
                arg.item() if dev.type == "cpu" and arg.numel() == 1 else None)
    if isinstance(arg, (str, int, float, bytes)) or arg is None:
        return arg
    if isinstance(arg, (tuple, list)):
        return tuple(hash_arg(a) for a in arg)
    if isinstance(arg, dict):
        return tuple(sorted(((hash_arg(k), hash_arg(v)) for k, v in arg.items()), key=lambda kv: repr(kv[0])))
    if dataclasses.is_dataclass(arg) and not isinstance(arg, type):
        return (type(arg),) + tuple(hash_arg(getattr(arg, f.name)) for f in dataclasses.fields(arg))
    return type(arg)


def _map_tensors(obj, fn: Callable[[torch.Tensor], Any]):
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, tuple):
        return tuple(_map_tensors(o, fn) for o in obj)
    if isinstance(obj, list):
        return [_map_tensors(o, fn) for o in obj]
    if isinstance(obj, dict):
        return {k: _map_tensors(v, fn) for k, v in obj.items()}
    return obj


def _flat_tensors(obj, out):
    if isinstance(obj, torch.Tensor):
        out.append(obj)
    elif isinstance(obj, (tuple, list)):
        for o in obj:
            _flat_tensors(o, out)
    elif isinstance(obj, dict):
        for v in obj.values():
            _flat_tensors(v, out)
    return out


class _Entry:
    __slots__ = ("graph", "static_args", "static_kwargs", "static_inputs", "outputs")


class GraphedCallable:
    """See the module docstring.  ``warmup`` eager runs precede each capture; ``pool`` lets several
    wrappers share one graph memory pool (``torch.cuda.graph_pool_handle()``).  ``check_status=True``
    makes every call synchronise and raise if a tensor-core kernel of the replay abandoned a bounded
    wait (``_lib.check_status``): outputs are undefined in that case.  Off by default, because it
    costs a device synchronisation per call."""

    def __init__(self, fn: Callable, warmup: int = 1, pool=None, check_status: bool = False):
        self.fn = fn
        self.warmup = max(1, int(warmup))
        self.pool = pool
        self.check_status = bool(check_status)
        self._entries: Dict[Tuple, _Entry] = {}
        self._lock = threading.Lock()
        functools.update_wrapper(self, fn.forward if isinstance(fn, torch.nn.Module) else fn)

    @property
    def num_graphs(self) -> int:
        return len(self._entries)

    def _capture(self, args, kwargs) -> _Entry:
        tensors = _flat_tensors((args, kwargs), [])
        cuda = [t for t in tensors if t.is_cuda]
        if not cuda:
            raise RuntimeError("graphed(): no CUDA tensor among the arguments")
        dev = cuda[0].device
        e = _Entry()
        # CUDA tensors get static copies; CPU tensors and scalars are baked in (they are part of the key)
        e.static_args, e.static_kwargs = _map_tensors((args, kwargs), lambda t: t.clone() if t.is_cuda else t)
        e.static_inputs = [t for t in _flat_tensors((e.static_args, e.static_kwargs), []) if t.is_cuda]
        with torch.cuda.device(dev), torch.no_grad():
            side = torch.cuda.Stream(dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(self.warmup):
                    self.fn(*e.static_args, **e.static_kwargs)
            torch.cuda.current_stream(dev).wait_stream(side)
            e.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(e.graph, pool=self.pool):
                e.outputs = self.fn(*e.static_args, **e.static_kwargs)
        return e

    def __call__(self, *args, **kwargs):
        key = (hash_arg(args), hash_arg(kwargs))
        with self._lock:
            e = self._entries.get(key)
            if e is None:
                e = self._entries[key] = self._capture(args, kwargs)
            live = [t for t in _flat_tensors((args, kwargs), []) if t.is_cuda]
            for dst, src in zip(e.static_inputs, live):
                if dst.data_ptr() != src.data_ptr():
                    dst.copy_(src)
            e.graph.replay()
            if self.check_status:
                from . import _lib
                _lib.check_status(e.static_inputs[0].device)
            return e.outputs


def graphed(fn: Callable, warmup: int = 1, pool=None, check_status: bool = False) -> GraphedCallable:
    return GraphedCallable(fn, warmup=warmup, pool=pool, check_status=check_status)


def apply_auto_graph(module: torch.nn.Module, filter_func: Callable[[torch.nn.Module], bool] = None,
                     recursive: bool = True, **kwargs) -> torch.nn.Module:
    """Replace ``forward`` of ``module`` (``recursive=False``) or of every sub-module accepted by
    ``filter_func`` (q8_kernels/graph/graph.py:503-510) with a graphed version."""
    targets = [module] if not recursive else [m for m in module.modules() if filter_func is None or filter_func(m)]
    for m in targets:
        if not isinstance(getattr(m, "forward", None), GraphedCallable):
            m.forward = GraphedCallable(m.forward, **kwargs)
    return module
