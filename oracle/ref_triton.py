"""Runner for the staged, unmodified reference (oracle/_ref/, see oracle/stage_reference.py).  TEST INFRASTRUCTURE ONLY.

Gives tests and the baseline legs of the benchmark access to the reference's own entry points:
    htree_forward                   src/parallel.py:874-1159   (Triton path, needs a CUDA device)
    htree_forward_triton_autograd   src/backward.py:1196-1208  (Triton forward + backward)
    htree_forward_naive             src/naive.py:133-234       (loop oracle, runs on the CPU)
The files are imported as they are.  `quiet(True)` swaps, in the loaded modules' namespaces only, the reference's
`_cuda_timer` (two device synchronisations and an INFO log line around every kernel, src/parallel.py:57-67) for a
no-op and raises its loggers to WARNING; timings are taken both ways ("as shipped" / "timer neutralised").
The product package never imports this module.
"""
from __future__ import annotations

import contextlib
import importlib
import logging
import os
import sys
import time
from types import SimpleNamespace
from typing import Optional, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")

_mods: Optional[SimpleNamespace] = None
_orig_timer = None


def available() -> Tuple[bool, str]:
    if not os.path.exists(os.path.join(REF, "src", "parallel.py")):
        return False, "oracle/_ref is empty (run oracle/stage_reference.py where the reference checkout exists)"
    return True, ""


def legal_max_top_nodes(top_k: int, compression_rate: int) -> int:
    """The only max_top_nodes the reference accepts (src/parallel.py:917-920): top_k * compression_rate."""
    return int(top_k) * int(compression_rate)


def load(need_triton: bool = True) -> SimpleNamespace:
    """Import the staged modules (cached).  need_triton=False loads only the CPU oracle src/naive.py."""
    global _mods, _orig_timer
    ok, why = available()
    if not ok:
        raise RuntimeError(why)
    if REF not in sys.path:
        sys.path.insert(0, REF)
    other = sys.modules.get("src")
    if other is not None and os.path.join(REF, "src") not in [os.path.abspath(p) for p in getattr(other, "__path__", [])]:
        raise RuntimeError("another top-level module named 'src' is already imported")
    if _mods is None:
        _mods = SimpleNamespace(naive=importlib.import_module("src.naive"), parallel=None, backward=None)
    if need_triton and _mods.parallel is None:
        _mods.parallel = importlib.import_module("src.parallel")
        _mods.backward = importlib.import_module("src.backward")
        _orig_timer = _mods.parallel._cuda_timer
    return _mods


@contextlib.contextmanager
def _no_timer(label: str):
    yield


def quiet(on: bool) -> None:
    """on: neutralise _cuda_timer and silence the INFO logging of the loaded reference modules; off: as shipped."""
    m = load()
    timer = _no_timer if on else _orig_timer
    m.parallel._cuda_timer = timer
    m.backward._cuda_timer = timer
    level = logging.WARNING if on else logging.INFO
    for mod in (m.parallel, m.backward):
        mod.logger.setLevel(level)


def silence_log_output() -> None:
    """Keep the reference's per-kernel INFO lines off stdout/stderr while it runs "as shipped" (the lines are still
    formatted and emitted by its logger; they go to a null handler)."""
    m = load()
    for mod in (m.parallel, m.backward):
        for h in list(mod.logger.handlers):
            mod.logger.removeHandler(h)
        mod.logger.addHandler(logging.NullHandler())
        mod.logger.propagate = False


def forward(q, k, v, compression_rate, top_k, scale=None, rope_base=10000.0, save=False):
    """Reference Triton forward at the legal max_top_nodes.  Returns out, or (out, bwd_ctx) with save=True."""
    m = load()
    return m.parallel.htree_forward(q, k, v, compression_rate=compression_rate,
                                    max_top_nodes=legal_max_top_nodes(top_k, compression_rate), top_k_per_layer=top_k,
                                    scale=scale, rope_base=rope_base, _save_for_backward=save)


def time_forward(q, k, v, compression_rate, top_k, warmup=2, iters=2):
    """Average forward latency in ms, the method of speed_test.py:73-96 (CUDA events around `iters` calls)."""
    import torch
    with torch.no_grad():
        for _ in range(max(warmup, 0)):
            forward(q, k, v, compression_rate, top_k)
        torch.cuda.synchronize()
        a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            forward(q, k, v, compression_rate, top_k)
        b.record()
        torch.cuda.synchronize()
    return a.elapsed_time(b) / max(iters, 1)


def time_forward_backward(q, k, v, dO, compression_rate, top_k, warmup=1, iters=1, wall_budget_s: float = 1e9):
    """(forward ms, backward ms, iterations done) of htree_forward_triton_autograd + .backward, the method of
    speed_test_bwd.py:78-125.  q, k, v must require grad.  Stops early when `wall_budget_s` of wall time is used up."""
    import torch
    m = load()
    mtn = legal_max_top_nodes(top_k, compression_rate)
    t_start = time.perf_counter()

    def fwd():
        return m.backward.htree_forward_triton_autograd(q, k, v, compression_rate=compression_rate, max_top_nodes=mtn,
                                                        top_k_per_layer=top_k)

    for _ in range(max(warmup, 1)):
        q.grad = k.grad = v.grad = None
        out = fwd()
        out.backward(dO)
        del out
    torch.cuda.synchronize()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    tf = tb = 0.0
    done = 0
    for _ in range(iters):
        q.grad = k.grad = v.grad = None
        ev[0].record()
        out = fwd()
        ev[1].record()
        out.backward(dO)
        ev[2].record()
        torch.cuda.synchronize()
        del out
        tf += ev[0].elapsed_time(ev[1]); tb += ev[1].elapsed_time(ev[2])
        done += 1
        if time.perf_counter() - t_start > wall_budget_s:
            break
    q.grad = k.grad = v.grad = None
    return tf / done, tb / done, done


def naive_forward(q, k, v, compression_rate, top_k, scale=None, rope_base=10000.0):
    """The reference's CPU loop oracle htree_forward_naive at the legal max_top_nodes (tensors on the CPU)."""
    m = load(need_triton=False)
    return m.naive.htree_forward_naive(q, k, v, compression_rate=compression_rate,
                                       max_top_nodes=legal_max_top_nodes(top_k, compression_rate),
                                       top_k_per_layer=top_k, scale=scale, rope_base=rope_base)


def time_naive(q, k, v, dO, compression_rate, top_k, runs=1):
    """Wall-clock seconds (forward, forward+backward) of the reference's CPU oracle: htree_forward_naive and
    htree_forward_naive_autograd + .backward (src/naive.py:133-234, 239-411); median of `runs`.  dO=None: forward only."""
    import statistics
    import torch
    m = load(need_triton=False)
    mtn = legal_max_top_nodes(top_k, compression_rate)
    tf, tfb = [], []
    for _ in range(runs):
        t0 = time.perf_counter()
        with torch.no_grad():
            m.naive.htree_forward_naive(q, k, v, compression_rate=compression_rate, max_top_nodes=mtn, top_k_per_layer=top_k)
        tf.append(time.perf_counter() - t0)
        if dO is not None:
            qq, kk, vv = (x.detach().clone().requires_grad_(True) for x in (q, k, v))
            t0 = time.perf_counter()
            out = m.naive.htree_forward_naive_autograd(qq, kk, vv, compression_rate=compression_rate, max_top_nodes=mtn,
                                                       top_k_per_layer=top_k)
            out.backward(dO)
            tfb.append(time.perf_counter() - t0)
    return statistics.median(tf), (statistics.median(tfb) if tfb else None)


def time_nsa(q, k, v, block_size=64, block_counts=16, warmup=2, iters=2):
    """Forward latency in ms of the NSA comparison baseline the reference ships (ref_nsa/, adapted from
    flash-linear-attention; staged unmodified), called as speed_test.py:261-270 calls it: the full pipeline (pooling,
    compression, selection, execution) with a zero compression gate.  Raises whatever its imports raise."""
    import torch
    if REF not in sys.path:
        sys.path.insert(0, REF)
    from ref_nsa.nsa_parallel import parallel_nsa
    B, T, HQ, K = q.shape
    gate = torch.zeros(B, T, HQ, device=q.device, dtype=q.dtype)
    scale = K ** -0.5

    def run():
        return parallel_nsa(q, k, v, g_cmp=gate, block_indices=None, block_size=block_size, scale=scale, block_counts=block_counts)

    with torch.no_grad():
        for _ in range(warmup):
            run()
        torch.cuda.synchronize()
        a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            run()
        b.record()
        torch.cuda.synchronize()
    return a.elapsed_time(b) / max(iters, 1)
