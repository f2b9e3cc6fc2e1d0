"""Shared helpers of the parity tests: seeded inputs, golden fixtures, selection comparison with the documented
near-tie rule, and error statistics in the reference's own protocol (p99 hard / max soft,
correctness_test_bwd.py:121-138 of skywong14/htree)."""
from __future__ import annotations

import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TDT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def make_inputs(B, T, H, H_kv, K, V, dtype, seed):
    """CPU float32 generator, q, k, v, dO drawn in that order, then cast (same recipe as tests/golden/make_golden.py)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, K, generator=g)
    k = torch.randn(B, T, H_kv, K, generator=g)
    v = torch.randn(B, T, H_kv, V, generator=g)
    dO = torch.randn(B, T, H, V, generator=g)
    dt = TDT[dtype]
    return q.to(dt), k.to(dt), v.to(dt), dO.to(dt)


def case_inputs(c):
    return make_inputs(c["B"], c["T"], c["H"], c["H_kv"], c["K"], c["V"], c["dtype"], c["seed"])


def golden_cases():
    import importlib.util
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLDEN_DIR, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.CASES


def load_golden(name):
    return np.load(os.path.join(GOLDEN_DIR, name + ".npz"))


def f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def compare_selections(ours: np.ndarray, ref: np.ndarray, importance: np.ndarray, ref_parents: np.ndarray, CR: int,
                       eps: float):
    """Compare the selections made at one level.

    ours, ref    [n, TK] int32 selected node ids (ascending, -1 padded), one row per group
    importance   [n, TK*CR] oracle importance by candidate position at that level (-1 = no candidate)
    ref_parents  [n, TK] the parent list the level consumed (oracle side); only meaningful where both sides consumed
                 the same list, which the caller guarantees by masking rows whose earlier levels differed
    Returns (n_exact, n_near_tie, n_bad).  A differing row is a documented near-tie iff every node that only one side
    kept has an oracle importance within eps (relative) of the boundary importance (the TK-th largest)."""
    n, TK = ref.shape
    exact = near = bad = 0
    for i in range(n):
        if np.array_equal(ours[i], ref[i]):
            exact += 1
            continue
        so, sr = set(ours[i][ours[i] >= 0].tolist()), set(ref[i][ref[i] >= 0].tolist())
        imp = importance[i]
        valid = imp >= 0
        node_of_pos = ref_parents[i][np.arange(imp.size) // CR].astype(np.int64) * CR + np.arange(imp.size) % CR
        pos_of_node = {int(node_of_pos[j]): j for j in np.nonzero(valid)[0]}
        srt = np.sort(imp[valid])[::-1]
        boundary = srt[min(TK, srt.size) - 1]
        ok = len(so) == len(sr)
        for node in so ^ sr:
            j = pos_of_node.get(int(node))
            if j is None or abs(float(imp[j]) - float(boundary)) > eps * float(boundary):
                ok = False
        if ok:
            near += 1
        else:
            bad += 1
    return exact, near, bad


def err_stats(a: np.ndarray, b: np.ndarray):
    d = np.abs(a.astype(np.float64) - b.astype(np.float64)).ravel()
    return dict(max=float(d.max()), p99=float(np.quantile(d, 0.99)), mean=float(d.mean()),
                rel=float(d.max() / max(1e-30, np.abs(b).max())))
