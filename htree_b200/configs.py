"""The benchmark / parity workloads (cfg1 .. cfg5: the configurations the reference is benchmarked and checked on) and their data-independent cost model.

Counts follow the expansion rule of the operator (src/naive.py:108-118, 182-190 of skywong14/htree): at level l a
query at position t scores nc_l(t) candidates and accumulates acc_l(t) of them; both depend only on t and the shape.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np

# name -> parameters.  `mode`: what the reference measures on it.  max_top_nodes is the literal value of the config
# (the reference itself would have to be called with top_k*compression_rate, which gives the same result).
CONFIGS: Dict[str, dict] = {
    "cfg1": dict(B=1, T=2048, H=8, H_kv=2, D=64, dtype="float32", CR=16, MTN=64, TK=32, mode="fwd"),
    "cfg2": dict(B=1, T=32768, H=32, H_kv=2, D=128, dtype="bfloat16", CR=16, MTN=128, TK=64, mode="fwd"),
    "cfg3": dict(B=4, T=65536, H=64, H_kv=4, D=128, dtype="bfloat16", CR=16, MTN=256, TK=64, mode="fwd+bwd"),
    "cfg4": dict(B=1, T=524288, H=32, H_kv=4, D=128, dtype="bfloat16", CR=16, MTN=512, TK=64, mode="fwd"),
    "cfg5": dict(B=2, T=16384, H=16, H_kv=2, D=64, dtype="bfloat16", CR=8, MTN=64, TK=64, mode="fwd+bwd", keys="clustered"),
    "cfg5_f32": dict(B=2, T=16384, H=16, H_kv=2, D=64, dtype="float32", CR=8, MTN=64, TK=64, mode="fwd+bwd", keys="clustered"),
}


def make_inputs(c: dict, device, seed: int = 42, want_dO: bool = True):
    """Seeded synthetic q, k, v (and dO) of a workload on `device`, in the operator's layouts [B,T,H,D] / [B,T,H_kv,D].
    All N(0,1) like the reference's benchmarks (speed_test.py:66-69); with keys="clustered" (the near-tie stress
    workload) the keys are N(0,1) plus a rank-4 component shared by all positions with N(0, std 3) coefficients."""
    import torch
    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}[c["dtype"]]
    g = torch.Generator(device=device).manual_seed(seed)
    B, T, H, Hkv, D = c["B"], c["T"], c["H"], c["H_kv"], c["D"]

    def randn(*shape):
        return torch.randn(*shape, generator=g, device=device, dtype=torch.float32)

    q = randn(B, T, H, D).to(tdt)
    k = randn(B, T, Hkv, D)
    if c.get("keys") == "clustered":
        k = k + (3.0 * randn(B, T, Hkv, 4)) @ randn(4, D)
    k = k.to(tdt)
    v = randn(B, T, Hkv, D).to(tdt)
    dO = randn(B, T, H, D).to(tdt) if want_dO else None
    return q, k, v, dO


def describe(c: dict) -> str:
    return (f"B={c['B']},T={c['T']},H_q={c['H']},H_kv={c['H_kv']},head_dim={c['D']},{c['dtype']},"
            f"compression_rate={c['CR']},max_top_nodes={c['MTN']},top_k={c['TK']},{c['mode']}")


def level_sizes(T: int, CR: int, MTN: int) -> List[int]:
    sizes, n = [int(T)], int(T)
    while n > MTN:
        n = (n + CR - 1) // CR
        sizes.append(n)
    return sizes


def attend_counts(T: int, CR: int, TK: int, L: int) -> Tuple[np.ndarray, np.ndarray]:
    """(nc [L,T], acc [L,T]): candidates scored / accumulated per level for every query position."""
    t = np.arange(T, dtype=np.int64)
    nc = np.zeros((L, T), np.int64)
    acc = np.zeros((L, T), np.int64)
    n_par = np.minimum(TK, (t // CR ** (L - 1)) // CR + 1)
    for l in range(L - 1, -1, -1):
        nc[l] = (n_par - 1) * CR + (t // CR ** l) % CR + 1
        if l > 0:
            n_par = np.minimum(TK, nc[l])
            acc[l] = nc[l] - n_par
        else:
            acc[l] = nc[l]
    return nc, acc


def cost_model(c: dict) -> dict:
    """Algorithmic FLOPs and compulsory HBM bytes of one forward / one backward over the whole workload.

    F_fwd = 2*G*B*H_kv*(K*sum nc + V*sum acc); F_bwd = B*H_kv*G*(6K+4V)*sum acc (selections saved);
    compulsory forward bytes = q and out once, leaves twice (tree build + attention), pooled levels three times,
    gmax/gsum once.  Padding, re-gathered rows and recomputation are not counted."""
    B, T, H, Hkv, D, CR, TK = c["B"], c["T"], c["H"], c["H_kv"], c["D"], c["CR"], c["TK"]
    G = H // Hkv
    es = 4 if c["dtype"] == "float32" else 2
    sizes = level_sizes(T, CR, c["MTN"])
    L = len(sizes)
    nc, acc = attend_counts(T, CR, TK, L)
    s_nc, s_acc = int(nc.sum()), int(acc.sum())
    f_fwd = 2 * G * B * Hkv * (D * s_nc + D * s_acc)
    f_bwd = B * Hkv * G * (6 * D + 4 * D) * s_acc
    upper = sum(sizes[1:])
    bytes_fwd = es * B * T * H * 2 * D + 2 * es * B * T * Hkv * 2 * D + 3 * es * B * Hkv * 2 * D * upper + 8 * B * T * H
    gather_fwd = es * B * Hkv * D * (s_nc + s_acc)
    # chunks (one parent's CR children) a (batch, position, kv head) group visits: the selection kernel scores the upper
    # levels that have more candidates than top_k; the accumulation kernel visits those again plus the leaves
    par = -(-nc // CR)
    sel_chunks = int(sum(par[l][nc[l] > TK].sum() for l in range(1, L)))
    acc_chunks = sel_chunks + int(par[0].sum())
    return dict(levels=sizes, flops_fwd=f_fwd, flops_bwd=f_bwd, bytes_fwd=bytes_fwd, gather_bytes_fwd=gather_fwd,
                scored_rows=s_nc * B * Hkv, accumulated_rows=s_acc * B * Hkv,
                selection_chunks=sel_chunks * B * Hkv, accumulation_chunks=acc_chunks * B * Hkv)
