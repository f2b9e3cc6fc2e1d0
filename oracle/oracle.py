"""numpy/ctypes front-end of the CPU oracle (oracle/htree_oracle.c).  TEST INFRASTRUCTURE ONLY.

The shipped CUDA path never imports this module; it exists so that tests, the smoke check and the CPU-baseline leg
of the benchmark can evaluate the reference semantics (src/naive.py of skywong14/htree) on the host.

Every array is numpy float32.  Tensors whose storage type is bf16/fp16 are represented by float32 arrays holding
representable values; `dtype` ("float32" | "bfloat16" | "float16") tells the oracle where to apply storage rounding.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Dict, List, Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libhtree_oracle.so")
_DT = {"float32": 0, "bfloat16": 1, "float16": 2}
_lib = None


def build(force: bool = False) -> str:
    """Compile htree_oracle.c with gcc + OpenMP into oracle/_build/ (same recipe as oracle/Makefile)."""
    src = os.path.join(_HERE, "htree_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        os.makedirs(os.path.dirname(_SO), exist_ok=True)
        subprocess.check_call(["gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fPIC", "-shared", "-o", _SO, src, "-lm"])
    return _SO


class _Shape(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("B", "T", "H", "H_kv", "K", "V", "CR", "TK", "L", "n_pos")] + [
        ("scale", ctypes.c_float)]


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = ctypes.CDLL(_SO)
        _lib.ho_forward.restype = ctypes.c_int
        _lib.ho_backward.restype = ctypes.c_int
        _lib.ho_num_levels.restype = ctypes.c_int
        _lib.ho_max_threads.restype = ctypes.c_int
    return _lib


def _fp(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def max_threads() -> int:
    return int(_load().ho_max_threads())


def use_all_threads() -> int:
    """Run with one OpenMP thread per CPU this process may use, whatever OMP_NUM_THREADS says."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    _load().ho_set_threads(int(n))
    return max_threads()


def num_levels(T: int, CR: int, MTN: int) -> int:
    return int(_load().ho_num_levels(int(T), int(CR), int(MTN)))


def level_sizes(T: int, CR: int, MTN: int) -> List[int]:
    sizes, n = [int(T)], int(T)
    while n > MTN:
        n = (n + CR - 1) // CR
        sizes.append(n)
    return sizes


def round_storage(a: np.ndarray, dtype: str) -> np.ndarray:
    """Round a float32 array to values representable in `dtype` (round-to-nearest-even), still as float32."""
    out = _f32(a).copy()
    _load().ho_round(_fp(out), ctypes.c_int64(out.size), _DT[dtype])
    return out


def rope_cache(K: int, n_pos: int, rope_base: float = 10000.0):
    """cos/sin tables [n_pos, K/2] in float32 arithmetic, as src/naive.py:63-70 computes them.

    float32 pow/cos of numpy and torch differ in the last bit for some entries, and the angle pos*inv_freq is rounded
    to float32 before the cosine, so a one-ulp change of inv_freq moves angles of large positions visibly.  When torch
    is importable its CPU float32 kernels are used, which makes the tables bit-identical to the reference's; the numpy
    fallback agrees to within a few ulp of the angle."""
    try:
        import torch
        inv_freq = 1.0 / (rope_base ** (torch.arange(0, K, 2, dtype=torch.float32) / K))
        freqs = torch.outer(torch.arange(n_pos, dtype=torch.float32), inv_freq)
        return freqs.cos().numpy(), freqs.sin().numpy()
    except ImportError:
        expo = np.arange(0, K, 2, dtype=np.float32) / np.float32(K)
        inv_freq = (np.float32(1.0) / np.power(np.float32(rope_base), expo, dtype=np.float32)).astype(np.float32)
        freqs = np.outer(np.arange(n_pos, dtype=np.float32), inv_freq).astype(np.float32)
        return np.cos(freqs).astype(np.float32), np.sin(freqs).astype(np.float32)


def build_tree(k: np.ndarray, v: np.ndarray, CR: int, MTN: int, dtype: str = "float32"):
    """Mean-pool tree (src/naive.py:41-60).  Returns (layers_k, layers_v), level 0 = the inputs."""
    lib = _load()
    lk, lv = [_f32(k)], [_f32(v)]
    B, n, Hkv, K = lk[0].shape
    V = lv[0].shape[-1]
    while n > MTN:
        npar = (n + CR - 1) // CR
        pk = np.empty((B, npar, Hkv, K), np.float32)
        pv = np.empty((B, npar, Hkv, V), np.float32)
        lib.ho_build_level(_fp(lk[-1]), _fp(pk), B, n, Hkv, K, CR, _DT[dtype])
        lib.ho_build_level(_fp(lv[-1]), _fp(pv), B, n, Hkv, V, CR, _DT[dtype])
        lk.append(pk); lv.append(pv); n = npar
    return lk, lv


def _ptr_array(arrs: Sequence[np.ndarray]):
    return (ctypes.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])


def forward(q, k, v, compression_rate=16, max_top_nodes=8192, top_k_per_layer=512, scale=None, rope_base=10000.0,
            dtype="float32", queries=None, return_trace=False, layers=None, cache=None,
            return_importance=False) -> Dict[str, np.ndarray]:
    """htree forward on the host.  Mirrors htree_forward_naive (src/naive.py:133-234).

    `max_top_nodes` may be smaller than top_k*compression_rate (the reference asserts equality; the extra top levels
    this creates select every candidate, so results equal the reference called with max_top_nodes = top_k*CR
    whenever both are defined).  `queries`: optional int32 [nq,3] array of (b, t, h_kv) groups; default all groups.
    Returns dict: out [nq,G,V] (un-rounded), out_rounded, gmax, gsum [nq,G], parents [L,nq,TK], gap [L,nq],
    importance [L,nq,TK*CR] with return_importance, and,
    with return_trace, tr_max/tr_sum [L,nq,G], tr_out [L,nq,G,V].  With queries=None the arrays are reshaped to the
    reference layouts ([B,T,H,V] etc.).
    """
    lib = _load()
    q = _f32(q)
    B, T, H, K = q.shape
    lk, lv = layers if layers is not None else build_tree(k, v, compression_rate, max_top_nodes, dtype)
    Hkv, V = lk[0].shape[2], lv[0].shape[3]
    G, L, TK, CR = H // Hkv, len(lk), int(top_k_per_layer), int(compression_rate)
    assert H % Hkv == 0 and K % 2 == 0 and G <= 64
    assert lk[-1].shape[1] <= TK * CR, "top level must fit into top_k*compression_rate candidates"
    if scale is None:
        scale = K ** -0.5
    n_pos = TK * CR + 1024
    cosc, sinc = cache if cache is not None else rope_cache(K, n_pos, rope_base)
    sh = _Shape(B, T, H, Hkv, K, V, CR, TK, L, cosc.shape[0], float(scale))
    level_n = np.array([a.shape[1] for a in lk], np.int32)
    if queries is None:
        qarr, nq = None, B * T * Hkv
    else:
        qarr = np.ascontiguousarray(queries, np.int32).reshape(-1, 3); nq = qarr.shape[0]
    out = np.empty((nq, G, V), np.float32)
    gmax = np.empty((nq, G), np.float32); gsum = np.empty((nq, G), np.float32)
    parents = np.empty((L, nq, TK), np.int32)
    gap = np.empty((L, nq), np.float32)
    tr_max = tr_sum = tr_out = None
    if return_trace:
        tr_max = np.empty((L, nq, G), np.float32); tr_sum = np.empty((L, nq, G), np.float32)
        tr_out = np.empty((L, nq, G, V), np.float32)
    imp = np.empty((L, nq, TK * CR), np.float32) if return_importance else None
    rc = lib.ho_forward(ctypes.byref(sh), _fp(q), _ptr_array(lk), _ptr_array(lv), _fp(level_n), _fp(cosc), _fp(sinc),
                        _fp(qarr), ctypes.c_int64(nq), _fp(out), _fp(gmax), _fp(gsum), _fp(parents), _fp(tr_max),
                        _fp(tr_sum), _fp(tr_out), _fp(gap), _fp(imp))
    if rc != 0:
        raise RuntimeError(f"oracle forward failed with status {rc}")
    res = dict(out=out, out_rounded=round_storage(out, dtype), gmax=gmax, gsum=gsum, parents=parents, gap=gap,
               layers_k=lk, layers_v=lv, cos=cosc, sin=sinc, num_layers=L, scale=float(scale))
    if return_trace:
        res.update(tr_max=tr_max, tr_sum=tr_sum, tr_out=tr_out)
    if return_importance:
        res["importance"] = imp        # [L, nq, TK*CR], always indexed by flat group number
    if queries is None:
        res["out"] = out.reshape(B, T, H, V); res["out_rounded"] = res["out_rounded"].reshape(B, T, H, V)
        res["gmax"] = gmax.reshape(B, T, H); res["gsum"] = gsum.reshape(B, T, H)
        res["parents"] = parents.reshape(L, B, T, Hkv, TK); res["gap"] = gap.reshape(L, B, T, Hkv)
        if return_trace:
            res["tr_max"] = tr_max.reshape(L, B, T, H); res["tr_sum"] = tr_sum.reshape(L, B, T, H)
            res["tr_out"] = tr_out.reshape(L, B, T, H, V)
    return res


def backward(q, fwd: Dict[str, np.ndarray], dO, compression_rate=16, top_k_per_layer=512, dtype="float32",
             queries=None):
    """Analytical backward (src/naive.py:321-396) given a forward() result.

    queries=None: `fwd` must be a full-tensor result; returns dq, dk, dv rounded to `dtype` like the reference's
    autograd function, plus the un-rounded fp32 versions (dq_f32, ...).
    queries [nq,3]: `fwd` must come from forward(queries=...) with the same list and dO is [nq,G,V]; returns dq_f32
    [nq,G,K] for those groups and the partial dk_f32/dv_f32 they contribute (before the mean-pool step)."""
    lib = _load()
    q = _f32(q); dO = _f32(dO)
    B, T, H, K = q.shape
    lk, lv = fwd["layers_k"], fwd["layers_v"]
    Hkv, V, L = lk[0].shape[2], lv[0].shape[3], len(lk)
    G = H // Hkv
    sh = _Shape(B, T, H, Hkv, K, V, int(compression_rate), int(top_k_per_layer), L, fwd["cos"].shape[0], fwd["scale"])
    level_n = np.array([a.shape[1] for a in lk], np.int32)
    out_st = _f32(fwd["out_rounded"])
    dks = [np.zeros_like(a) for a in lk]; dvs = [np.zeros_like(a) for a in lv]
    parents = np.ascontiguousarray(fwd["parents"], np.int32)
    if queries is None:
        qarr, nq = None, B * T * Hkv
        dq = np.zeros_like(q)
    else:
        qarr = np.ascontiguousarray(queries, np.int32).reshape(-1, 3); nq = qarr.shape[0]
        dq = np.zeros((nq, G, K), np.float32)
    rc = lib.ho_backward(ctypes.byref(sh), _fp(q), _ptr_array(lk), _ptr_array(lv), _fp(level_n), _fp(fwd["cos"]),
                         _fp(fwd["sin"]), _fp(qarr), ctypes.c_int64(nq), _fp(out_st), _fp(dO), _fp(_f32(fwd["gmax"])),
                         _fp(_f32(fwd["gsum"])), _fp(parents), _fp(dq), _ptr_array(dks), _ptr_array(dvs))
    if rc != 0:
        raise RuntimeError(f"oracle backward failed with status {rc}")
    if queries is not None:
        return dict(dq_f32=dq, dk_levels=dks, dv_levels=dvs)
    for l in range(L - 1, 0, -1):
        n_child = lk[l - 1].shape[1]
        lib.ho_tree_backward_level(_fp(dks[l]), _fp(dks[l - 1]), B, n_child, Hkv, K, int(compression_rate))
        lib.ho_tree_backward_level(_fp(dvs[l]), _fp(dvs[l - 1]), B, n_child, Hkv, V, int(compression_rate))
    return dict(dq=round_storage(dq, dtype), dk=round_storage(dks[0], dtype), dv=round_storage(dvs[0], dtype),
                dq_f32=dq, dk_f32=dks[0], dv_f32=dvs[0])


def attend_counts(T: int, CR: int, TK: int, L: int):
    """Data-independent per-query candidate / accumulation counts per level (closed form of the expansion rule).
    Returns (nc [L,T], acc [L,T]) int64: candidates scored and candidates accumulated at each level."""
    t = np.arange(T, dtype=np.int64)
    nc = np.zeros((L, T), np.int64); acc = np.zeros((L, T), np.int64)
    n_par = np.minimum(TK, (t // CR ** (L - 1)) // CR + 1)
    for l in range(L - 1, -1, -1):
        nc[l] = (n_par - 1) * CR + (t // CR ** l) % CR + 1
        if l > 0:
            n_par = np.minimum(TK, nc[l]); acc[l] = nc[l] - n_par
        else:
            acc[l] = nc[l]
    return nc, acc
