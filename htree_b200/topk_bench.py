"""Selector micro-benchmark: the k largest of n values, `batch` independent problems, 0 / 1 / 8 int32 payload words.

    python -m htree_b200.topk_bench [--n 8192] [--k 512] [--batch 512] [--reps 200]

Mirrors the experiment of the reference's topk_test/benchmark.py:34-46 (N=8192, K=512, BATCH=512; bitonic vs radix select
vs library) with CUDA kernels of this library (htree_b200_topk: threshold search, the selector the attention kernels use;
radix select; bitonic) and torch.topk as the library entry.  Prints one JSON line per (method, payload).
"""
from __future__ import annotations

import argparse
import json
from typing import Optional, Tuple

import torch

from . import _lib

METHODS = {"threshold_search": 0, "radix_select": 1, "bitonic": 2}


def topk(values: torch.Tensor, k: int, method: str = "threshold_search", pay1: Optional[torch.Tensor] = None,
         pay8: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, ...]:
    """values [batch, n] fp32 on a CUDA device -> (out_val [batch,k], out_idx [batch,k] int32, out_pay1, out_pay8)."""
    if not values.is_cuda or values.dtype != torch.float32 or not values.is_contiguous():
        raise ValueError("values must be a contiguous float32 CUDA tensor")
    batch, n = values.shape
    dev = values.device
    out_val = torch.empty(batch, k, dtype=torch.float32, device=dev)
    out_idx = torch.empty(batch, k, dtype=torch.int32, device=dev)
    out_pay1 = torch.empty(batch, k, dtype=torch.int32, device=dev) if pay1 is not None else None
    out_pay8 = torch.empty(batch, k, 8, dtype=torch.int32, device=dev) if pay8 is not None else None
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().htree_b200_topk(
            values.data_ptr(), pay1.data_ptr() if pay1 is not None else None,
            pay8.data_ptr() if pay8 is not None else None, batch, n, int(k), METHODS[method], out_val.data_ptr(),
            out_idx.data_ptr(), out_pay1.data_ptr() if out_pay1 is not None else None,
            out_pay8.data_ptr() if out_pay8 is not None else None, torch.cuda.current_stream().cuda_stream), "topk")
    return out_val, out_idx, out_pay1, out_pay8


def _time(fn, warmup: int, reps: int) -> Tuple[float, float, float]:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(reps):
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2], times[len(times) // 10], times[len(times) * 9 // 10]


def main(argv=None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=512)
    ap.add_argument("--batch", type=int, default=512)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--reps", type=int, default=200)
    args = ap.parse_args(argv)
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    for n_pay in (0, 1, 8):
        vals = torch.randn(args.batch, args.n, generator=g, device=dev)
        pay1 = torch.randint(0, 100000, (args.batch, args.n), generator=g, device=dev, dtype=torch.int32) if n_pay >= 1 else None
        pay8 = torch.randint(0, 100000, (args.batch, args.n, 8), generator=g, device=dev, dtype=torch.int32) if n_pay >= 8 else None
        ref_val, ref_idx = torch.topk(vals, args.k, dim=-1)
        ref_sorted = ref_idx.sort(dim=-1).values

        def library():
            v, i = torch.topk(vals, args.k, dim=-1)
            out = [v, i]
            if pay1 is not None:
                out.append(torch.gather(pay1, 1, i))
            if pay8 is not None:
                out.append(torch.gather(pay8, 1, i[:, :, None].expand(-1, -1, 8)))
            return out

        runs = {name: (lambda name=name: topk(vals, args.k, name, pay1, pay8)) for name in METHODS}
        runs["torch.topk (+ gather)"] = library
        for name, fn in runs.items():
            ok = None
            if name in METHODS:
                _, idx, _, _ = fn()
                ok = bool(torch.equal(idx.long().sort(dim=-1).values, ref_sorted))
            med, p10, p90 = _time(fn, args.warmup, args.reps)
            print(json.dumps({"method": name, "payload_words": n_pay, "n": args.n, "k": args.k, "batch": args.batch,
                              "median_ms": round(med, 4), "p10_ms": round(p10, 4), "p90_ms": round(p90, 4),
                              "same_set_as_torch": ok}), flush=True)


if __name__ == "__main__":
    main()
