"""Generate the golden fixtures in this folder by running the REFERENCE's own CPU oracle.

Run once, in a container that has the reference checkout (skywong14/htree) available:

    python tests/golden/make_golden.py /path/to/htree

It imports src/naive.py from that checkout (nothing is copied), runs htree_forward_naive(return_trace=True) and
HTreeFunction forward+backward on seeded inputs, and writes small .npz files.  The reference asserts
max_top_nodes == top_k*compression_rate, so it is always called with that value ("legal twin"); cases whose
`mtn_literal` is smaller describe how the new implementation will be called for the same expected result.

Input recipe (shared with the tests): CPU float32 torch.Generator().manual_seed(seed) -> q, k, v, dO in that order,
cast to the case dtype.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name: B,T,H,H_kv,K,V,CR,TK,mtn_literal,dtype,seed,backward
CASES = {
    # three pooled levels, ragged tails at every level (T not a multiple of CR), real eviction at two levels
    "f32_T300_cr4_tk8": dict(B=1, T=300, H=4, H_kv=2, K=16, V=16, CR=4, TK=8, MTN=32, dtype="float32", seed=0, bwd=True),
    # K != V, GQA group 4, batch 2
    "f32_T200_cr4_tk4_kv": dict(B=2, T=200, H=8, H_kv=2, K=32, V=16, CR=4, TK=4, MTN=16, dtype="float32", seed=1, bwd=True),
    # bf16 storage: pooled levels and outputs are rounded
    "bf16_T512_cr8_tk16": dict(B=1, T=512, H=8, H_kv=2, K=32, V=32, CR=8, TK=16, MTN=128, dtype="bfloat16", seed=2, bwd=True),
    # single level: T <= max_top_nodes -> dense causal attention
    "f32_T64_dense": dict(B=1, T=64, H=2, H_kv=1, K=16, V=16, CR=4, TK=16, MTN=64, dtype="float32", seed=3, bwd=True),
    # literal max_top_nodes smaller than top_k*CR: the implementation builds one more (pass-through) level
    "f32_T500_cr4_tk8_mtn16": dict(B=1, T=500, H=4, H_kv=2, K=16, V=16, CR=4, TK=8, MTN=16, dtype="float32", seed=4, bwd=True),
    # scaled-down twin of the CPU-runnable headline case (GQA group 4, D=64, CR=16, Top-K 32), forward only
    "f32_T1024_cr16_tk32": dict(B=1, T=1024, H=8, H_kv=2, K=64, V=64, CR=16, TK=32, MTN=64, dtype="float32", seed=5, bwd=False),
    "f16_T256_cr4_tk8": dict(B=1, T=256, H=4, H_kv=1, K=32, V=32, CR=4, TK=8, MTN=32, dtype="float16", seed=6, bwd=False),
}

TDT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def make_inputs(c):
    g = torch.Generator().manual_seed(c["seed"])
    q = torch.randn(c["B"], c["T"], c["H"], c["K"], generator=g)
    k = torch.randn(c["B"], c["T"], c["H_kv"], c["K"], generator=g)
    v = torch.randn(c["B"], c["T"], c["H_kv"], c["V"], generator=g)
    dO = torch.randn(c["B"], c["T"], c["H"], c["V"], generator=g)
    dt = TDT[c["dtype"]]
    return q.to(dt), k.to(dt), v.to(dt), dO.to(dt)


def main(ref_root: str) -> None:
    spec = importlib.util.spec_from_file_location("ref_naive", os.path.join(ref_root, "src", "naive.py"))
    naive = importlib.util.module_from_spec(spec)
    sys.modules["ref_naive"] = naive
    spec.loader.exec_module(naive)
    torch.set_num_threads(os.cpu_count() or 1)
    for name, c in CASES.items():
        q, k, v, dO = make_inputs(c)
        twin = c["TK"] * c["CR"]
        out, tr = naive.htree_forward_naive(q, k, v, c["CR"], twin, c["TK"], None, 10000.0, return_trace=True)
        L = tr["num_layers"]
        rec = dict(out=out.float().numpy(), num_layers=np.int32(L))
        for l, lt in tr["layers"].items():
            if lt.selected_parents is not None:
                rec[f"sel_{l}"] = lt.selected_parents.numpy()          # selection made at level l
            rec[f"lmax_{l}"] = lt.layer_max.numpy()
            rec[f"lsum_{l}"] = lt.layer_sum.numpy()
            if c["T"] <= 512:   # keep the fixtures small
                rec[f"lout_{l}"] = lt.layer_output.numpy().astype(np.float32)
        if c["bwd"]:
            qq, kk, vv = (x.clone().requires_grad_(True) for x in (q, k, v))
            o2 = naive.htree_forward_naive_autograd(qq, kk, vv, c["CR"], twin, c["TK"], None, 10000.0)
            assert torch.equal(o2, out)
            o2.backward(dO)
            rec.update(dq=qq.grad.float().numpy(), dk=kk.grad.float().numpy(), dv=vv.grad.float().numpy())
        cos, sin = naive._build_rope_cache(c["K"], twin + 1024, torch.device("cpu"), 10000.0)
        rec.update(cos_head=cos[:64].numpy(), cos_tail=cos[-8:].numpy(), sin_tail=sin[-8:].numpy())
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **rec)
        print(name, "levels", L, "out", tuple(out.shape), flush=True)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.environ.get("HTREE_REFERENCE", "../htree"))
