"""Benchmark of the htree hot path: forward + backward tokens/s at T=64K bf16 (benchmark configuration "cfg3") on N GPUs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg3] [--t-scale S]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = tree build + forward + backward over the whole workload.  On one GPU the step runs on the operator's own
layouts, q/dO [B,T,H,D] and k/v [B,T,H_kv,D], through htree_forward / htree_backward.  On N > 1 GPUs the (batch, KV head)
units of the workload are dealt round-robin to the ranks (no data-path collective; each rank's slices are cut from the
full tensors in the untimed set-up); total work is fixed, so scaling is "strong".
Rank 0 prints ONE JSON line.  `value` times the step with inputs resident in HBM; `e2e` times the same step through the
public Python API with pinned HOST buffers (H2D of q,k,v,dO and D2H of out,dq,dk,dv inside the timed region).
`roofline` describes the slower of the two attention kernels.  Beside the headline the line carries
  workloads        the other benchmark configurations on one GPU (cfg2 and cfg4 forward, cfg5 bf16 / fp32 forward+backward)
  mode_b           (N > 1) cfg4 forward with the query positions split over the ranks and the pooled levels all-gathered
  triton_baseline  (N = 1) the unmodified reference's Triton path on the same GPU, when it has been staged under oracle/_ref
  nsa_baseline     (N = 1) the NSA comparison baseline the reference ships, timed beside the htree forward as its speed script does
  cpu_baseline     the reference's CPU oracle (src/naive.py, from oracle/_ref) at its own CPU-runnable configuration
                   cfg1, and the C port of it (oracle/) on a bounded sample of the headline workload
--impl reference times the unmodified reference itself on the headline workload: its Triton path on one GPU when it
is staged and a GPU is present, else the C port of its CPU oracle on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from htree_b200 import configs  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum per launch, one ncu capture) of the attention kernels on
# the default workload at a quarter of the sequence length (B=4, T=16384).  DRAM traffic grows in proportion to the number
# of (batch, position, kv head) groups, so the bench scales the figure by the ratio of groups.
NCU_TRAFFIC_BYTES_QUARTER_CFG3 = {"forward": (1.081223e9 + 0.191851e9) + (1.419880e9 + 1.077576e9),   # selection + accumulation
                                  "backward": 3.929301e9 + 2.410741e9,
                                  "capture": "kernels as of commit b82f34d"}

TDT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def es_bytes(c: dict) -> int:
    return 4 if c["dtype"] == "float32" else 2


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples of one GPU while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=self.file,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        self.file.flush(); self.file.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.file.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.file.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def measure_limits(device) -> dict:
    """Ceilings of the two on-chip memory paths the attention kernels live on, measured live with the kernels' own access
    patterns by the benchmark's probe library (htree_b200/csrc/bench/probes.cu): random 256-byte rows read from, and
    fp32 reductions into random 512-byte rows of, a 64 MiB buffer (L2-resident)."""
    import ctypes
    from htree_b200 import build as hbuild
    if not os.path.exists(hbuild.PROBES_LIB):
        return {"unavailable": "probe library not built"}
    L = ctypes.CDLL(hbuild.PROBES_LIB)
    for fn in (L.htree_probe_gather, L.htree_probe_reduction):
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.POINTER(ctypes.c_float), ctypes.c_void_p]
    buf = torch.zeros(64 << 20, dtype=torch.uint8, device=device)
    out = {}
    val = ctypes.c_float()
    st = torch.cuda.current_stream().cuda_stream
    if L.htree_probe_gather(buf.data_ptr(), buf.numel(), 5, ctypes.byref(val), st) == 0:
        out["l2_gather_gbs"] = float(val.value)
    if L.htree_probe_reduction(buf.data_ptr(), buf.numel(), 5, ctypes.byref(val), st) == 0:
        out["l2_reduction_gbs"] = float(val.value)
    del buf
    return out


# --------------------------------------------------------------------------------------------- CPU legs

def cpu_oracle_leg(c: dict, seconds: float, steps: int = 1, warmup: int = 0):
    """Time the C port of the reference's CPU oracle (oracle/) forward(+backward) on a bounded sample of the workload:
    groups (t, kv head 0, batch 0) with t uniform over the sequence, all host threads.  Returns (tokens/s, info)."""
    from oracle import oracle
    oracle.build()
    oracle.use_all_threads()
    T, D, G = c["T"], c["D"], c["H"] // c["H_kv"]
    rng = np.random.default_rng(42)

    def rnd(*shape):
        x = rng.standard_normal(shape, dtype=np.float32)
        return oracle.round_storage(x, c["dtype"])

    k = rnd(1, T, 1, D); v = rnd(1, T, 1, D)
    cache = oracle.rope_cache(D, c["TK"] * c["CR"] + 1024)
    bwd = "bwd" in c["mode"]

    def run(n):
        ts = np.sort(rng.integers(0, T, size=n)).astype(np.int32)
        queries = np.stack([np.zeros(n, np.int32), ts, np.zeros(n, np.int32)], 1)
        # only the sampled rows of q / dO are read; place them at their positions of a sparse [1,T,G,D] array
        qs = np.zeros((1, T, G, D), np.float32); qs[0, ts] = rnd(n, G, D)
        t0 = time.perf_counter()
        layers = oracle.build_tree(k, v, c["CR"], c["MTN"], c["dtype"])
        fw = oracle.forward(qs, k, v, c["CR"], c["MTN"], c["TK"], dtype=c["dtype"], queries=queries, layers=layers, cache=cache)
        if bwd:
            oracle.backward(qs, fw, rnd(n, G, D), c["CR"], c["TK"], c["dtype"], queries=queries)
        return time.perf_counter() - t0

    probe = 32
    per_group = run(probe) / probe
    n = int(max(64, min(8192, seconds / max(per_group, 1e-6))))
    times = []
    for i in range(warmup + steps):
        dt = run(n)
        if i >= warmup:
            times.append(dt)
    dt = statistics.median(times)
    tokens_per_s = n / (c["H_kv"] * dt)     # one token needs H_kv groups (and B*T tokens make the workload)
    info = dict(cores=oracle.max_threads(), kind="port",
                sample=f"{n} (t, kv-head) groups with t uniform in [0,{T}) of one (batch, kv head) unit, "
                       f"{'forward+backward' if bwd else 'forward'}, tree build included, median of {len(times)} run(s)",
                seconds_per_step=dt)
    return tokens_per_s, info


def naive_reference_leg(with_backward: bool = True) -> dict:
    """The reference's own CPU oracle (src/naive.py, staged unmodified under oracle/_ref) at its CPU-runnable
    configuration cfg1: B=1, T=2048, H=8, H_kv=2, D=64, fp32, compression_rate 16, top_k 32; called with the only
    max_top_nodes it accepts (top_k * compression_rate).  Wall clock on the host cores, all torch threads."""
    from oracle import ref_triton
    ok, why = ref_triton.available()
    if not ok:
        return {"unavailable": why}
    c = configs.CONFIGS["cfg1"]
    torch.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    g = torch.Generator().manual_seed(42)
    q = torch.randn(c["B"], c["T"], c["H"], c["D"], generator=g)
    k = torch.randn(c["B"], c["T"], c["H_kv"], c["D"], generator=g)
    v = torch.randn(c["B"], c["T"], c["H_kv"], c["D"], generator=g)
    dO = torch.randn(c["B"], c["T"], c["H"], c["D"], generator=g) if with_backward else None
    tf, tfb = ref_triton.time_naive(q, k, v, dO, c["CR"], c["TK"], runs=1)
    out = {"kind": "reference", "impl": "src/naive.py (htree_forward_naive, htree_forward_naive_autograd) from oracle/_ref",
           "workload": "cfg1: " + configs.describe(c), "cores": torch.get_num_threads(),
           "forward_s": tf, "forward_tokens_per_s": c["B"] * c["T"] / tf, "unit": "tokens/s"}
    if tfb is not None:
        out.update(forward_backward_s=tfb, forward_backward_tokens_per_s=c["B"] * c["T"] / tfb)
    return out


# --------------------------------------------------------------------------------------------- reference (Triton) legs

def triton_leg(c: dict, dev, fwd_bwd: bool, as_shipped: bool, warmup: int, iters: int, wall_budget_s: float) -> dict:
    """The unmodified reference's Triton path on one workload (legal max_top_nodes = top_k * compression_rate),
    timed by its own method (CUDA events; speed_test.py:73-96, speed_test_bwd.py:78-125)."""
    from oracle import ref_triton
    q, k, v, dO = configs.make_inputs(c, dev, seed=42, want_dO=fwd_bwd)
    ref_triton.quiet(not as_shipped)
    res = {"workload": configs.describe(c), "max_top_nodes_called": ref_triton.legal_max_top_nodes(c["TK"], c["CR"]),
           "variant": "as shipped (device synchronised and a log line emitted around every kernel)" if as_shipped
           else "_cuda_timer neutralised, logger at WARNING"}
    tokens = c["B"] * c["T"]
    if fwd_bwd:
        for x in (q, k, v):
            x.requires_grad_(True)
        f, b, n = ref_triton.time_forward_backward(q, k, v, dO, c["CR"], c["TK"], warmup=warmup, iters=iters,
                                                   wall_budget_s=wall_budget_s)
        res.update(forward_ms=f, backward_ms=b, ms=f + b, iterations=n, tokens_per_s=tokens / ((f + b) * 1e-3),
                   api="htree_forward_triton_autograd + .backward")
    else:
        ms = ref_triton.time_forward(q, k, v, c["CR"], c["TK"], warmup=warmup, iters=iters)
        res.update(forward_ms=ms, ms=ms, iterations=iters, tokens_per_s=tokens / (ms * 1e-3), api="htree_forward")
    ref_triton.quiet(True)
    del q, k, v, dO
    torch.cuda.empty_cache()
    return res


def triton_baseline(dev, ours: dict, budget_s: float) -> dict:
    """Reference Triton numbers beside ours on the same GPU.  `ours`: {"cfg2_fwd_ms", "cfg3_fwd_ms", "cfg3_fwdbwd_ms"}."""
    from oracle import ref_triton, stage_reference
    ok, why = ref_triton.available()
    if not ok:
        return {"unavailable": why}
    t_begin = time.perf_counter()
    out = {"source": "oracle/_ref (byte-identical copies of src/parallel.py, src/backward.py)",
           "files_unmodified": stage_reference.verify(), "legs": {}}
    try:
        import triton
        out["triton"] = triton.__version__
        ref_triton.load()
        ref_triton.silence_log_output()
        c2, c3 = dict(configs.CONFIGS["cfg2"]), dict(configs.CONFIGS["cfg3"])
        c3q = dict(c3, T=c3["T"] // 4)
        legs = out["legs"]
        legs["cfg2_fwd"] = triton_leg(c2, dev, False, False, 2, 2, budget_s)
        legs["cfg2_fwd_as_shipped"] = triton_leg(c2, dev, False, True, 1, 2, budget_s)
        legs["cfg3_fwd"] = triton_leg(c3, dev, False, False, 1, 2, budget_s)
        legs["cfg3_fwd_as_shipped"] = triton_leg(c3, dev, False, True, 0, 2, budget_s)
        legs["cfg3_quarter_fwdbwd"] = triton_leg(c3q, dev, True, False, 1, 1, budget_s)
        # the key-stationary dK/dV kernels loop over all T queries in every program: cost grows ~16x for 4x the length
        est_s = (legs["cfg3_quarter_fwdbwd"]["forward_ms"] * 4 + legs["cfg3_quarter_fwdbwd"]["backward_ms"] * 16) * 1e-3
        left = budget_s - (time.perf_counter() - t_begin)
        if est_s * 2.2 < left:
            legs["cfg3_fwdbwd"] = triton_leg(c3, dev, True, False, 1, 1, left)
            legs["cfg3_fwdbwd_as_shipped"] = triton_leg(c3, dev, True, True, 0, 1, left)
        else:
            legs["cfg3_fwdbwd"] = {"skipped": f"estimated {est_s:.0f} s per iteration from the quarter-length run; "
                                              f"{left:.0f} s of the budget left"}
        ratios = {}
        if ours.get("cfg2_fwd_ms"):
            ratios["cfg2_fwd"] = legs["cfg2_fwd"]["ms"] / ours["cfg2_fwd_ms"]
        if ours.get("cfg3_fwd_ms"):
            ratios["cfg3_fwd"] = legs["cfg3_fwd"]["ms"] / ours["cfg3_fwd_ms"]
        if ours.get("cfg3_fwdbwd_ms") and "ms" in legs.get("cfg3_fwdbwd", {}):
            ratios["cfg3_fwdbwd"] = legs["cfg3_fwdbwd"]["ms"] / ours["cfg3_fwdbwd_ms"]
        out["ours_over_triton"] = ratios     # speed ratio: reference time / our time on the same workload
    except Exception as e:   # a JIT failure of the reference must not lose the rest of the line
        out["error"] = f"{type(e).__name__}: {e}"[:500]
    out["seconds"] = time.perf_counter() - t_begin
    return out


def nsa_leg(dev, ours_cfg2_fwd_ms) -> dict:
    """The NSA comparison of the reference's speed script (speed_test.py:157-215, 261-270): its NSA baseline (ref_nsa/,
    staged unmodified; needs the flash-linear-attention package) timed beside the htree forward on the cfg2 tensors at
    its script's budget (16 selected blocks of 64 tokens + the compressed blocks).  A competitor baseline, not part of
    the operator; reported for completeness."""
    from oracle import ref_triton
    ok, why = ref_triton.available()
    if not ok:
        return {"unavailable": why}
    c = dict(configs.CONFIGS["cfg2"])
    try:
        q, k, v, _ = configs.make_inputs(c, dev, seed=42, want_dO=False)
        ms = ref_triton.time_nsa(q, k, v, block_size=64, block_counts=16, warmup=2, iters=2)
        res = {"workload": "cfg2 tensors: " + configs.describe(c), "nsa": "parallel_nsa(block_size=64, block_counts=16, zero compression gate)",
               "nsa_forward_ms": ms, "htree_forward_ms": ours_cfg2_fwd_ms,
               "htree_over_nsa": (ms / ours_cfg2_fwd_ms) if ours_cfg2_fwd_ms else None}
        del q, k, v
        torch.cuda.empty_cache()
        return res
    except Exception as e:
        return {"unavailable": f"{type(e).__name__}: {e}"[:400]}


# --------------------------------------------------------------------------------------------- GPU helpers

def time_gpu(fn, steps: int, warmup: int):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a = torch.cuda.Event(enable_timing=True); b = torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def side_workload(name: str, dev, pk: dict, steps: int = 3, warmup: int = 3) -> dict:
    """One of the other benchmark configurations on one GPU, inputs resident, operator layouts."""
    import htree_b200 as ht
    c = dict(configs.CONFIGS[name])
    bwd = "bwd" in c["mode"]
    q, k, v, dO = configs.make_inputs(c, dev, seed=42, want_dO=bwd)
    CR, MTN, TK = c["CR"], c["MTN"], c["TK"]
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    f_ms, b_ms = [], []

    def step(record=False):
        if record:
            ev[0].record()
        if bwd:
            out, ctx = ht.htree_forward(q, k, v, CR, MTN, TK, _save_for_backward=True)
            if record:
                ev[1].record()
            ht.htree_backward(dO, q, out, ctx)
        else:
            ht.htree_forward(q, k, v, CR, MTN, TK)
            if record:
                ev[1].record()
        if record:
            ev[2].record()
            torch.cuda.synchronize()
            f_ms.append(ev[0].elapsed_time(ev[1])); b_ms.append(ev[1].elapsed_time(ev[2]))

    for _ in range(warmup):
        step()
    for _ in range(steps):
        step(True)
    ht.check_status(dev)
    cm = configs.cost_model(c)
    fwd_ms = statistics.mean(f_ms)
    res = {"workload": f"{name}: {configs.describe(c)}", "steps": steps, "forward_ms": fwd_ms,
           "forward_tflops": cm["flops_fwd"] / (fwd_ms * 1e-3) / 1e12}
    ms = fwd_ms
    flops = cm["flops_fwd"]
    if bwd:
        bwd_ms = statistics.mean(b_ms)
        res.update(backward_ms=bwd_ms, backward_tflops=cm["flops_bwd"] / (bwd_ms * 1e-3) / 1e12)
        ms += bwd_ms
        flops += cm["flops_bwd"]
    peak = pk.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"])
    res.update(ms=ms, tokens_per_s=c["B"] * c["T"] / (ms * 1e-3), tflops=flops / (ms * 1e-3) / 1e12,
               roofline_frac=flops / (ms * 1e-3) / 1e12 / peak,
               arithmetic=("fp32 storage: split-half tensor-core kernels (64-wide heads; hi + lo half pairs, three MMAs per product)"
                           if c["dtype"] == "float32" else "bf16/half tensor cores"))
    del q, k, v, dO
    torch.cuda.empty_cache()
    return res


# --------------------------------------------------------------------------------------------- main

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg3", choices=sorted(configs.CONFIGS))
    ap.add_argument("--t-scale", type=int, default=1, help="divide T by this (debug only; reported in config)")
    ap.add_argument("--shard", default="auto", choices=["auto", "units", "sequence", "sequence-balanced"],
                    help="units: (batch, kv head) round-robin; sequence: query positions split, pooled levels all-gathered "
                         "(forward-only workloads); auto = sequence for cfg4, units otherwise")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--bind-host", action="store_true",
                    help="end-to-end leg: keep this rank on the CPUs next to its GPU before it allocates its pinned host buffers")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-workloads", action="store_true", help="skip the other configurations / mode B / Triton legs")
    ap.add_argument("--no-triton", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--triton-seconds", type=float, default=150.0)
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    c = dict(configs.CONFIGS[args.workload])
    if args.t_scale > 1:
        c["T"] //= args.t_scale
    metric = f"{'fwd+bwd' if 'bwd' in c['mode'] else 'fwd'} tokens/s at T={c['T']} {c['dtype']}"
    cfg_desc = {"workload": f"{args.workload}: {configs.describe(c)}",
                "l2": "inputs larger than L2 (q/dO/out exceed 126 MB on every rank); no explicit flush"}

    if args.impl == "reference":
        if rank != 0:
            return
        reference_arm(args, c, metric, cfg_desc)
        return

    import htree_b200 as ht
    from htree_b200 import _lib, dist as hdist, ops as hops

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback exists)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as tdist
        tdist.init_process_group("nccl", device_id=dev)
    tdt = TDT[c["dtype"]]

    B, T, H, Hkv, D, CR, TK, MTN = c["B"], c["T"], c["H"], c["H_kv"], c["D"], c["CR"], c["TK"], c["MTN"]
    G = H // Hkv
    bwd = "bwd" in c["mode"]
    seq_mode = (args.shard in ("sequence", "sequence-balanced") or (args.shard == "auto" and args.workload == "cfg4")) and not bwd
    seq_ranges = None
    units = list(range(B * Hkv))

    if seq_mode:
        # one long sequence per batch element: every rank holds the same k, v and its own slice of the queries
        cfg_desc["sharding"] = ("query positions split evenly over ranks; k, v replicated; one all_gather_into_tensor per "
                                "pooled tree level (NCCL)")
        q_full, k, v, _ = configs.make_inputs(c, dev, seed=42, want_dO=False)
        n_lv = len(configs.level_sizes(T, CR, MTN))
        if args.shard == "sequence-balanced" and world > 1:
            seq_ranges = hdist.balanced_query_ranges(T, world, CR, TK, MTN)
            t0, t1 = seq_ranges[rank]
            cfg_desc["sharding"] = cfg_desc["sharding"].replace("split evenly", "split by equal work (cost model)")
        else:
            t0, t1 = hdist.query_range(T, world, rank, CR, n_lv) if world > 1 else (0, T)
        q = q_full[:, t0:t1].contiguous() if world > 1 else q_full
        del q_full
        dO = None
        cfg_desc["tensors"] = f"per rank q [{B},{t1 - t0},{H},{D}], k/v [{B},{T},{Hkv},{D}]"
    else:
        q, k, v, dO = configs.make_inputs(c, dev, seed=42, want_dO=bwd)
        if world > 1:
            # this rank's (batch, KV head) units as a batch of single-KV-head problems, cut out here, outside the timing
            units = hdist.unit_partition(B * Hkv, world, rank)
            sl = hdist.gather_units(q, k, v, units, extra=[dO] if bwd else [])
            del q, k, v, dO
            q, k, v = sl[0], sl[1], sl[2]
            dO = sl[3] if bwd else None
            torch.cuda.empty_cache()
            cfg_desc["sharding"] = "(batch, kv head) units dealt round-robin to ranks, no collective"
            cfg_desc["tensors"] = (f"per rank q/dO [{len(units)},{T},{G},{D}], k/v [{len(units)},{T},1,{D}] (H_kv=1 per unit), "
                                   f"sliced from [{B},{T},{H},{D}] / [{B},{T},{Hkv},{D}] in the untimed set-up")
        else:
            cfg_desc["sharding"] = "one GPU: the whole workload"
            cfg_desc["tensors"] = f"q/dO [{B},{T},{H},{D}], k/v [{B},{T},{Hkv},{D}] (the operator's layouts), htree_forward + htree_backward"
    torch.cuda.empty_cache()

    def step(q_, k_, v_, dO_, timers=None):
        if timers is not None:
            timers[0].record()
        if bwd:
            out, ctx = ht.htree_forward(q_, k_, v_, CR, MTN, TK, _save_for_backward=True)
            if timers is not None:
                timers[1].record()
            dq, dk, dv = ht.htree_backward(dO_, q_, out, ctx)
            if timers is not None:
                timers[2].record()
            return out, dq, dk, dv
        if seq_mode and world > 1:
            out = hdist.htree_forward_sequence_parallel(q_, k_, v_, CR, MTN, TK, ranges=seq_ranges)
        else:
            out = ht.htree_forward(q_, k_, v_, CR, MTN, TK)
        if timers is not None:
            timers[1].record()
        return (out,)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            tdist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        tdist.all_reduce(t, op=tdist.ReduceOp.MAX)
        return float(t.item())

    for _ in range(max(3, args.warmup)):
        step(q, k, v, dO)
    barrier()

    # ---- resident-input timing ----
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    launches0 = _lib.launch_count()
    if sampler:
        sampler.start()
    barrier()
    t_begin = torch.cuda.Event(enable_timing=True); t_end = torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for i in range(args.steps):
        step(q, k, v, dO, ev[i])
    t_end.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    launches = _lib.launch_count() - launches0
    if world > 1:
        lt = torch.tensor([launches], device=dev, dtype=torch.float64)
        tdist.all_reduce(lt)
        launches = int(lt.item())
    ms_total = max_over_ranks(t_begin.elapsed_time(t_end))
    ms_step = ms_total / args.steps
    fwd_ms = max_over_ranks(statistics.mean(e[0].elapsed_time(e[1]) for e in ev))
    bwd_ms = max_over_ranks(statistics.mean(e[1].elapsed_time(e[2]) for e in ev)) if bwd else None
    ht.check_status(dev)

    # ---- the forward's two launches apart: the selection kernel alone (selection-only replay on the step's own tree) ----
    sel_ms = None
    if not (seq_mode and world > 1):
        _, fctx = ht.htree_forward(q, k, v, CR, MTN, TK, _save_for_backward=True)

        def select_only():
            return hops.recompute_parents(q, fctx["layers_k"], fctx["layers_v"], fctx["cos_cache"], fctx["sin_cache"], CR, TK, MTN,
                                          fctx["scale"], fctx["layers_k_rot"])

        select_only()
        torch.cuda.synchronize()
        s0 = torch.cuda.Event(enable_timing=True); s1 = torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(3):
            select_only()
        s1.record()
        torch.cuda.synchronize()
        sel_ms = max_over_ranks(s0.elapsed_time(s1) / 3)
        del fctx
        torch.cuda.empty_cache()

    # ---- streaming kernels: mean-pool tree build + key pre-rotation, timed alone (inputs larger than L2) ----
    sa = torch.cuda.Event(enable_timing=True); sb = torch.cuda.Event(enable_timing=True)
    hops.build_tree(k, v, CR, MTN, 10000.0)
    torch.cuda.synchronize()
    n_tb = 10
    sa.record()
    for _ in range(n_tb):
        hops.build_tree(k, v, CR, MTN, 10000.0)
    sb.record()
    torch.cuda.synchronize()
    tree_ms = sa.elapsed_time(sb) / n_tb

    # ---- end-to-end timing with host buffers ----
    e2e = None
    if not args.no_e2e:
        from htree_b200 import host as hhost
        affinity = hhost.bind_host_to_device(dev) if args.bind_host else None
        host_in = [x.cpu().pin_memory() for x in ((q, k, v, dO) if bwd else (q, k, v))]
        outs = step(q, k, v, dO)
        host_out = [torch.empty(o.shape, dtype=tdt, pin_memory=True) for o in outs]
        del outs

        from htree_b200 import host as hhost

        def e2e_step():
            if seq_mode:      # a single long sequence cannot be cut along the batch: plain copies around the call
                dev_in = [h.to(dev, non_blocking=True) for h in host_in]
                res = step(dev_in[0], dev_in[1], dev_in[2], None)
                host_out[0].copy_(res[0], non_blocking=True)
                torch.cuda.synchronize()
                return
            # one (batch, KV head) unit per pipeline stage (two in flight): strided copies out of / into the host tensors
            hhost.forward_backward_host(host_in[0], host_in[1], host_in[2], host_in[3] if bwd else None, CR, MTN, TK,
                                        chunk="unit", device=dev, outputs=host_out)

        e2e_step()
        barrier()
        ht.check_status(dev)
        n_e2e = max(1, min(args.steps, 3))
        a = torch.cuda.Event(enable_timing=True); b_ = torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_e2e):
            e2e_step()
        b_.record()
        barrier()
        e2e_ms = max_over_ranks(a.elapsed_time(b_)) / n_e2e
        h2d = sum(h.numel() * h.element_size() for h in host_in)
        d2h = sum(h.numel() * h.element_size() for h in host_out)
        if world > 1:
            tt = torch.tensor([h2d, d2h], device=dev, dtype=torch.float64)
            tdist.all_reduce(tt)
            h2d, d2h = int(tt[0].item()), int(tt[1].item())
        # the copy ceilings of this run: every rank moves its own inputs up and its own results down, all ranks at once,
        # nothing else running; e2e cannot be faster than the slower direction (or than the kernels)
        link = None
        try:
            dev_in = [torch.empty(h.shape, dtype=h.dtype, device=dev) for h in host_in]
            dev_out = [torch.empty(h.shape, dtype=h.dtype, device=dev) for h in host_out]
            for d_, h_ in zip(dev_in, host_in):
                d_.copy_(h_, non_blocking=True)
            barrier()
            ev_l = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev_l[0].record()
            for d_, h_ in zip(dev_in, host_in):
                d_.copy_(h_, non_blocking=True)
            ev_l[1].record()
            for d_, h_ in zip(dev_out, host_out):
                h_.copy_(d_, non_blocking=True)
            ev_l[2].record()
            barrier()
            up_ms = max_over_ranks(ev_l[0].elapsed_time(ev_l[1])); down_ms = max_over_ranks(ev_l[1].elapsed_time(ev_l[2]))
            # both directions at once (uploads on a second stream), as the pipeline runs them
            side = torch.cuda.Stream(dev)
            ev_d = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            barrier()
            side.wait_stream(torch.cuda.current_stream(dev))
            ev_d[0].record()
            with torch.cuda.stream(side):
                for d_, h_ in zip(dev_in, host_in):
                    d_.copy_(h_, non_blocking=True)
            for d_, h_ in zip(dev_out, host_out):
                h_.copy_(d_, non_blocking=True)
            torch.cuda.current_stream(dev).wait_stream(side)
            ev_d[1].record()
            barrier()
            both_ms = max_over_ranks(ev_d[0].elapsed_time(ev_d[1]))
            bytes_in = sum(h.numel() * h.element_size() for h in host_in)
            bytes_out = sum(h.numel() * h.element_size() for h in host_out)
            link = {"h2d_ms_all_ranks_at_once": up_ms, "d2h_ms_all_ranks_at_once": down_ms,
                    "both_directions_ms_all_ranks_at_once": both_ms,
                    "h2d_gbs_per_rank": bytes_in / (up_ms * 1e-3) / 1e9, "d2h_gbs_per_rank": bytes_out / (down_ms * 1e-3) / 1e9,
                    "note": "contiguous copies of this rank's pinned tensors, one direction at a time and both at once; max over ranks; "
                            "a step cannot be shorter than the both-directions time"}
            del dev_in, dev_out
        except Exception as e:
            link = {"error": f"{type(e).__name__}: {e}"[:200]}
        e2e = {"value": B * T / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms, "copy_ceiling": link,
               "host_affinity": affinity,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": n_e2e,
               "host_tensors": cfg_desc.get("tensors"),
               "api": ("htree_forward_sequence_parallel with pinned host tensors copied in and out around the call" if seq_mode
                       else "htree_b200.host.forward_backward_host: pinned host tensors in and out, (batch, KV head) "
                            "units pipelined over three streams (H2D | kernels | D2H), strided row copies")}
        del host_in, host_out

    # ---- mode B: cfg4 forward, query positions split over the ranks (measured on every rank, reported by rank 0) ----
    mode_b = None
    if world > 1 and not args.no_workloads and not seq_mode and args.t_scale == 1:
        del q, k, v, dO
        torch.cuda.empty_cache()
        try:
            mode_b = measure_mode_b(dev, world, rank, max_over_ranks, barrier)
        except Exception as e:     # every rank raises or none does (same code, same shapes): the headline survives
            mode_b = {"error": f"{type(e).__name__}: {e}"[:400]}

    if rank != 0:
        if world > 1:
            tdist.destroy_process_group()
        return

    pk = peaks()
    cm = configs.cost_model(c)
    dominant = "backward" if (bwd and bwd_ms > fwd_ms) else "forward"
    dom_ms = bwd_ms if dominant == "backward" else fwd_ms
    dom_flops = (cm["flops_bwd"] if dominant == "backward" else cm["flops_fwd"]) / world   # per launch on one rank
    peak_tf = pk.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"])
    achieved = dom_flops / (dom_ms * 1e-3) / 1e12
    roofline = {"kernel": f"{dominant} attention kernel(s) (all tree levels, one pass per step per rank)",
                "bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                "frac": achieved / peak_tf, "peak_source": f"{pk['_source']} bf16 dense, sustained",
                "traffic": (NCU_TRAFFIC_BYTES_QUARTER_CFG3[dominant] * (B * T * Hkv) / (4 * 16384 * 4) / world
                            if args.workload == "cfg3" else None),
                "traffic_source": (f"ncu capture at T=16384 ({NCU_TRAFFIC_BYTES_QUARTER_CFG3['capture']}) scaled by the number "
                                   "of groups") if args.workload == "cfg3" else None,
                "algorithmic_flops_per_launch": dom_flops,
                "forward_ms": fwd_ms, "backward_ms": bwd_ms,
                "forward_tflops": cm["flops_fwd"] / world / (fwd_ms * 1e-3) / 1e12,
                "backward_tflops": (cm["flops_bwd"] / world / (bwd_ms * 1e-3) / 1e12) if bwd else None,
                "forward_requested_gather_gbs": cm["gather_bytes_fwd"] / world / (fwd_ms * 1e-3) / 1e9,
                "forward_compulsory_hbm_frac": cm["bytes_fwd"] / world / (fwd_ms * 1e-3) / 1e9 / pk["hbm_gbs"]}
    # what actually bounds the two attention kernels: gathered rows per second (forward) and bytes of fp32 reductions
    # into the dK/dV level buffers per second (backward: 2 * D floats per accumulated row), against ceilings measured now
    limits = measure_limits(dev)
    if "l2_gather_gbs" in limits:
        limits["forward_gather_gbs"] = roofline["forward_requested_gather_gbs"]
        limits["forward_gather_frac"] = limits["forward_gather_gbs"] / limits["l2_gather_gbs"]
    if sel_ms is not None and "l2_gather_gbs" in limits and es_bytes(c) == 2 and D == 128 and CR == 16:
        # bytes the two kernels actually move from L2 per launch: the selection kernel gathers a chunk's pre-rotated keys
        # and reads its two fp32 table rows; the pipelined accumulation kernel copies a chunk's blocked keys, blocked
        # values and two packed-half table rows into shared memory
        acc_ms = fwd_ms - tree_ms - sel_ms
        sel_bytes = cm["selection_chunks"] / world * (CR * D * 2 + 2 * (D // 2) * 4)
        acc_bytes = cm["accumulation_chunks"] / world * (2 * CR * D * 2 + 2 * (D // 2) * 2)
        limits["selection_kernel_ms"] = sel_ms
        limits["accumulation_kernel_ms"] = acc_ms
        limits["selection_kernel_l2_gbs"] = sel_bytes / (sel_ms * 1e-3) / 1e9
        limits["accumulation_kernel_l2_gbs"] = acc_bytes / (acc_ms * 1e-3) / 1e9
        limits["selection_kernel_l2_frac"] = limits["selection_kernel_l2_gbs"] / limits["l2_gather_gbs"]
        limits["accumulation_kernel_l2_frac"] = limits["accumulation_kernel_l2_gbs"] / limits["l2_gather_gbs"]
    if bwd and "l2_reduction_gbs" in limits:
        red_bytes = cm["accumulated_rows"] * 2 * D * 4 / world
        limits["backward_reduction_gbs"] = red_bytes / (bwd_ms * 1e-3) / 1e9
        limits["backward_reduction_frac"] = limits["backward_reduction_gbs"] / limits["l2_reduction_gbs"]
    es = 4 if c["dtype"] == "float32" else 2
    lv_sizes = cm["levels"]
    n_rows = B * Hkv if (seq_mode or world == 1) else len(units)
    tree_bytes = es * n_rows * 2 * D * sum(lv_sizes[i] + lv_sizes[i + 1] for i in range(len(lv_sizes) - 1))     # pool K and V
    if es == 2:
        copies = 1 + (1 if D in (64, 128) and CR in (8, 16) else 0) + (1 if D == 128 and CR == 16 else 0)     # K -> K', V -> V^, K' -> K'^
        tree_bytes += copies * 2 * 2 * n_rows * D * sum(lv_sizes)                                                # each: read + write of every level
    streaming = {"kernels": "tree_build_kernel + rotate_keys / block_values / block_keys kernels (all levels, rank 0)", "ms": tree_ms,
                 "algorithmic_bytes": tree_bytes, "achieved": tree_bytes / (tree_ms * 1e-3) / 1e9, "unit": "GB/s",
                 "peak": pk["hbm_gbs"], "frac": tree_bytes / (tree_ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                 "note": "CUDA events around 10 back-to-back builds, includes launch gaps between the per-level kernels"}
    line = {"metric": metric, "value": B * T / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if c["dtype"] == "bfloat16" else c["dtype"],
            "data": "synthetic", "config": cfg_desc,
            "fwd_tokens_per_s": B * T / (fwd_ms * 1e-3), "roofline": roofline, "limits": limits, "streaming": streaming, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": clocks}
    if mode_b is not None:
        line["mode_b"] = mode_b

    if world == 1:
        if not seq_mode:
            del dO
        del q, k, v
        torch.cuda.empty_cache()
        ours = {}
        if args.workload == "cfg3" and args.t_scale == 1:
            ours.update(cfg3_fwd_ms=fwd_ms, cfg3_fwdbwd_ms=ms_step)
        if not args.no_workloads and args.t_scale == 1:
            wl = {}
            for name in ("cfg2", "cfg4", "cfg5", "cfg5_f32"):
                if name == args.workload:
                    continue
                try:
                    wl[name] = side_workload(name, dev, pk)
                except Exception as e:
                    wl[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
            line["workloads"] = wl
            if "forward_ms" in wl.get("cfg2", {}):
                ours["cfg2_fwd_ms"] = wl["cfg2"]["forward_ms"]
            if not args.no_triton:
                line["triton_baseline"] = triton_baseline(dev, ours, args.triton_seconds)
                line["nsa_baseline"] = nsa_leg(dev, ours.get("cfg2_fwd_ms"))
        if not args.no_cpu_baseline:
            tps, info = cpu_oracle_leg(c, args.cpu_seconds)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": info["cores"], "kind": info["kind"],
                                    "sample": info["sample"],
                                    "note": "C port (oracle/) of the reference's CPU oracle on a sample of the headline workload; "
                                            "the reference's own src/naive.py at its CPU-runnable configuration is `reference_cpu`"}
            try:
                line["cpu_baseline"]["reference_cpu"] = naive_reference_leg(with_backward=False)
            except Exception as e:
                line["cpu_baseline"]["reference_cpu"] = {"error": f"{type(e).__name__}: {e}"[:300]}
    print(json.dumps(line), flush=True)
    if world > 1:
        tdist.destroy_process_group()


def measure_mode_b(dev, world, rank, max_over_ranks, barrier) -> dict:
    """cfg4 forward through htree_forward_sequence_parallel: even and work-balanced split of the query positions; per
    step the max over ranks of CUDA-event times; the tree-build + all-gather (+ key rotation) part also timed alone."""
    from htree_b200 import dist as hdist, ops as hops
    c = dict(configs.CONFIGS["cfg4"])
    B, T, H, Hkv, D, CR, TK, MTN = c["B"], c["T"], c["H"], c["H_kv"], c["D"], c["CR"], c["TK"], c["MTN"]
    L = len(configs.level_sizes(T, CR, MTN))
    q_full, k, v, _ = configs.make_inputs(c, dev, seed=42, want_dO=False)
    out = {"workload": "cfg4: " + configs.describe(c), "n_gpus": world, "splits": {}}
    splits = {}
    try:
        splits["even"] = [hdist.query_range(T, world, r, CR, L) for r in range(world)]
    except ValueError as e:
        out["splits"]["even"] = {"unavailable": str(e)}
    splits["balanced"] = hdist.balanced_query_ranges(T, world, CR, TK, MTN)
    for name, ranges in splits.items():
        t0, t1 = ranges[rank]
        q = q_full[:, t0:t1].contiguous()

        def fwd():
            return hdist.htree_forward_sequence_parallel(q, k, v, CR, MTN, TK, ranges=ranges)

        def tree():
            lk, lv = hdist.build_tree_sequence_parallel(k, v, CR, MTN, ranges=ranges)
            hops.rotate_keys(lk, CR, MTN, 10000.0)

        for _ in range(3):
            fwd()
        barrier()
        ms = max_over_ranks(time_gpu(fwd, 3, 0))
        barrier()
        tree_ms = max_over_ranks(time_gpu(tree, 3, 1))
        barrier()
        out["splits"][name] = {"ms_per_step": ms, "tokens_per_s": B * T / (ms * 1e-3), "tree_allgather_rotate_ms": tree_ms,
                               "ranges": [list(r) for r in ranges]}
        del q
    del q_full, k, v
    torch.cuda.empty_cache()
    return out


def reference_arm(args, c, metric, cfg_desc):
    """--impl reference: the unmodified reference on the headline workload."""
    from oracle import ref_triton
    base = {"impl": "reference", "metric": metric, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "data": "synthetic",
            "config": cfg_desc}
    staged, why = ref_triton.available()
    bwd = "bwd" in c["mode"]
    triton_error = None
    if staged and torch.cuda.is_available():
        try:
            dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
            torch.cuda.set_device(dev)
            ref_triton.load()
            ref_triton.silence_log_output()
            budget = 200.0
            leg = triton_leg(c, dev, bwd, False, max(1, min(args.warmup, 2)), max(1, args.steps), budget)
            cpu = naive_reference_leg(with_backward=False)
            line = dict(base, value=leg["tokens_per_s"], ms_per_step=leg["ms"], dtype=c["dtype"] + " storage, TF32 tl.dot (Triton)",
                        steps_timed=leg["iterations"],
                        reference={"kind": "reference", "path": "Triton kernels of src/parallel.py + src/backward.py from oracle/_ref, "
                                   "one GPU (the reference has no multi-GPU path)", **leg},
                        cpu_baseline={"value": cpu.get("forward_tokens_per_s"), "unit": "tokens/s", "cores": cpu.get("cores"),
                                      "kind": "reference", "sample": "the reference's CPU oracle src/naive.py, forward, at its own "
                                      "CPU-runnable configuration " + str(cpu.get("workload")), "detail": cpu},
                        e2e={"value": leg["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
            print(json.dumps(line), flush=True)
            return
        except Exception as e:
            triton_error = f"{type(e).__name__}: {e}"[:400]
    n_iter = max(1, args.steps)
    budget = max(2.0, min(10.0, 150.0 / (n_iter + args.warmup + 1)))
    tps, info = cpu_oracle_leg(c, budget, steps=n_iter, warmup=args.warmup)
    line = dict(base, value=tps, ms_per_step=info["seconds_per_step"] * 1e3,
                dtype="f32 arithmetic on " + c["dtype"] + " values",
                cpu_baseline={"value": tps, "unit": "tokens/s", "cores": info["cores"], "kind": info["kind"],
                              "sample": info["sample"]},
                e2e={"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                note="CPU oracle arm: the C port (oracle/) of the reference's src/naive.py on all host threads; the "
                     "reference's Triton path was not run: " + (triton_error or why or "no CUDA device"))
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
