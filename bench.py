"""Benchmark of the htree hot path: forward + backward tokens/s at T=64K bf16 (benchmark configuration "cfg3") on N GPUs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg3] [--t-scale S]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One step = tree build + fused forward + backward over the whole workload.  The (batch, KV head) units of the workload
are dealt round-robin to the ranks (no data-path collective); total work is fixed, so scaling is "strong".
Rank 0 prints ONE JSON line.  `value` times the step with inputs resident in HBM; `e2e` times the same step through the
public Python API with pinned HOST buffers (H2D of q,k,v,dO and D2H of out,dq,dk,dv inside the timed region).
`roofline` describes the slower of the two attention kernels; `cpu_baseline` is the CPU oracle (a port of the
reference's naive path) on a bounded sample of the same workload.  --impl reference times that CPU port alone.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

from htree_b200 import configs  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM traffic per launch of the attention kernels at the default workload, from the ncu captures summarised under
# profiles/ (None until a capture exists for the kernel that is currently dominant).
# Measured with `ncu --set full` on the same workload at a quarter of the sequence length (profiles/*_cfg3_quarter.md);
# DRAM traffic grows in proportion to the number of (batch, position, kv head) groups, so the figure is scaled by the
# ratio of groups.  Values are dram__bytes_read.sum + dram__bytes_write.sum per launch for cfg3 / T=16384.
NCU_TRAFFIC_BYTES_QUARTER_CFG3 = {"forward": (1.081870e9 + 0.193277e9) + (1.421465e9 + 1.073665e9),   # selection + accumulation
                                  "backward": 3.897394e9 + 2.394069e9}


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


# --------------------------------------------------------------------------------------------- CPU oracle leg

def measure_limits(device) -> dict:
    """Ceilings of the two on-chip memory paths the attention kernels live on, measured live with the kernels' own access
    patterns (htree_b200_probe_gather / _probe_reduction): random 256-byte rows read from, and fp32 reductions into
    random 512-byte rows of, a 64 MiB buffer (L2-resident)."""
    import ctypes
    from htree_b200 import _lib
    buf = torch.zeros(64 << 20, dtype=torch.uint8, device=device)
    out = {}
    val = ctypes.c_float()
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib().htree_b200_probe_gather(buf.data_ptr(), buf.numel(), 5, ctypes.byref(val), st), "probe_gather")
    out["l2_gather_gbs"] = float(val.value)
    _lib.check(_lib.lib().htree_b200_probe_reduction(buf.data_ptr(), buf.numel(), 5, ctypes.byref(val), st), "probe_reduction")
    out["l2_reduction_gbs"] = float(val.value)
    del buf
    return out


def cpu_oracle_leg(c: dict, seconds: float, steps: int = 1, warmup: int = 0):
    """Time the CPU oracle (port of the reference's naive path) forward(+backward) on a bounded sample of the workload:
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


# --------------------------------------------------------------------------------------------- GPU leg

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
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    c = dict(configs.CONFIGS[args.workload])
    if args.t_scale > 1:
        c["T"] //= args.t_scale
    metric = f"{'fwd+bwd' if 'bwd' in c['mode'] else 'fwd'} tokens/s at T={c['T']} {c['dtype']}"
    cfg_desc = {"workload": f"{args.workload}: {configs.describe(c)}",
                "sharding": "(batch, kv head) units dealt round-robin to ranks, no collective",
                "l2": "inputs larger than L2 (per-rank q/dO/out exceed 126 MB); no explicit flush"}

    if args.impl == "reference":
        if rank != 0:
            return
        n_iter = max(1, args.steps)
        budget = max(2.0, min(10.0, 150.0 / (n_iter + args.warmup + 1)))
        tps, info = cpu_oracle_leg(c, budget, steps=n_iter, warmup=args.warmup)
        line = {"impl": "reference", "metric": metric, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": info["seconds_per_step"] * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f32 arithmetic on " + c["dtype"] + " values", "data": "synthetic", "config": cfg_desc,
                "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": info["cores"], "kind": info["kind"],
                                 "sample": info["sample"]},
                "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "note": "the reference's own CPU path is a Python loop (src/naive.py) that cannot travel to this box; "
                        "this arm times its C restatement (oracle/) on all host threads"}
        print(json.dumps(line), flush=True)
        return

    import htree_b200 as ht
    from htree_b200 import _lib, dist as hdist

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (no CPU fallback exists)"
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as tdist
        tdist.init_process_group("nccl", device_id=dev)
    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}[c["dtype"]]

    B, T, H, Hkv, D, CR, TK, MTN = c["B"], c["T"], c["H"], c["H_kv"], c["D"], c["CR"], c["TK"], c["MTN"]
    G = H // Hkv
    bwd = "bwd" in c["mode"]
    seq_mode = (args.shard in ("sequence", "sequence-balanced") or (args.shard == "auto" and args.workload == "cfg4")) and not bwd
    seq_ranges = None
    if seq_mode:
        cfg_desc["sharding"] = ("query positions split evenly over ranks; k, v replicated; one all_gather_into_tensor per "
                                "pooled tree level (NCCL)")
    units = hdist.unit_partition(B * Hkv, world, rank) if not seq_mode else list(range(B * Hkv))
    U = len(units)
    gen = torch.Generator(device=dev).manual_seed(42 + (0 if seq_mode else rank))

    def randn(*shape):
        return torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32).to(tdt)

    if seq_mode:
        # one long sequence per batch element: every rank holds the same k, v and its own slice of the queries
        k = randn(B, T, Hkv, D); v = randn(B, T, Hkv, D)
        n_lv = len(configs.level_sizes(T, CR, MTN))
        if args.shard == "sequence-balanced" and world > 1:
            seq_ranges = hdist.balanced_query_ranges(T, world, CR, TK, MTN)
            t0, t1 = seq_ranges[rank]
            cfg_desc["sharding"] = cfg_desc["sharding"].replace("split evenly", "split by equal work (cost model)")
        else:
            t0, t1 = hdist.query_range(T, world, rank, CR, n_lv) if world > 1 else (0, T)
        gen.manual_seed(1042 + rank)
        q = randn(B, t1 - t0, H, D)
        dO = None
    else:
        # local problem: U independent single-KV-head sequences
        q = randn(U, T, G, D); k = randn(U, T, 1, D); v = randn(U, T, 1, D)
        dO = randn(U, T, G, D) if bwd else None

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
        if seq_mode:
            out = hdist.htree_forward_sequence_parallel(q_, k_, v_, CR, MTN, TK, ranges=seq_ranges) if world > 1 else ht.htree_forward(q_, k_, v_, CR, MTN, TK)
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

    # ---- streaming kernels: mean-pool tree build + key pre-rotation, timed alone (inputs larger than L2) ----
    from htree_b200 import ops as hops
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
        host_in = [x.cpu().pin_memory() for x in ((q, k, v, dO) if bwd else (q, k, v))]
        outs = step(q, k, v, dO)
        res_dt = [tdt] * len(outs)
        host_out = [torch.empty(o.shape, dtype=d, pin_memory=True) for o, d in zip(outs, res_dt)]
        del outs

        from htree_b200 import host as hhost
        e2e_chunk = "unit"              # one (batch, KV head) unit per pipeline stage (two in flight): small head/tail

        def e2e_step():
            if seq_mode:      # a single long sequence cannot be cut along the batch: plain copies around the call
                dev_in = [h.to(dev, non_blocking=True) for h in host_in]
                res = step(dev_in[0], dev_in[1], dev_in[2], None)
                host_out[0].copy_(res[0], non_blocking=True)
                torch.cuda.synchronize()
                return
            hhost.forward_backward_host(host_in[0], host_in[1], host_in[2], host_in[3] if bwd else None, CR, MTN, TK,
                                        chunk=e2e_chunk, device=dev, outputs=host_out)

        e2e_step()
        barrier()
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
        e2e = {"value": B * T / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": n_e2e,
               "api": ("htree_forward_sequence_parallel with pinned host tensors copied in and out around the call" if seq_mode
                       else "htree_b200.host.forward_backward_host: pinned host tensors in and out, (batch, KV head) "
                            "units pipelined over three streams (H2D | kernels | D2H)")}
        del host_in, host_out

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
    roofline = {"kernel": f"fused {dominant} attention kernel (all tree levels, one launch per step per rank)",
                "bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
                "frac": achieved / peak_tf, "peak_source": f"{pk['_source']} bf16 dense, sustained",
                "traffic": (NCU_TRAFFIC_BYTES_QUARTER_CFG3[dominant] * (B * T * Hkv) / (4 * 16384 * 4) / world
                            if args.workload == "cfg3" else None),
                "traffic_source": "ncu capture at T=16384 scaled by the number of groups" if args.workload == "cfg3" else None,
                "algorithmic_flops_per_launch": dom_flops,
                "forward_ms": fwd_ms, "backward_ms": bwd_ms,
                "forward_tflops": cm["flops_fwd"] / world / (fwd_ms * 1e-3) / 1e12,
                "backward_tflops": (cm["flops_bwd"] / world / (bwd_ms * 1e-3) / 1e12) if bwd else None,
                "forward_requested_gather_gbs": cm["gather_bytes_fwd"] / world / (fwd_ms * 1e-3) / 1e9,
                "forward_compulsory_hbm_frac": cm["bytes_fwd"] / world / (fwd_ms * 1e-3) / 1e9 / pk["hbm_gbs"]}
    # what actually bounds the two attention kernels: gathered rows per second (forward) and bytes of fp32 reductions
    # into the dK/dV level buffers per second (backward: 2 * D floats per accumulated row), against ceilings measured now
    limits = measure_limits(dev)
    limits["forward_gather_gbs"] = roofline["forward_requested_gather_gbs"]
    limits["forward_gather_frac"] = limits["forward_gather_gbs"] / limits["l2_gather_gbs"]
    if bwd:
        red_bytes = cm["accumulated_rows"] * 2 * D * 4 / world
        limits["backward_reduction_gbs"] = red_bytes / (bwd_ms * 1e-3) / 1e9
        limits["backward_reduction_frac"] = limits["backward_reduction_gbs"] / limits["l2_reduction_gbs"]
    es = 4 if c["dtype"] == "float32" else 2
    lv_sizes = cm["levels"]
    n_rows = B * Hkv if seq_mode else U
    tree_bytes = es * n_rows * 2 * D * sum(lv_sizes[i] + lv_sizes[i + 1] for i in range(len(lv_sizes) - 1))     # pool K and V
    if es == 2:
        tree_bytes += 2 * 2 * n_rows * D * sum(lv_sizes)                                                         # K -> K'
    streaming = {"kernels": "tree_build_kernel + rotate_keys_kernel (all levels, rank 0)", "ms": tree_ms,
                 "algorithmic_bytes": tree_bytes, "achieved": tree_bytes / (tree_ms * 1e-3) / 1e9, "unit": "GB/s",
                 "peak": pk["hbm_gbs"], "frac": tree_bytes / (tree_ms * 1e-3) / 1e9 / pk["hbm_gbs"],
                 "note": "CUDA events around 10 back-to-back builds, includes launch gaps between the per-level kernels"}
    line = {"metric": metric, "value": B * T / (ms_step * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16" if c["dtype"] == "bfloat16" else c["dtype"],
            "data": "synthetic", "config": cfg_desc,
            "fwd_tokens_per_s": B * T / (fwd_ms * 1e-3), "roofline": roofline, "limits": limits, "streaming": streaming, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": clocks}
    if not args.no_cpu_baseline and world == 1:
        tps, info = cpu_oracle_leg(c, args.cpu_seconds)
        line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": info["cores"], "kind": info["kind"],
                                "sample": info["sample"]}
    print(json.dumps(line), flush=True)
    if world > 1:
        tdist.destroy_process_group()


if __name__ == "__main__":
    main()
