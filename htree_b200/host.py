"""Host-buffer entry points: inputs and results live in (pinned) host memory, the device only holds a window of them.

The reference has no counterpart (its scripts create tensors on the device, speed_test.py:66-69).  These functions are
what a caller with host-resident activations uses: the batch dimension is cut into chunks, and three CUDA streams
overlap the host->device copy of chunk i+1, the kernels of chunk i and the device->host copy of chunk i-1.  Chunks are
independent because every batch element is (htree_forward/htree_backward never mix batch elements)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib, ops


_stream_cache = {}


def _streams(dev):
    """Three streams per device, created once: the caching allocator keeps one pool per stream, so fresh streams on
    every call would mean fresh cudaMalloc calls (which synchronise the device) on every call."""
    key = (dev.type, dev.index)
    if key not in _stream_cache:
        _stream_cache[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return _stream_cache[key]


def bind_host_to_device(device) -> Optional[dict]:
    """Restrict the calling process to the CPUs next to `device` (the `local_cpulist` of its PCI function in sysfs), so
    that host memory it allocates and first touches afterwards - pinned staging buffers above all - lands on the NUMA
    node the GPU hangs off.  With several ranks per host, copies from the far node share the inter-socket link.
    Returns {"cpus": n, "numa_node": k} or None where the information is not available; never raises."""
    import os
    try:
        dev = torch.device(device)
        idx = dev.index if dev.index is not None else torch.cuda.current_device()
        pr = torch.cuda.get_device_properties(idx)
        bdf = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        base = f"/sys/bus/pci/devices/{bdf}"
        with open(base + "/local_cpulist") as f:
            spec = f.read().strip()
        cpus = set()
        for part in spec.split(","):
            if "-" in part:
                a, b = part.split("-")
                cpus.update(range(int(a), int(b) + 1))
            elif part:
                cpus.add(int(part))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        node = None
        try:
            with open(base + "/numa_node") as f:
                node = int(f.read().strip())
        except (OSError, ValueError):
            pass
        return {"cpus": len(cpus), "numa_node": node}
    except Exception:
        return None


def _copy_unit(dst: torch.Tensor, src: torch.Tensor, stream) -> None:
    """dst <- src for two views of shape [1, T, heads, D] whose rows (one position: heads * D elements) are contiguous;
    either side may be a slice of a larger [B, T, H, D] tensor (rows a fixed pitch apart) in pinned host memory."""
    assert dst.shape == src.shape and dst.dtype == src.dtype
    T, es = dst.shape[1], dst.element_size()
    width = dst.shape[2] * dst.shape[3] * es
    for x in (dst, src):
        assert x.stride(3) == 1 and x.stride(2) == x.shape[3], "rows must be contiguous"
    _lib.check(_lib.lib().htree_b200_copy_rows(dst.data_ptr(), dst.stride(1) * es, src.data_ptr(), src.stride(1) * es, width, T,
                                               stream.cuda_stream), "copy_rows")


def forward_backward_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, dO: Optional[torch.Tensor],
                          compression_rate: int = 16, max_top_nodes: int = 8192, top_k_per_layer: int = 512,
                          scale: Optional[float] = None, rope_base: float = 10000.0, chunk: int = 1,
                          device=None, outputs: Optional[Tuple[torch.Tensor, ...]] = None):
    """htree forward (and backward when dO is given) for HOST tensors q [B,T,H,K], k, v [B,T,H_kv,*], dO [B,T,H,V].

    Returns host tensors (out,) or (out, dq, dk, dv) in the input dtype; pass `outputs` (pinned, same shapes) to reuse
    buffers.  `chunk` batch elements are resident on the device at a time (two chunks in flight).  The call returns
    after everything has arrived in host memory.  chunk="unit" moves and computes one (batch, KV head) unit at a time
    (strided copies of that head group's slices): the units are independent too, and the smaller the piece the less of
    the first upload and the last download is left outside the overlap."""
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    B = q.shape[0]
    bwd = dO is not None
    if outputs is None:
        pin = q.is_pinned()
        outs = [torch.empty((B,) + tuple(q.shape[1:3]) + (v.shape[-1],), dtype=q.dtype, pin_memory=pin)]
        if bwd:
            outs += [torch.empty(q.shape, dtype=q.dtype, pin_memory=pin), torch.empty(k.shape, dtype=k.dtype, pin_memory=pin),
                     torch.empty(v.shape, dtype=v.dtype, pin_memory=pin)]
    else:
        outs = list(outputs)
    s_in, s_run, s_out = _streams(dev)
    s_in.wait_stream(torch.cuda.current_stream(dev))
    if chunk == "unit":
        return _by_units(q, k, v, dO, outs, dev, (s_in, s_run, s_out), compression_rate, max_top_nodes, top_k_per_layer, scale,
                         rope_base)
    keep = []                      # device tensors stay referenced until the final synchronisation
    for b0 in range(0, B, chunk):
        b1 = min(B, b0 + chunk)
        with torch.cuda.stream(s_in):
            dev_in = [x[b0:b1].to(dev, non_blocking=True) for x in ((q, k, v, dO) if bwd else (q, k, v))]
            ready = torch.cuda.Event(); ready.record(s_in)
        with torch.cuda.stream(s_run):
            s_run.wait_event(ready)
            if bwd:
                o, ctx = ops.htree_forward(dev_in[0], dev_in[1], dev_in[2], compression_rate, max_top_nodes,
                                           top_k_per_layer, scale, rope_base, _save_for_backward=True)
                dq, dk, dv = ops.htree_backward(dev_in[3], dev_in[0], o, ctx, _typed=True)
                res = [o, dq, dk, dv]
                del ctx
            else:
                res = [ops.htree_forward(dev_in[0], dev_in[1], dev_in[2], compression_rate, max_top_nodes,
                                         top_k_per_layer, scale, rope_base)]
            done = torch.cuda.Event(); done.record(s_run)
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            for h, r in zip(outs, res):
                h[b0:b1].copy_(r, non_blocking=True)
        for t in dev_in + res:     # the caching allocator must not hand these blocks to another stream early
            t.record_stream(s_run); t.record_stream(s_out)
        keep.append((dev_in, res))
        if len(keep) > 2:
            keep.pop(0)
    s_out.synchronize(); s_run.synchronize(); s_in.synchronize()
    return tuple(outs)


EDGE_WINDOWS = 4          # query windows of the first and of the last unit of a call
WINDOW_TARGET = 8192      # positions per query window of the unit pipeline; a call of n units uses at most ceil(8/n) windows per unit


def _t_chunks(T: int, target: Optional[int] = None, most: int = 8):
    """Cut [0, T) into at most `most` windows of about `target` positions (multiples of 256 except the last)."""
    n = max(1, min(most, T // (target or WINDOW_TARGET)))
    step = -(-T // n)
    step = -(-step // 256) * 256
    return [(a, min(T, a + step)) for a in range(0, T, step)]


def _by_units(q, k, v, dO, outs, dev, streams, compression_rate, max_top_nodes, top_k_per_layer, scale, rope_base):
    """One (batch, KV head) unit at a time, and inside a unit one window of query positions at a time.

    A unit reads q/dO slices [1,T,G,D] and k/v slices [1,T,1,D] and writes the same slices of the results.  Its k and v
    go up first and the tree is built once; q, dO, out and dq then move window by window (the forward takes a query
    window, the backward accumulates dK/dV across windows), so that only one window's upload precedes the first kernel
    and only one window's download follows the last one."""
    s_in, s_run, s_out = streams
    B, T, H, K = q.shape
    H_kv, V = k.shape[2], v.shape[-1]
    G = H // H_kv
    bwd = dO is not None
    if scale is None:
        scale = K ** -0.5
    # windows shorten the exposed first upload / last download but cost launch tails: every unit is windowed when a call
    # has few units, otherwise only the first and the last one (whose upload / download nothing else hides)
    n_units = B * H_kv
    most_all = max(1, min(8, -(-8 // n_units)))
    windows_all = _t_chunks(T, most=most_all)
    windows_edge = _t_chunks(T, most=max(most_all, EDGE_WINDOWS))
    keep = []

    def held(ts):
        for t in ts:
            t.record_stream(s_run); t.record_stream(s_out)
        keep.append(ts)
        if len(keep) > 6:
            keep.pop(0)

    with torch.cuda.device(dev):
        for b in range(B):
            for hk in range(H_kv):
                hs = slice(hk * G, (hk + 1) * G)
                with torch.cuda.stream(s_in):
                    k_d = torch.empty((1, T, 1, K), dtype=k.dtype, device=dev)
                    v_d = torch.empty((1, T, 1, V), dtype=v.dtype, device=dev)
                    _copy_unit(k_d, k[b:b + 1, :, hk:hk + 1], s_in)
                    _copy_unit(v_d, v[b:b + 1, :, hk:hk + 1], s_in)
                    kv_ready = torch.cuda.Event(); kv_ready.record(s_in)
                with torch.cuda.stream(s_run):
                    s_run.wait_event(kv_ready)
                    layers = ops.build_tree(k_d, v_d, compression_rate, max_top_nodes, rope_base)
                held([k_d, v_d] + [x for lv in layers if lv is not None for x in lv])
                acc = {}
                windows = windows_edge if b * H_kv + hk in (0, n_units - 1) else windows_all
                for wi, (t0, t1) in enumerate(windows):
                    first, last = wi == 0, wi == len(windows) - 1
                    with torch.cuda.stream(s_in):
                        q_d = torch.empty((1, t1 - t0, G, K), dtype=q.dtype, device=dev)
                        _copy_unit(q_d, q[b:b + 1, t0:t1, hs], s_in)
                        q_ready = torch.cuda.Event(); q_ready.record(s_in)
                        if bwd:
                            dO_d = torch.empty((1, t1 - t0, G, V), dtype=dO.dtype, device=dev)
                            _copy_unit(dO_d, dO[b:b + 1, t0:t1, hs], s_in)
                            dO_ready = torch.cuda.Event(); dO_ready.record(s_in)
                    with torch.cuda.stream(s_run):
                        s_run.wait_event(q_ready)
                        if bwd:
                            o, ctx = ops.htree_forward(q_d, k_d, v_d, compression_rate, max_top_nodes, top_k_per_layer, scale,
                                                       rope_base, _save_for_backward=True, _q_offset=t0, _layers=layers)
                            fwd_done = torch.cuda.Event(); fwd_done.record(s_run)
                            s_run.wait_event(dO_ready)
                            dq, dk, dv = ops.htree_backward(dO_d, q_d, o, ctx, _typed=True,
                                                            _window=dict(t0=t0, first=first, last=last, acc=acc))
                            del ctx
                        else:
                            o = ops.htree_forward(q_d, k_d, v_d, compression_rate, max_top_nodes, top_k_per_layer, scale,
                                                  rope_base, _q_offset=t0, _layers=layers)
                            fwd_done = torch.cuda.Event(); fwd_done.record(s_run)
                        done = torch.cuda.Event(); done.record(s_run)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(fwd_done)
                        _copy_unit(outs[0][b:b + 1, t0:t1, hs], o, s_out)
                        if bwd:
                            s_out.wait_event(done)
                            _copy_unit(outs[1][b:b + 1, t0:t1, hs], dq, s_out)
                            if last:
                                _copy_unit(outs[2][b:b + 1, :, hk:hk + 1], dk, s_out)
                                _copy_unit(outs[3][b:b + 1, :, hk:hk + 1], dv, s_out)
                    held([q_d, o] + ([dO_d, dq] if bwd else []) + ([dk, dv] if bwd and last else []))
                if bwd:
                    held([x for lst in (acc["dk"], acc["dv"]) for x in lst])
    s_out.synchronize(); s_run.synchronize(); s_in.synchronize()
    return tuple(outs)
