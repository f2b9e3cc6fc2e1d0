"""Multi-GPU sharding of the htree operator: one process per GPU, torch.distributed for the plumbing.

The reference (skywong14/htree) is single-GPU; both modes below are new.  They rest on one property of the operator:
given the tree, every (batch, query position, KV head) group is independent (src/naive.py:180-213 loops over them).

Mode A — units.  A unit is one (batch, KV head) pair: it reads q[b, :, hk*G:(hk+1)*G], k[b, :, hk], v[b, :, hk] and
writes the same slices of out / dq / dk / dv.  Units are dealt round-robin to ranks; a rank runs its units as a batch
of independent single-KV-head problems.  Forward and backward need no communication at all.

Mode B — query positions of one long sequence.  Rank r owns the query range [r*T/n, (r+1)*T/n); k and v are
replicated inputs.  Each rank pools only its own slice of every tree level and one all_gather per pooled level puts
the complete coarse levels into local HBM before the attention kernel starts; the kernels only ever read local
memory.  Requires T/n to be a multiple of compression_rate^(levels-1) so that no pooled node straddles two ranks.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import configs


# ---------------------------------------------------------------- mode A: (batch, KV head) units

def unit_partition(n_units: int, world_size: int, rank: int) -> List[int]:
    """Units owned by `rank`: round-robin, so every rank gets floor or ceil of n_units/world_size of them."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of {world_size}")
    return list(range(rank, n_units, world_size))


def unit_of(b: int, hk: int, H_kv: int) -> int:
    return b * H_kv + hk


def gather_units(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, units: Sequence[int], extra: Sequence[torch.Tensor] = ()):
    """Slices of the full tensors for `units`, as a batch of single-KV-head problems.

    q [B,T,H,K] -> [U,T,G,K];  k, v [B,T,H_kv,*] -> [U,T,1,*];  every tensor in `extra` is sliced like q."""
    B, T, H, _ = q.shape
    H_kv = k.shape[2]
    G = H // H_kv

    def heads(x, u):
        b, hk = divmod(u, H_kv)
        return x[b, :, hk * G:(hk + 1) * G]

    ql = torch.stack([heads(q, u) for u in units]).contiguous()
    kl = torch.stack([k[u // H_kv, :, u % H_kv:u % H_kv + 1] for u in units]).contiguous()
    vl = torch.stack([v[u // H_kv, :, u % H_kv:u % H_kv + 1] for u in units]).contiguous()
    el = [torch.stack([heads(x, u) for u in units]).contiguous() for x in extra]
    return (ql, kl, vl, *el)


def scatter_units(local: torch.Tensor, full: torch.Tensor, units: Sequence[int], H_kv: int) -> None:
    """Inverse of gather_units for a q-shaped ([U,T,G,*] -> [B,T,H,*]) or k-shaped ([U,T,1,*] -> [B,T,H_kv,*]) tensor."""
    per = local.shape[2]
    for i, u in enumerate(units):
        b, hk = divmod(u, H_kv)
        full[b, :, hk * per:(hk + 1) * per] = local[i]


# ---------------------------------------------------------------- mode B: query positions

def query_range(T: int, world_size: int, rank: int, compression_rate: int, n_levels: int) -> Tuple[int, int]:
    """[t0, t1) owned by `rank`.  Raises if the split would cut a node of the coarsest pooled level."""
    if T % world_size:
        raise ValueError(f"T={T} is not divisible by world_size={world_size}")
    span = T // world_size
    grain = compression_rate ** (n_levels - 1)
    if span % grain:
        raise ValueError(f"T/world_size={span} must be a multiple of compression_rate^(levels-1)={grain}")
    return rank * span, (rank + 1) * span


def balanced_query_ranges(T: int, world_size: int, compression_rate: int, top_k: int, max_top_nodes: int):
    """Contiguous query ranges [t0, t1) per rank with (nearly) equal WORK instead of equal length.

    The cost of a query grows with its position until every level is saturated (later positions score more
    candidates at the upper levels), so an even split leaves the last ranks with up to ~15 % more work.  Boundaries
    stay multiples of compression_rate^(levels-1), so no pooled node straddles two ranks."""
    import numpy as np
    sizes = configs.level_sizes(T, compression_rate, max_top_nodes)
    L = len(sizes)
    grain = compression_rate ** (L - 1)
    if T % grain or T // grain < world_size:
        raise ValueError(f"T={T} must be a multiple of compression_rate^(levels-1)={grain} with at least one block per rank")
    nc, acc = configs.attend_counts(T, compression_rate, top_k, L)
    scored = np.where(nc[1:] > top_k, nc[1:], 0).sum(0) if L > 1 else 0      # candidates of the selection passes
    cost = (scored + 2 * acc.sum(0)).astype(np.float64)                     # accumulation ~2x a selection-only score
    block_cost = cost.reshape(-1, grain).sum(1)
    csum = np.concatenate([[0.0], np.cumsum(block_cost)])
    n_blocks = block_cost.size
    cuts = [0]
    for r in range(1, world_size):
        target = csum[-1] * r / world_size
        j = int(np.searchsorted(csum, target))
        j = max(cuts[-1] + 1, min(j, n_blocks - (world_size - r)))
        cuts.append(j)
    cuts.append(n_blocks)
    return [(cuts[r] * grain, cuts[r + 1] * grain) for r in range(world_size)]


def build_tree_sequence_parallel(k: torch.Tensor, v: torch.Tensor, compression_rate: int, max_top_nodes: int,
                                 group=None, _build=None, ranges=None):
    """Tree build for mode B: pool the local leaf range, all-gather every pooled level.

    k, v are the full (replicated) leaves [B,T,H_kv,*].  Returns full-length (layers_k, layers_v) in local memory.
    `_build(k, v, compression_rate, max_top_nodes)` replaces the CUDA tree build in host-only tests.
    `ranges`: per-rank leaf ranges [(t0, t1), ...] (multiples of compression_rate^(levels-1)); default = even split.

    Even ranges of a single sequence (B == 1) take the direct route: every rank pools its leaves straight into its own
    slot of the full-length level buffers and one in-place all_gather_into_tensor per level and tensor completes them;
    nothing is staged, padded or concatenated.  Uneven ranges (or B > 1, where a rank's slot is not one contiguous
    piece) pad the pooled slices to the longest one for the all-gather and copy them into place."""
    import torch.distributed as dist
    direct = _build is None
    if _build is None:
        from .ops import build_tree as _build
    build_tree = _build

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    B, T, H_kv, K = k.shape
    sizes = configs.level_sizes(T, compression_rate, max_top_nodes)
    L = len(sizes)
    if world == 1 or L == 1:
        return build_tree(k, v, compression_rate, max_top_nodes)
    if ranges is None:
        ranges = [query_range(T, world, r, compression_rate, L) for r in range(world)]
    t0, t1 = ranges[rank]
    grain = compression_rate ** (L - 1)
    assert all(a % grain == 0 and b % grain == 0 and b > a for a, b in ranges) and ranges[0][0] == 0 and ranges[-1][1] == T
    span = t1 - t0
    even = all(b - a == span for a, b in ranges)
    if direct and even and B == 1:
        from .ops import build_tree_into
        layers_k = [k] + [torch.empty(B, n, H_kv, K, dtype=k.dtype, device=k.device) for n in sizes[1:]]
        layers_v = [v] + [torch.empty(B, n, H_kv, v.shape[-1], dtype=v.dtype, device=v.device) for n in sizes[1:]]
        slots_k = [layers_k[l][:, rank * (span // compression_rate ** l):(rank + 1) * (span // compression_rate ** l)] for l in range(1, L)]
        slots_v = [layers_v[l][:, rank * (span // compression_rate ** l):(rank + 1) * (span // compression_rate ** l)] for l in range(1, L)]
        build_tree_into(k[:, t0:t1], v[:, t0:t1], slots_k, slots_v, compression_rate, span // grain)
        for l in range(1, L):
            for full, slot in ((layers_k[l], slots_k[l - 1]), (layers_v[l], slots_v[l - 1])):
                dist.all_gather_into_tensor(full.view(-1), slot.reshape(-1), group=group)   # in place: the slot is this rank's part of `full`
        return layers_k, layers_v
    # pool the local slice to the same depth: its top level is this rank's share of the global top level
    lk, lv = build_tree(k[:, t0:t1].contiguous(), v[:, t0:t1].contiguous(), compression_rate, (t1 - t0) // grain)
    assert len(lk) == L
    layers_k, layers_v = [k], [v]
    for l in range(1, L):
        step = compression_rate ** l
        lens = [(b - a) // step for a, b in ranges]
        n_max = max(lens)
        for src, dst in ((lk[l], layers_k), (lv[l], layers_v)):
            n_loc = src.shape[1]
            assert n_loc == lens[rank] and sum(lens) == sizes[l]
            if n_loc < n_max:
                pad = torch.zeros((B, n_max - n_loc) + tuple(src.shape[2:]), dtype=src.dtype, device=src.device)
                src = torch.cat([src, pad], dim=1)
            gathered = torch.empty((world * B,) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
            dist.all_gather_into_tensor(gathered, src.contiguous(), group=group)   # rank-major along dim 0
            gathered = gathered.view(world, B, n_max, H_kv, src.shape[-1])
            full = torch.empty((B, sizes[l], H_kv, src.shape[-1]), dtype=src.dtype, device=src.device)
            at = 0
            for r in range(world):
                full[:, at:at + lens[r]] = gathered[r, :, :lens[r]]
                at += lens[r]
            dst.append(full)
    return layers_k, layers_v


def default_query_ranges(T: int, world_size: int, compression_rate: int, top_k: int, max_top_nodes: int):
    """The split htree_forward_sequence_parallel uses when none is given: by equal work where the sequence has at least one
    block of compression_rate^(levels-1) positions per rank, else the even split."""
    L = len(configs.level_sizes(T, compression_rate, max_top_nodes))
    if world_size == 1:
        return [(0, T)]
    try:
        return balanced_query_ranges(T, world_size, compression_rate, top_k, max_top_nodes)
    except ValueError:
        return [query_range(T, world_size, r, compression_rate, L) for r in range(world_size)]


def htree_forward_sequence_parallel(q_local: torch.Tensor, k: torch.Tensor, v: torch.Tensor, compression_rate: int = 16,
                                    max_top_nodes: int = 8192, top_k_per_layer: int = 512, scale: Optional[float] = None,
                                    rope_base: float = 10000.0, group=None, ranges=None) -> torch.Tensor:
    """Mode B forward: q_local holds this rank's query positions [B, t1-t0, H, K]; k, v are the full sequence.
    `ranges`: per-rank query ranges; None = the even split (use default_query_ranges for the work-balanced one, which
    the caller also needs in order to cut q).  Returns out_local [B, t1-t0, H, V]."""
    import torch.distributed as dist
    from .ops import htree_forward

    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    T = k.shape[1]
    L = len(configs.level_sizes(T, compression_rate, max_top_nodes))
    if ranges is not None:
        t0, t1 = ranges[rank]
    else:
        t0, t1 = query_range(T, world, rank, compression_rate, L) if world > 1 else (0, T)
    assert q_local.shape[1] == t1 - t0
    from .ops import block_values, rotate_keys
    layers_k, layers_v = build_tree_sequence_parallel(k, v, compression_rate, max_top_nodes, group, ranges=ranges)
    layers_kr = rotate_keys(layers_k, compression_rate, max_top_nodes, rope_base)   # local work on the gathered levels
    layers_vb = block_values(layers_v, compression_rate, max_top_nodes, layers_kr) if layers_kr is not None else None
    return htree_forward(q_local, k, v, compression_rate, max_top_nodes, top_k_per_layer, scale, rope_base,
                         _q_offset=t0, _layers=(layers_k, layers_v, layers_kr, layers_vb))
