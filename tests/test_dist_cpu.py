"""Host-side sharding logic on CPU: unit partition / gather / scatter, query ranges, and the all-gather layout of the
sequence-sharded tree build under a real world_size-2 gloo group (the CUDA tree build is replaced by a torch one)."""
import os
import socket

import pytest
import torch
import torch.distributed as tdist
import torch.multiprocessing as mp

from htree_b200 import configs, dist as hdist


def test_unit_partition_covers_every_unit_once():
    for n_units, world in ((16, 1), (16, 2), (16, 8), (6, 4)):
        seen = sorted(u for r in range(world) for u in hdist.unit_partition(n_units, world, r))
        assert seen == list(range(n_units))
        sizes = [len(hdist.unit_partition(n_units, world, r)) for r in range(world)]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        hdist.unit_partition(4, 2, 2)


def test_gather_scatter_units_roundtrip():
    B, T, H, Hkv, K, V = 2, 5, 8, 2, 4, 6
    q = torch.randn(B, T, H, K); k = torch.randn(B, T, Hkv, K); v = torch.randn(B, T, Hkv, V); dO = torch.randn(B, T, H, V)
    units = [1, 2]
    ql, kl, vl, dl = hdist.gather_units(q, k, v, units, extra=(dO,))
    assert ql.shape == (2, T, H // Hkv, K) and kl.shape == (2, T, 1, K) and vl.shape == (2, T, 1, V)
    assert torch.equal(ql[0], q[0, :, 4:8]) and torch.equal(kl[1], k[1, :, 0:1]) and torch.equal(dl[1], dO[1, :, 0:4])
    full_q = torch.zeros_like(q); full_k = torch.zeros_like(k)
    hdist.scatter_units(ql, full_q, units, Hkv); hdist.scatter_units(kl, full_k, units, Hkv)
    assert torch.equal(full_q[0, :, 4:8], q[0, :, 4:8]) and torch.equal(full_q[1, :, 0:4], q[1, :, 0:4])
    assert float(full_q[0, :, 0:4].abs().sum()) == 0.0 and torch.equal(full_k[1, :, 0], k[1, :, 0])


def test_query_range_grain():
    assert hdist.query_range(524288, 8, 3, 16, 4) == (196608, 262144)
    with pytest.raises(ValueError):
        hdist.query_range(524288, 8, 0, 16, 6)       # 65536 per rank is not a multiple of 16^5
    with pytest.raises(ValueError):
        hdist.query_range(1000, 3, 0, 16, 2)


def test_balanced_ranges_cover_the_sequence_and_even_out_the_cost():
    import numpy as np
    T, CR, TK, MTN = 524288, 16, 64, 512
    for world in (2, 4, 8):
        ranges = hdist.balanced_query_ranges(T, world, CR, TK, MTN)
        assert ranges[0][0] == 0 and ranges[-1][1] == T
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:])) and all(a % 4096 == 0 for a, _ in ranges)
        nc, acc = configs.attend_counts(T, CR, TK, 4)
        cost = np.where(nc[1:] > TK, nc[1:], 0).sum(0) + 2 * acc.sum(0)
        per_rank = np.array([cost[a:b].sum() for a, b in ranges], dtype=np.float64)
        even = np.array([cost[r * T // world:(r + 1) * T // world].sum() for r in range(world)], dtype=np.float64)
        assert per_rank.max() / per_rank.mean() < 1.05 < even.max() / even.mean()   # block granularity 4096 tokens


def _torch_build(k, v, cr, mtn):
    lk, lv = [k], [v]
    while lk[-1].shape[1] > mtn:
        n = lk[-1].shape[1]
        assert n % cr == 0
        lk.append(lk[-1].view(k.shape[0], n // cr, cr, *k.shape[2:]).float().mean(2).to(k.dtype))
        lv.append(lv[-1].view(v.shape[0], n // cr, cr, *v.shape[2:]).float().mean(2).to(v.dtype))
    return lk, lv


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    tdist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        k = torch.randn(2, 256, 2, 8, generator=g); v = torch.randn(2, 256, 2, 4, generator=g)
        lk, lv = hdist.build_tree_sequence_parallel(k, v, 4, 10, _build=_torch_build)     # 256 -> 64 -> 16 -> 4
        rk, rv = _torch_build(k, v, 4, 10)
        ok = len(lk) == len(rk) == 4 and all(torch.allclose(a, b, atol=1e-6) for a, b in zip(lk + lv, rk + rv))
        # uneven (work-balanced) ranges: slices are padded for the all-gather and stitched back
        lk2, lv2 = hdist.build_tree_sequence_parallel(k, v, 4, 10, _build=_torch_build, ranges=[(0, 192), (192, 256)])
        ok = ok and all(torch.allclose(a, b, atol=1e-6) for a, b in zip(lk2 + lv2, rk + rv))
        q.put((rank, bool(ok)))
    finally:
        tdist.destroy_process_group()


def test_sequence_parallel_tree_build_gloo_world2():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=60) for _ in procs)
    for p in procs:
        p.join(60)
    assert results == [(0, True), (1, True)]


def test_cost_model_matches_published_counts():
    m = configs.cost_model(configs.CONFIGS["cfg3"])
    assert m["levels"] == [65536, 4096, 256]
    assert abs(m["flops_fwd"] / 1e12 - 16.903) < 1e-3 and abs(m["flops_bwd"] / 1e12 - 40.974) < 1e-3
    assert abs(m["bytes_fwd"] / 1e9 - 9.905) < 1e-3
