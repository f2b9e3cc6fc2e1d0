"""Host-side logic that needs no GPU: query windows of the host-buffer pipeline, the default sequence split, the staged
reference (when present) against the committed golden fixtures, and the storage-type rule of htree_backward."""
import os

import numpy as np
import pytest
import torch

from tests import parity


def test_query_windows_cover_the_sequence():
    from htree_b200 import host
    for T, most in ((65536, 8), (65536, 4), (16384, 8), (1000, 8), (524288, 2), (8193, 8), (70000, 3)):
        w = host._t_chunks(T, most=most)
        assert w[0][0] == 0 and w[-1][1] == T and len(w) <= most
        for (a, b), (c, _) in zip(w, w[1:] + [(T, T)]):
            assert b == c and b > a
        assert all(a % 256 == 0 for a, _ in w)
    assert host._t_chunks(65536, most=1) == [(0, 65536)]
    assert len(host._t_chunks(65536, target=512, most=8)) == 8


def test_default_sequence_split_is_work_balanced_where_possible():
    from htree_b200 import dist as hdist
    T, CR, TK, MTN = 524288, 16, 64, 512                      # four levels: boundaries are multiples of 4096
    r = hdist.default_query_ranges(T, 8, CR, TK, MTN)
    assert r == hdist.balanced_query_ranges(T, 8, CR, TK, MTN)
    assert r[0][0] == 0 and r[-1][1] == T and all(a % 4096 == 0 and b > a for a, b in r)
    assert r[0][1] - r[0][0] > r[-1][1] - r[-1][0]             # early positions are cheaper: the first rank gets more of them
    assert hdist.default_query_ranges(T, 1, CR, TK, MTN) == [(0, T)]
    r2 = hdist.default_query_ranges(8192, 2, 16, 64, 512)      # two levels: boundaries are multiples of 16
    assert r2[0][0] == 0 and r2[0][1] == r2[1][0] and r2[1][1] == 8192 and r2[0][1] % 16 == 0 and r2[0][1] > 4096


def test_staged_reference_matches_the_golden_fixtures():
    """oracle/_ref holds byte-identical copies of the reference's files (manifest check), and its CPU oracle reproduces a
    committed fixture that was generated from the reference checkout: the staged files are the reference."""
    from oracle import ref_triton, stage_reference
    ok, why = ref_triton.available()
    if not ok:
        pytest.skip(why)
    assert stage_reference.verify()
    name = "f32_T64_dense"
    c, g = parity.golden_cases()[name], parity.load_golden(name)
    q, k, v, _ = parity.case_inputs(c)
    assert ref_triton.legal_max_top_nodes(c["TK"], c["CR"]) == c["TK"] * c["CR"]
    out = ref_triton.naive_forward(q, k, v, c["CR"], c["TK"])
    assert np.array_equal(out.float().numpy(), g["out"].astype(np.float32))


def test_backward_refuses_an_output_gradient_of_another_dtype():
    from htree_b200 import ops
    q = torch.zeros(1, 4, 2, 16, dtype=torch.bfloat16)
    ctx = dict(layers_k=[torch.zeros(1, 4, 1, 16, dtype=torch.bfloat16)], layers_v=[torch.zeros(1, 4, 1, 16, dtype=torch.bfloat16)],
               num_layers=1, compression_rate=4, top_k_per_layer=2, max_top_nodes=8, scale=0.25, cos_cache=None, sin_cache=None)
    with pytest.raises(ValueError, match="dtype"):
        ops.htree_backward(torch.zeros(1, 4, 2, 16), q, q, ctx)


def test_cost_model_chunk_counts_match_a_walk_over_every_query():
    """The bytes the bench charges to the forward's two kernels rest on the number of chunks (one parent's children) a
    group visits; count them position by position for a small shape and compare with the closed form."""
    from htree_b200 import configs
    c = dict(B=2, T=3000, H=8, H_kv=2, D=128, CR=16, TK=8, MTN=32, dtype="bfloat16", mode="fwd")
    cm = configs.cost_model(c)
    sizes = configs.level_sizes(c["T"], c["CR"], c["MTN"])
    L, CR, TK = len(sizes), c["CR"], c["TK"]
    sel = acc = 0
    for t in range(c["T"]):
        n_par = min(TK, (t // CR ** (L - 1)) // CR + 1)
        for l in range(L - 1, -1, -1):
            nc = (n_par - 1) * CR + (t // CR ** l) % CR + 1
            chunks = -(-nc // CR)
            assert chunks == n_par
            if l > 0:
                if nc > TK:
                    sel += chunks
                    acc += chunks
                n_par = min(TK, nc)
            else:
                acc += chunks
    groups = c["B"] * c["H_kv"]
    assert cm["selection_chunks"] == sel * groups
    assert cm["accumulation_chunks"] == acc * groups


def test_binding_the_host_side_to_a_device_never_raises():
    """Without a GPU (or without the sysfs entries) the helper reports None and leaves the affinity alone."""
    from htree_b200 import host
    before = os.sched_getaffinity(0)
    got = host.bind_host_to_device("cuda:0")
    assert got is None or (isinstance(got, dict) and got["cpus"] >= 1)
    if got is None:
        assert os.sched_getaffinity(0) == before
    os.sched_setaffinity(0, before)
