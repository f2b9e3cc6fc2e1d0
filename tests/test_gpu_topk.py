"""The stand-alone selectors of the selector micro-benchmark against torch.topk: same winner sets, payloads follow their
winners, ties go to the smaller index, order of the output as documented."""
from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("method", ["threshold_search", "radix_select", "bitonic"])
@pytest.mark.parametrize("batch,n,k,n_pay", [(512, 8192, 512, 8), (7, 1024, 64, 1), (3, 8192, 8192, 0), (5, 2048, 2, 0)])
def test_selectors_match_torch_topk(method, batch, n, k, n_pay):
    from htree_b200 import topk_bench
    g = torch.Generator(device="cuda").manual_seed(n + k)
    vals = torch.randn(batch, n, generator=g, device="cuda")
    vals[0, : n // 2] = -vals[0, n // 2:].abs()          # a problem with negative and positive keys
    pay1 = torch.randint(0, 1 << 20, (batch, n), generator=g, device="cuda", dtype=torch.int32) if n_pay >= 1 else None
    pay8 = torch.randint(0, 1 << 20, (batch, n, 8), generator=g, device="cuda", dtype=torch.int32) if n_pay >= 8 else None
    val, idx, p1, p8 = topk_bench.topk(vals, k, method, pay1, pay8)
    ref_val, ref_idx = torch.topk(vals, k, dim=-1)
    assert torch.equal(idx.long().sort(dim=-1).values, ref_idx.sort(dim=-1).values)
    assert torch.equal(val, torch.gather(vals, 1, idx.long()))
    if method == "bitonic":
        assert torch.equal(val, ref_val)                                 # sorted by descending value
    else:
        assert bool((idx[:, 1:] > idx[:, :-1]).all())                    # ascending index
    if p1 is not None:
        assert torch.equal(p1, torch.gather(pay1, 1, idx.long()))
    if p8 is not None:
        assert torch.equal(p8, torch.gather(pay8, 1, idx.long()[:, :, None].expand(-1, -1, 8)))


@pytest.mark.parametrize("method", ["threshold_search", "radix_select", "bitonic"])
def test_ties_go_to_the_smaller_index(method):
    from htree_b200 import topk_bench
    vals = torch.zeros(2, 1024, device="cuda")
    vals[0, 100:110] = 1.0          # 10 clear winners, 22 of the remaining equal keys must be the first 22 by index
    vals[1] = -3.5                  # every key equal
    _, idx, _, _ = topk_bench.topk(vals, 32, method)
    want0 = sorted(list(range(100, 110)) + list(range(22)))
    assert sorted(idx[0].tolist()) == want0
    assert sorted(idx[1].tolist()) == list(range(32))


def test_ragged_sizes_and_argument_errors():
    from htree_b200 import topk_bench
    vals = torch.randn(4, 1000, device="cuda")
    for method in ("threshold_search", "radix_select"):
        _, idx, _, _ = topk_bench.topk(vals, 37, method)
        assert torch.equal(idx.long().sort(dim=-1).values, torch.topk(vals, 37, dim=-1).indices.sort(dim=-1).values)
    with pytest.raises(RuntimeError):
        topk_bench.topk(vals, 37, "bitonic")                      # the network needs powers of two
    with pytest.raises(RuntimeError):
        topk_bench.topk(torch.randn(1, 10000, device="cuda"), 8)  # more keys than shared memory holds
    with pytest.raises(ValueError):
        topk_bench.topk(vals.cpu(), 8)
