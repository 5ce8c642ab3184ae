"""Native auxiliary ops (sign packing, top-k selection) against their PyTorch definitions."""
import pytest
import torch

from powersgd_b200.ops import signpack
from powersgd_b200.ops.topk import topk_abs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 31, 32, 1000, 65537])
def test_sign_pack_unpack_vote_match_cpu_definition(n):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(n)
    xs = [torch.randn(n, generator=g) for _ in range(5)]
    xs[0][0] = 0.0
    words_cpu = torch.stack([signpack.pack_signs(x) for x in xs])
    words_gpu = torch.stack([signpack.pack_signs(x.to(dev)) for x in xs])
    assert torch.equal(words_cpu, words_gpu.cpu())
    assert torch.equal(signpack.unpack_signs(words_gpu[0], n).cpu(), torch.where(xs[0] < 0, -1.0, 1.0))
    acc = torch.ones(n, device=dev)
    signpack.unpack_signs(words_gpu[1], n, scale=0.5, out=acc, accumulate=True)
    assert torch.allclose(acc.cpu(), 1.0 + 0.5 * torch.where(xs[1] < 0, -1.0, 1.0))
    for voters in (4, 5):
        assert torch.equal(signpack.vote_signs(words_gpu[:voters], n).cpu(), signpack.vote_signs(words_cpu[:voters], n))
        assert torch.equal(signpack.majority_vote(words_gpu[:voters]).cpu(), signpack.majority_vote(words_cpu[:voters]))


@pytest.mark.parametrize("n,k", [(10, 3), (1000, 1), (4097, 100), (1 << 20, 4300), (300000, 300000), (5000, 4999)])
def test_topk_abs_selects_the_same_set_as_torch(n, k):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(n + k)
    x = torch.randn(n, generator=g).to(dev)
    mem = torch.full_like(x, float("nan"))
    values, positions = topk_abs(x, k, memory=mem)
    torch.cuda.synchronize()
    assert positions.dtype == torch.int32 and values.shape == (k,)
    pos = positions.long()
    assert pos.unique().numel() == k
    assert torch.equal(values, x[pos])
    ref_vals, _ = torch.topk(x.abs(), k, sorted=True)
    assert torch.equal(values.abs().sort(descending=True).values, ref_vals)
    expect_mem = x.clone()
    expect_mem[pos] = 0.0
    assert torch.equal(mem, expect_mem)


def test_topk_abs_with_ties_and_zeros():
    dev = torch.device("cuda:0")
    x = torch.zeros(1000, device=dev)
    x[::10] = 2.0
    x[5::10] = -2.0
    values, positions = topk_abs(x, 150)
    assert (values.abs() == 2.0).all() and positions.long().unique().numel() == 150
    values, positions = topk_abs(x, 300)
    assert int((values.abs() == 2.0).sum()) == 200 and positions.long().unique().numel() == 300
