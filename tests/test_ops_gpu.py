"""Native auxiliary ops (sign packing, top-k selection) against their PyTorch definitions."""
import pytest
import torch

from powersgd_b200.ops import signpack
from powersgd_b200.ops.topk import sparse_combine, sparse_combine_status, topk_abs, topk_abs_many

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


def test_topk_abs_many_matches_per_tensor_selection():
    """One batched call (four launches) against torch.topk per tensor: same value multisets, positions
    consistent with values, memories = tensors with the taken entries zeroed; repeated calls reuse the
    cached tables; ties and an all-equal tensor included."""
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(3)
    shapes = [(64, 3, 3, 3), (10,), (1,), (512, 4608), (300, 1200), (64,), (130, 650), (2048,)]
    tensors = [torch.randn(s, generator=g).to(dev) for s in shapes]
    tensors[5].fill_(1.5)                       # all equal: any subset is a valid answer
    tensors[7][::2] = tensors[7][1::2]          # pairs of exact ties
    ks = [max(1, t.numel() // 7) for t in tensors]
    ks[1], ks[2] = 10, 1                        # k == n
    for rep in range(2):
        mems = [torch.full_like(t, float("nan")) for t in tensors] if rep == 0 else mems
        values, positions = topk_abs_many(tensors, ks, mems)
        torch.cuda.synchronize()
        assert values.shape == (sum(ks),) and positions.dtype == torch.int32
        at = 0
        for t, k, m in zip(tensors, ks, mems):
            v, p = values[at : at + k], positions[at : at + k].long()
            at += k
            flat = t.reshape(-1)
            assert p.unique().numel() == k and int(p.min()) >= 0 and int(p.max()) < flat.numel()
            assert torch.equal(v, flat[p])
            ref, _ = torch.topk(flat.abs(), k, sorted=True)
            assert torch.equal(v.abs().sort(descending=True).values, ref)
            expect = flat.clone()
            expect[p] = 0.0
            assert torch.equal(m.reshape(-1), expect)
        tensors[0].mul_(-1.0)                   # same pointers, new data: the cached tables stay valid


def test_sparse_combine_matches_sequential_index_add_bitwise():
    """The cooperative scatter-combine launch against one index_add_ per worker in rank order:
    identical bits (fixed summation order), also where several workers hit the same position."""
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(7)
    workers = 5
    numels = [27 * 64, 1, 650 * 130, 10, 1 << 20]
    sizes = [max(1, n // 8) for n in numels]
    ends = torch.tensor(sizes).cumsum(0).tolist()
    total = ends[-1]
    values = torch.randn(workers, total, generator=g).to(dev)
    positions = torch.empty(workers, total, dtype=torch.int32)
    start = 0
    for n, k, end in zip(numels, sizes, ends):
        for w in range(workers):
            positions[w, start:end] = torch.randperm(n, generator=g)[:k].to(torch.int32)   # unique per worker, collisions across workers
        start = end
    positions = positions.to(dev)
    outs = [torch.full((n,), float("nan"), device=dev) for n in numels]
    sparse_combine(values, positions, outs, ends, float(workers))
    torch.cuda.synchronize()
    assert sparse_combine_status(dev) == 0
    start = 0
    for n, out, end in zip(numels, outs, ends):
        ref = torch.zeros(n, device=dev)
        for w in range(workers):
            ref.index_add_(0, positions[w, start:end].long(), values[w, start:end] / workers)
        assert torch.allclose(out, ref, atol=1e-6), (n, (out - ref).abs().max().item())
        assert torch.equal(out, ref), (n, "same sum, different rounding")
        start = end
    # a second call reuses the barrier word
    sparse_combine(values, positions, outs, ends, 1.0)
    torch.cuda.synchronize()
    assert sparse_combine_status(dev) == 0 and bool(torch.isfinite(outs[-1]).all())


def test_batched_tall_svd_matches_torch():
    from powersgd_b200.ops.svd import svd_many

    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(0)
    mats = [torch.randn(2048, 18, generator=g), torch.randn(32, 2, generator=g), torch.randn(10, 512, generator=g),
            torch.randn(300, 32, generator=g), torch.randn(64, 64, generator=g)]
    mats[3][:, 5] = mats[3][:, 4]  # a rank-deficient one
    mats = [m.to(dev) for m in mats]
    for m, (u, s, v) in zip(mats, svd_many(mats)):
        k = min(m.shape)
        assert u.shape == (m.shape[0], k) and v.shape == (m.shape[1], k) and s.shape == (k,)
        assert (s[:-1] >= s[1:] - 1e-6).all()
        ref = torch.linalg.svdvals(m)
        assert torch.allclose(s, ref, rtol=1e-4, atol=1e-4 * ref[0].item())
        recon = (u * s) @ v.t()
        assert (recon - m).norm() / m.norm() < 1e-4
        keep = s > 1e-4 * s[0]
        eye = torch.eye(int(keep.sum()), device=dev)
        assert torch.allclose(u[:, keep].t() @ u[:, keep], eye, atol=1e-3)
        assert torch.allclose(v[:, keep].t() @ v[:, keep], eye, atol=1e-3)


def test_atomo_reducer_on_gpu_uses_native_svd():
    from powersgd_b200.paper import reducers as R

    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    grads = [torch.randn(16, 8, 3, 3, device=dev), torch.randn(64, device=dev), torch.randn(10, 40, device=dev)]
    outs, mems = [torch.zeros_like(g) for g in grads], [torch.zeros_like(g) for g in grads]
    red = R.AtomoReducer(1, dev, None, rank=2)
    assert red.svd_on_cpu is False
    bits = red.reduce(grads, outs, mems)
    assert bits > 0 and all(torch.isfinite(o).all() for o in outs)
