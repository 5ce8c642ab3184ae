"""Semantics of the public aggregators on CPU (mirrors tests/powersgd_test.py of the
reference and adds oracle equality against it when it is importable)."""
import copy

import pytest
import torch

from powersgd_b200 import AllReduce, BasicConfig, BasicPowerSGD, Config, PowerSGD, optimizer_step
from powersgd_b200.plan import CompressionPlan, avg_compressed_size, should_compress

from conftest import reference_library


def small_convnet():
    return torch.nn.Sequential(
        torch.nn.Conv2d(3, 100, 3),
        torch.nn.ReLU(),
        torch.nn.Conv2d(100, 50, 5),
        torch.nn.Linear(50, 1),
    )


def test_warmup_steps_are_plain_allreduce():
    params = list(small_convnet().parameters())
    agg = PowerSGD(params, Config(rank=1, min_compression_rate=10, start_compressing_after_num_steps=2))
    grads = [torch.randn_like(p) for p in params]
    before = [g.clone() for g in grads]
    out = agg.aggregate(grads)
    assert agg.step_counter == 1
    for g in grads:
        assert torch.count_nonzero(g) == 0
    for o, b in zip(out, before):
        assert torch.equal(o, b)


def test_error_feedback_identity_float64():
    torch.set_default_dtype(torch.float64)
    params = list(small_convnet().parameters())
    agg = PowerSGD(
        params, Config(rank=2, min_compression_rate=10, start_compressing_after_num_steps=0, num_iters_per_step=3)
    )
    grads = [torch.randn_like(p) for p in params]
    before = [g.clone() for g in grads]
    out = agg.aggregate(grads)
    for b, o, g in zip(before, out, grads):
        assert torch.allclose(b, o + g)
    assert any(torch.count_nonzero(g) > 0 for g in grads)


def test_mask_uses_raw_shape():
    cfg = Config(rank=2, min_compression_rate=2, num_iters_per_step=2)
    # conv [64,64,3,3]: min over ALL dims is 3, sum is 134
    assert avg_compressed_size((64, 64, 3, 3), cfg) == 0.5 * 2 * 2 * 134
    assert should_compress((64, 64, 3, 3), cfg)
    assert not should_compress((64,), cfg)
    assert should_compress((10, 512), cfg)
    assert not should_compress((10, 512), cfg._replace(min_compression_rate=10))


def test_plan_groups_resnet_like():
    shapes = [(64, 3, 3, 3), (64, 64, 3, 3), (64, 64, 3, 3), (128, 64, 1, 1), (10, 512)]
    plan = CompressionPlan.build(shapes, rank=2)
    assert [(g.n, g.m, g.r, g.batch) for g in plan.groups] == [
        (64, 27, 2, 1),
        (64, 576, 2, 2),
        (128, 64, 2, 1),
        (10, 512, 2, 1),
    ]
    assert plan.p_total == 2 * (64 + 2 * 64 + 128 + 10)
    assert plan.q_total == 2 * (27 + 2 * 576 + 64 + 512)
    assert plan.groups[1].p_offset == 64 * 2


def test_rank_larger_than_matrix():
    p = [torch.zeros(3, 50), torch.zeros(40, 2, 2)]
    core = BasicPowerSGD(p, BasicConfig(rank=8))
    assert [g.r for g in core.plan.groups] == [3, 4]
    g = [torch.randn_like(t) for t in p]
    keep = [t.clone() for t in g]
    out = core.aggregate(g)
    for k, o, e in zip(keep, out, g):
        assert torch.allclose(k, o + e, atol=1e-5)


def test_rank1_uses_joint_norm():
    from powersgd_b200.orthogonalization import orthogonalize

    x = torch.randn(3, 7, 1)
    y = orthogonalize(x.clone())
    assert torch.allclose(y, x / x.norm())
    assert abs(y.norm().item() - 1.0) < 1e-6


def test_allreduce_empty_and_views():
    assert AllReduce().aggregate([]) == []
    g = [torch.ones(3), torch.full((2, 2), 2.0)]
    out = AllReduce().aggregate(g)
    assert out[0].data_ptr() + 3 * 4 == out[1].data_ptr()
    assert torch.equal(out[1], torch.full((2, 2), 2.0))


def test_optimizer_step_keeps_residual_in_grad():
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(40, 30), torch.nn.ReLU(), torch.nn.Linear(30, 5))
    params = list(model.parameters())
    opt = torch.optim.SGD(params, lr=0.1, momentum=0.9)
    agg = PowerSGD(params, Config(rank=2, min_compression_rate=1.5, start_compressing_after_num_steps=0))
    assert agg.is_compressed_mask == [True, False, True, False]
    x, y = torch.randn(16, 40), torch.randint(0, 5, (16,))
    torch.nn.functional.cross_entropy(model(x), y).backward()
    raw = [p.grad.clone() for p in params]
    w0 = [p.detach().clone() for p in params]
    optimizer_step(opt, agg)
    for p, r, w, keep in zip(params, raw, w0, agg.is_compressed_mask):
        applied = (w - p.detach()) / 0.1
        assert torch.allclose(applied + p.grad, r, atol=1e-5)
        if not keep:
            assert torch.count_nonzero(p.grad) == 0
    # second backward accumulates onto the residual
    res = [p.grad.clone() for p in params]
    torch.nn.functional.cross_entropy(model(x), y).backward()
    assert not torch.equal(params[0].grad, res[0])


def test_stats_properties():
    params = [torch.zeros(64, 64, 3, 3), torch.zeros(10, 512)]
    core = BasicPowerSGD(params, BasicConfig(rank=2, num_iters_per_step=2))
    assert core.uncompressed_num_floats == 64 * 64 * 9 + 5120
    assert core.compressed_num_floats == 0.5 * 2 * 2 * 134 + 0.5 * 2 * 2 * 522
    assert core.compression_rate == core.uncompressed_num_floats / core.compressed_num_floats


def test_state_dict_roundtrip_continues_identically():
    torch.manual_seed(1)
    params = list(small_convnet().parameters())
    cfg = Config(rank=2, min_compression_rate=4, start_compressing_after_num_steps=1, num_iters_per_step=1)
    a = PowerSGD(params, cfg)
    grads = [torch.randn_like(p) for p in params]
    for _ in range(3):
        a.aggregate(grads)
        for g in grads:
            g.add_(torch.randn_like(g))
    state = copy.deepcopy(a.state_dict(grads))
    b = PowerSGD(params, cfg)
    grads_b = [torch.zeros_like(p) for p in params]
    b.load_state_dict(state, grads_b)
    assert b.step_counter == a.step_counter and b._powersgd.step_counter == a._powersgd.step_counter
    for x, y in zip(grads, grads_b):
        assert torch.equal(x, y)
    oa, ob = a.aggregate(grads), b.aggregate(grads_b)
    for x, y in zip(oa, ob):
        assert torch.equal(x, y)
    bad = PowerSGD(params, cfg._replace(rank=3))
    with pytest.raises(ValueError):
        bad.load_state_dict(state)


def test_state_dict_restores_residuals_into_channels_last_gradients():
    """Convolution gradients stored channels_last (what TrainStep does on CUDA) are not viewable as
    [n, m] in logical order: the restore has to write through the tensor itself."""
    torch.manual_seed(2)
    params = [torch.zeros(16, 8, 3, 3), torch.zeros(10, 40)]
    cfg = Config(rank=2, min_compression_rate=2, start_compressing_after_num_steps=0)
    a = PowerSGD(params, cfg)
    fmt = torch.channels_last
    grads = [torch.randn(16, 8, 3, 3).contiguous(memory_format=fmt), torch.randn(10, 40)]
    a.aggregate(grads)  # leaves non-zero residuals
    assert float(grads[0].abs().sum()) > 0
    state = copy.deepcopy(a.state_dict(grads))
    b = PowerSGD(params, cfg)
    restored = [torch.zeros(16, 8, 3, 3).contiguous(memory_format=fmt), torch.zeros(10, 40)]
    b.load_state_dict(state, restored)
    for x, y in zip(grads, restored):
        assert torch.equal(x, y)
    assert restored[0].is_contiguous(memory_format=fmt)


@pytest.mark.parametrize("rank,iters,steps", [(1, 1, 3), (2, 2, 3), (4, 3, 4), (2, 1, 5)])
def test_matches_reference_library_bitwise(rank, iters, steps):
    ref = reference_library()
    if ref is None:
        pytest.skip("reference package not mounted")
    torch.manual_seed(3)
    model = torch.nn.Sequential(
        torch.nn.Conv2d(3, 16, 3), torch.nn.Conv2d(16, 16, 3), torch.nn.Conv2d(16, 16, 3), torch.nn.Linear(16, 10)
    )
    params = list(model.parameters())
    kw = dict(rank=rank, min_compression_rate=1.2, num_iters_per_step=iters, start_compressing_after_num_steps=1)
    ours = PowerSGD(params, Config(**kw))
    theirs = ref.PowerSGD(params, ref.Config(**kw))
    assert ours.is_compressed_mask == theirs.is_compressed_mask
    g1 = [torch.randn_like(p) for p in params]
    g2 = [g.clone() for g in g1]
    for _ in range(steps):
        o1, o2 = ours.aggregate(g1), theirs.aggregate(g2)
        for a, b in zip(o1, o2):
            assert torch.allclose(a, b, atol=1e-6, rtol=1e-5)
        for a, b in zip(g1, g2):
            assert torch.allclose(a, b, atol=1e-6, rtol=1e-5)
        noise = [torch.randn_like(p) for p in params]
        for a, b, n in zip(g1, g2, noise):
            a.add_(n)
            b.add_(n)
    assert torch.allclose(ours._powersgd._ps_buffer, theirs._powersgd._ps_buffer, atol=1e-5)
    assert torch.allclose(ours._powersgd._qs_buffer, theirs._powersgd._qs_buffer, atol=1e-5)


def test_channels_last_weights_are_matrices_in_place():
    """A channels_last convolution weight is the same row-major [out, rest] matrix in memory (with
    permuted columns): the compressor works on it in place, and error feedback stays exact."""
    from powersgd_b200.aggregators import view_as_matrix

    torch.manual_seed(0)
    w = torch.randn(16, 8, 3, 3, dtype=torch.float64).contiguous(memory_format=torch.channels_last)
    m = view_as_matrix(w)
    assert m.shape == (16, 72) and m.data_ptr() == w.data_ptr()
    assert torch.equal(m[3], w[3].permute(1, 2, 0).reshape(-1))  # row = one filter, [kh, kw, in] order
    grads = [w.clone(memory_format=torch.preserve_format), torch.randn(32, 16, 1, 1, dtype=torch.float64)]
    assert not grads[0].is_contiguous()
    original = [g.clone(memory_format=torch.preserve_format) for g in grads]
    agg = BasicPowerSGD(grads, BasicConfig(rank=2, num_iters_per_step=2), backend="torch")
    out = agg.aggregate(grads)
    for o, g, ref in zip(out, grads, original):
        assert o.shape == ref.shape
        assert torch.allclose(o + g, ref, atol=1e-12)  # approximation + residual = gradient
    assert float(grads[0].norm()) < float(original[0].norm())


def test_dense_layout_helpers():
    from powersgd_b200.utils import is_dense, like_strided, same_layout

    a = torch.randn(8, 4, 3, 3)
    cl = a.contiguous(memory_format=torch.channels_last)
    assert is_dense(a) and is_dense(cl) and not is_dense(a[:, ::2]) and not is_dense(a.permute(1, 0, 2, 3))
    assert same_layout(a, torch.empty_like(a)) and same_layout(cl, torch.empty_like(cl)) and not same_layout(a, cl)
    # a 1x1 convolution weight is the same memory in both formats although its strides differ
    w = torch.randn(16, 8, 1, 1)
    w_cl = w.contiguous(memory_format=torch.channels_last)
    assert same_layout(w, w_cl) and is_dense(w_cl)
    assert not same_layout(a, torch.randn(8, 4, 3, 2))
    # a flat run viewed like a channels_last tensor holds the elements in that tensor's memory order
    flat = torch.arange(cl.numel(), dtype=torch.float32)
    v = like_strided(flat, cl)
    assert v.shape == cl.shape and v.stride() == cl.stride() and v.data_ptr() == flat.data_ptr()
    assert v[0, 1, 0, 0] == 1 and v[0, 0, 0, 1] == 4  # channel is the fastest dimension
