"""Native sm_100a kernels against the PyTorch float32/float64 restatement of the same ops."""

import pytest
import torch

from powersgd_b200 import BasicConfig, BasicPowerSGD, Config, PowerSGD, optimizer_step

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return (a.double() - b.double()).norm().item() / max(b.double().norm().item(), 1e-30)


def _lowrank_grads(shapes, device, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = []
    for s in shapes:
        n = s[0]
        m = int(torch.Size(s).numel() // n)
        k = min(8, n, m)
        a = torch.randn(n, k, generator=g) @ torch.randn(k, m, generator=g) + 1e-1 * torch.randn(n, m, generator=g)
        out.append(a.view(s).to(device))
    return out


SHAPES = [(64, 3, 3, 3), (64, 64, 3, 3), (64, 64, 3, 3), (128, 64, 1, 1), (10, 512), (130, 650), (300, 1200), (33, 2100)]


def test_native_library_is_loaded():
    from powersgd_b200.ops import native

    assert native.available(), native.load_error()
    sm, major, minor, smem = [__import__("ctypes").c_int() for _ in range(4)]
    assert native.lib().psgd_device_info(sm, major, minor, smem) == 0
    assert sm.value > 0


@pytest.mark.parametrize("rank,iters,steps", [(1, 1, 3), (1, 2, 2), (2, 2, 3), (4, 1, 4), (4, 3, 2), (8, 2, 2), (16, 2, 2), (3, 2, 2)])
def test_compressor_matches_torch_path(rank, iters, steps):
    dev = torch.device("cuda:0")
    # skip shapes whose residual would be exhausted (rank * iters >= min dim): from there on the
    # factors are rounding noise and no two implementations agree
    shapes = [s for s in SHAPES if min(s[0], int(torch.Size(s).numel() // s[0])) > rank * iters + 2]
    assert len(shapes) >= 5
    params = [torch.zeros(s, device=dev) for s in shapes]
    cfg = BasicConfig(rank=rank, num_iters_per_step=iters)
    ours = BasicPowerSGD(params, cfg, backend="native")
    oracle = BasicPowerSGD(params, cfg, backend="torch")
    assert torch.equal(ours._ps_buffer, oracle._ps_buffer)
    ga = _lowrank_grads(shapes, dev, 0)
    gb = [g.clone() for g in ga]
    # beyond the signal rank (8) the trailing singular values are a near-degenerate noise floor:
    # the subspace is ill-conditioned and two correct algorithms differ more, element by element
    tol = 5e-5 if rank <= 8 else 1e-3
    for step in range(steps):
        before = [g.clone() for g in ga]
        oa = [o.clone() for o in ours.aggregate(ga)]
        ob = oracle.aggregate(gb)
        for x, y, b, res in zip(oa, ob, before, ga):
            assert _rel(x, y) < tol, (step, x.shape, _rel(x, y))
            # error-feedback identity holds to rounding, whatever the factors are
            assert _rel(x + res, b) < 1e-6
        for x, y in zip(ga, gb):
            assert _rel(x, y) < tol, (step, x.shape, _rel(x, y))
            # the compression error itself (norm of the residual) agrees to 1e-5 relative
            assert abs(x.double().norm().item() - y.double().norm().item()) <= (1e-5 if rank <= 8 else 1e-4) * y.double().norm().item()
        fresh = _lowrank_grads(shapes, dev, 100 + step)
        for x, y, f in zip(ga, gb, fresh):
            x.add_(f)
            y.add_(f)
    assert ours.step_counter == oracle.step_counter == steps


def test_orthonormal_factors_and_zero_gradient_recovery():
    dev = torch.device("cuda:0")
    shapes = [(96, 200), (96, 200), (50, 40)]
    params = [torch.zeros(s, device=dev) for s in shapes]
    core = BasicPowerSGD(params, BasicConfig(rank=4, num_iters_per_step=2), backend="native")
    zeros = [torch.zeros(s, device=dev) for s in shapes]
    out = core.aggregate(zeros)
    for o in out:
        assert torch.isfinite(o).all() and torch.count_nonzero(o) == 0
    # after an all-zero step the factors must still be usable
    g = _lowrank_grads(shapes, dev, 5)
    keep = [x.clone() for x in g]
    out = [o.clone() for o in core.aggregate(g)]
    for o, res, k in zip(out, g, keep):
        assert torch.isfinite(o).all()
        assert _rel(o + res, k) < 1e-6
        assert res.norm() < 0.9 * k.norm()
    # the basis that was orthonormalised last is orthonormal
    for q in core._qs:
        for b in range(q.shape[0]):
            gram = q[b].double().T @ q[b].double()
            assert torch.allclose(gram, torch.eye(q.shape[-1], device=dev, dtype=torch.float64), atol=1e-5)


def test_policy_wrapper_native_vs_torch():
    dev = torch.device("cuda:0")
    torch.manual_seed(0)
    model = torch.nn.Sequential(
        torch.nn.Conv2d(3, 32, 3), torch.nn.ReLU(), torch.nn.Conv2d(32, 32, 3), torch.nn.Flatten(), torch.nn.LazyLinear(10)
    ).to(dev)
    model(torch.randn(2, 3, 12, 12, device=dev))
    params = list(model.parameters())
    cfg = Config(rank=2, min_compression_rate=2, num_iters_per_step=2, start_compressing_after_num_steps=1)
    a, b = PowerSGD(params, cfg, backend="native"), PowerSGD(params, cfg, backend="torch")
    ga = [torch.randn_like(p) for p in params]
    gb = [g.clone() for g in ga]
    for _ in range(3):
        oa, ob = a.aggregate(ga), b.aggregate(gb)
        for x, y in zip(oa, ob):
            assert _rel(x, y) < 2e-5 or y.norm() == 0
        for x, y, keep in zip(ga, gb, a.is_compressed_mask):
            if keep:
                assert _rel(x, y) < 2e-5
            else:
                assert torch.count_nonzero(x) == 0
        n = [torch.randn_like(p) for p in params]
        for x, y, z in zip(ga, gb, n):
            x.add_(z)
            y.add_(z)


@pytest.mark.parametrize("nesterov,wd,damp", [(True, 1e-4, 0.0), (False, 0.0, 0.1), (False, 5e-4, 0.0)])
def test_fused_sgd_matches_torch_optimizer(nesterov, wd, damp):
    dev = torch.device("cuda:0")
    torch.manual_seed(1)

    def make():
        torch.manual_seed(1)
        return torch.nn.Sequential(
            torch.nn.Linear(200, 300), torch.nn.ReLU(), torch.nn.Linear(300, 129), torch.nn.ReLU(), torch.nn.Linear(129, 10)
        ).to(dev)

    ma, mb = make(), make()
    kw = dict(lr=0.05, momentum=0.9, nesterov=nesterov, weight_decay=wd, dampening=damp)
    oa, ob = torch.optim.SGD(ma.parameters(), **kw), torch.optim.SGD(mb.parameters(), **kw)
    cfg = Config(rank=4, min_compression_rate=2, num_iters_per_step=2, start_compressing_after_num_steps=1)
    pa = PowerSGD(list(ma.parameters()), cfg, backend="native")
    pb = PowerSGD(list(mb.parameters()), cfg, backend="torch")
    assert pa.supports_fused_step(oa) is False  # no grads yet
    x, y = torch.randn(64, 200, device=dev), torch.randint(0, 10, (64,), device=dev)
    for step in range(4):
        for m in (ma, mb):
            torch.nn.functional.cross_entropy(m(x), y).backward()
        assert pa.supports_fused_step(oa)
        optimizer_step(oa, pa)   # fused kernels
        optimizer_step(ob, pb)   # torch path + torch.optim.SGD
        for p, q in zip(ma.parameters(), mb.parameters()):
            assert _rel(p.detach(), q.detach()) < 1e-5, step
            assert _rel(p.grad, q.grad) < 5e-5 or q.grad.norm() == 0, step
        if step == 1:
            for g in oa.param_groups:
                g["lr"] = 0.02
            for g in ob.param_groups:
                g["lr"] = 0.02
    for p in ma.parameters():
        assert "momentum_buffer" in oa.state[p]


def test_determinism_same_inputs_same_bits():
    dev = torch.device("cuda:0")
    params = [torch.zeros(s, device=dev) for s in SHAPES]
    outs = []
    for _ in range(2):
        core = BasicPowerSGD(params, BasicConfig(rank=2, num_iters_per_step=2), backend="native")
        g = _lowrank_grads(SHAPES, dev, 3)
        o = [t.clone() for t in core.aggregate(g)]
        o2 = [t.clone() for t in core.aggregate(g)]
        outs.append((o, o2, [t.clone() for t in g]))
    for a, b in zip(outs[0], outs[1]):
        for x, y in zip(a, b):
            assert torch.equal(x, y)


def test_train_step_graph_matches_plain_loop():
    """TrainStep (side-stream branches, CUDA-graph replay) follows the same trajectory as the
    documented plain loop (backward + optimizer_step)."""
    from powersgd_b200.engine import TrainStep

    dev = torch.device("cuda:0")

    def make():
        torch.manual_seed(4)
        model = torch.nn.Sequential(torch.nn.Linear(96, 160), torch.nn.Tanh(), torch.nn.Linear(160, 64), torch.nn.Tanh(),
                                    torch.nn.Linear(64, 10)).to(dev)
        params = list(model.parameters())
        opt = torch.optim.SGD(params, lr=0.05, momentum=0.9, nesterov=True, weight_decay=1e-4)
        agg = PowerSGD(params, Config(rank=2, min_compression_rate=2, num_iters_per_step=2, start_compressing_after_num_steps=1))
        return model, opt, agg

    g = torch.Generator().manual_seed(0)
    batches = [(torch.randn(32, 96, generator=g).to(dev), torch.randint(0, 10, (32,), generator=g).to(dev)) for _ in range(8)]
    ma, oa, pa = make()
    step = TrainStep(ma, torch.nn.functional.cross_entropy, oa, pa, cuda_graph=True)
    la = [float(step(x, y).item()) for x, y in batches]
    assert step._graphs, "never captured"
    mb, ob, pb = make()
    lb = []
    for x, y in batches:
        loss = torch.nn.functional.cross_entropy(mb(x), y)
        loss.backward()
        optimizer_step(ob, pb)
        lb.append(float(loss.item()))
    assert pa.step_counter == pb.step_counter == 8
    assert pa._powersgd.step_counter == pb._powersgd.step_counter == 7
    for a, b in zip(la, lb):
        assert abs(a - b) < 1e-4 * max(1.0, abs(b)), (la, lb)
    for p, q in zip(ma.parameters(), mb.parameters()):
        assert _rel(p.detach(), q.detach()) < 1e-4


def test_train_step_with_channels_last_weights_matches_plain_loop():
    """TrainStep stores convolution weights channels_last, detaches the residuals during backward
    and folds the fresh gradients in with one launch. The documented plain loop on a model in the
    same layout (autograd accumulating onto p.grad) must follow the same trajectory."""
    from powersgd_b200.engine import TrainStep

    dev = torch.device("cuda:0")
    # an earlier TrainStep in this process may have switched convolution autotuning on; both arms
    # of this comparison must run the same deterministic algorithm choice
    torch.backends.cudnn.benchmark = False

    def make():
        torch.manual_seed(11)
        model = torch.nn.Sequential(
            torch.nn.Conv2d(3, 32, 3, padding=1, bias=False), torch.nn.BatchNorm2d(32), torch.nn.ReLU(),
            torch.nn.Conv2d(32, 64, 3, padding=1, stride=2, bias=False), torch.nn.BatchNorm2d(64), torch.nn.ReLU(),
            torch.nn.Conv2d(64, 64, 1, bias=False), torch.nn.ReLU(),
            torch.nn.AdaptiveAvgPool2d(1), torch.nn.Flatten(), torch.nn.Linear(64, 10),
        ).to(dev)
        params = list(model.parameters())
        opt = torch.optim.SGD(params, lr=0.05, momentum=0.9, nesterov=True, weight_decay=1e-4)
        agg = PowerSGD(params, Config(rank=2, min_compression_rate=2, num_iters_per_step=2, start_compressing_after_num_steps=0))
        return model, opt, agg

    g = torch.Generator().manual_seed(1)
    batches = [(torch.randn(16, 3, 16, 16, generator=g).to(dev), torch.randint(0, 10, (16,), generator=g).to(dev)) for _ in range(7)]
    ma, oa, pa = make()
    step = TrainStep(ma, torch.nn.functional.cross_entropy, oa, pa, cuda_graph=True, autotune=False)
    la = [float(step(x, y).item()) for x, y in batches]
    assert step._graphs, "never captured"
    conv_weights = [p for p in ma.parameters() if p.dim() == 4 and p.shape[2] > 1]
    assert conv_weights and all(not p.is_contiguous() and not p.grad.is_contiguous() for p in conv_weights)
    mb, ob, pb = make()
    mb.to(memory_format=torch.channels_last)
    lb = []
    for x, y in batches:
        loss = torch.nn.functional.cross_entropy(mb(x.contiguous(memory_format=torch.channels_last)), y)
        loss.backward()
        optimizer_step(ob, pb)
        lb.append(float(loss.item()))
    for a, b in zip(la, lb):
        assert abs(a - b) < 2e-3 * max(1.0, abs(b)), (la, lb)
    for p, q in zip(ma.parameters(), mb.parameters()):
        assert _rel(p.detach(), q.detach()) < 2e-3
    # the residual stays in p.grad, as the plain loop leaves it
    for p, q in zip(ma.parameters(), mb.parameters()):
        assert _rel(p.grad, q.grad) < 5e-3 or float(q.grad.abs().max()) == 0.0
    # batch-norm state: counters advance once per step (eager and replayed alike), statistics follow
    for (name, ba), (_n, bb) in zip(ma.named_buffers(), mb.named_buffers()):
        if ba.dtype == torch.long:
            assert int(ba) == int(bb) == len(batches), name
        else:
            assert _rel(ba, bb) < 2e-3, name
    # the counters are views of one tensor bumped by a single launch; checkpoints do not notice
    assert step._norm_counters is not None and step._norm_counters.tolist() == [len(batches)] * 2
    assert set(ma.state_dict()) == set(mb.state_dict())
    ma.load_state_dict(mb.state_dict())
    step(*batches[0])
    assert step._norm_counters.tolist() == [len(batches) + 1] * 2
    assert all(int(m.num_batches_tracked) == len(batches) + 1 for m in ma.modules() if isinstance(m, torch.nn.BatchNorm2d))


def test_compression_error_matches_upstream_package():
    """The native path against the UNMODIFIED upstream package (installed under baseline/_ref) on
    the same device: outputs and residuals agree, and the compression error (norm of what is left
    in the gradients) agrees to 1e-5 relative - including row pitches of 27 and 650 floats."""
    from conftest import reference_library

    ref = reference_library()
    if ref is None:
        pytest.skip("upstream package not installed under baseline/_ref")
    dev = torch.device("cuda:0")
    shapes = [(64, 3, 3, 3), (64, 64, 3, 3), (64, 64, 3, 3), (130, 650), (300, 1200), (10, 512), (16,), (2600, 650)]
    params = [torch.zeros(s, device=dev) for s in shapes]
    cfg = dict(rank=2, min_compression_rate=2, num_iters_per_step=2, start_compressing_after_num_steps=0)
    ours = PowerSGD(params, Config(**cfg), backend="native")
    theirs = ref.PowerSGD(params, ref.Config(**cfg))
    # same warm start: both draw from a device generator seeded 0, in the same order
    assert torch.equal(ours._powersgd._ps_buffer, theirs._powersgd._ps_buffer)
    ga = _lowrank_grads(shapes, dev, 21)
    gb = [g.clone() for g in ga]
    for step in range(3):
        oa = [o.clone() for o in ours.aggregate(ga)]
        ob = theirs.aggregate(gb)
        for x, y, keep in zip(oa, ob, ours.is_compressed_mask):
            assert _rel(x, y) < 5e-5 or float(y.norm()) == 0.0, (step, tuple(x.shape), _rel(x, y))
        for x, y, keep in zip(ga, gb, ours.is_compressed_mask):
            if keep:
                gap = abs(x.double().norm().item() - y.double().norm().item())
                assert gap <= 1e-5 * y.double().norm().item(), (step, tuple(x.shape), gap)
        fresh = _lowrank_grads(shapes, dev, 200 + step)
        for x, y, f in zip(ga, gb, fresh):
            x.add_(f)
            y.add_(f)


def test_scratch_garbage_never_reaches_an_output():
    """NaN canaries: every scratch buffer the kernels use between launches (partial sums of split
    tiles, orthonormalisation partials, summed-factor copies, the output arena) is filled with NaN
    before a step; a kernel that read a word it had not written this step would leak one."""
    dev = torch.device("cuda:0")
    params = [torch.zeros(s, device=dev) for s in SHAPES]
    core = BasicPowerSGD(params, BasicConfig(rank=4, num_iters_per_step=2), backend="native")
    g = _lowrank_grads(SHAPES, dev, 9)
    core.aggregate(g)  # binds and allocates
    nat = core._native
    for buf in [nat._partial, nat._partial_tc, nat._orth_part, nat._orth_rinv, nat._out_arena] + nat.h_loc + nat.h_in:
        buf.fill_(float("nan"))
    g = _lowrank_grads(SHAPES, dev, 10)
    keep = [x.clone() for x in g]
    out = core.aggregate(g)
    for o, res, k in zip(out, g, keep):
        assert torch.isfinite(o).all() and torch.isfinite(res).all()
        assert _rel(o + res, k) < 1e-6
    assert torch.isfinite(core._ps_buffer).all() and torch.isfinite(core._qs_buffer).all()


def test_single_worker_launch_count_and_warm_start_written_by_the_product():
    """One worker, rank 2 x 2 iterations: orth (2) + product + orth (2) + product + decompression;
    the product launch itself leaves the fresh factor in the warm-start buffer (no copy)."""
    dev = torch.device("cuda:0")
    shapes = [(64, 3, 3, 3), (64, 64, 3, 3), (130, 650), (256, 512)]  # access widths 1, 4, 2, 4 in ONE launch each
    params = [torch.zeros(s, device=dev) for s in shapes]
    core = BasicPowerSGD(params, BasicConfig(rank=2, num_iters_per_step=2), backend="native")
    g = _lowrank_grads(shapes, dev, 1)
    core.aggregate(g)
    nat = core._native
    assert nat.launches == 7, nat.launches
    widths = sorted({int(t["vec"]) for t in nat._tile_arrays["nt"]["f"]})
    assert widths == [1, 2, 4], widths
    # second half-iteration (right side) wrote P: the warm-start buffer equals the local factor
    assert torch.equal(core._ps_buffer, nat.h_loc[1][: core._ps_buffer.numel()])


def test_a_set_status_word_stops_the_next_training_step():
    """Failure detection is wired into the training step: when a bounded device-side wait gave up
    during an earlier step (here the host sets the status word the kernels would have set), the
    next step raises instead of training on with zeros in place of a peer's contribution."""
    from powersgd_b200.engine import TrainStep
    from powersgd_b200.parallel.symm import PowerSGDCommTimeout

    dev = torch.device("cuda:0")
    torch.manual_seed(3)
    model = torch.nn.Sequential(torch.nn.Linear(64, 96), torch.nn.ReLU(), torch.nn.Linear(96, 10)).to(dev)
    params = list(model.parameters())
    opt = torch.optim.SGD(params, lr=0.05, momentum=0.9)
    agg = PowerSGD(params, Config(rank=2, min_compression_rate=2, start_compressing_after_num_steps=0))
    step = TrainStep(model, torch.nn.functional.cross_entropy, opt, agg, cuda_graph=True)
    x, y = torch.randn(16, 64, device=dev), torch.randint(0, 10, (16,), device=dev)
    for _ in range(5):
        step(x, y)
    assert step._graphs
    native = agg._powersgd._native
    native._status.set(3)
    with pytest.raises(PowerSGDCommTimeout, match="training step 5"):
        step(x, y)
    native._status.set(0)
    step(x, y)  # cleared: training goes on, the device was never involved
    torch.cuda.synchronize()
    # the eager entry point looks as well
    native._status.set(3)
    with pytest.raises(PowerSGDCommTimeout):
        optimizer_step(opt, agg)
    native._status.set(0)
