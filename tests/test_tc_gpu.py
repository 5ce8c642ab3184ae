"""tcgen05 / TMA product kernels against the PyTorch float32 formulation of the same step."""
import pytest
import torch

from powersgd_b200 import BasicConfig, BasicPowerSGD

pytestmark = pytest.mark.gpu

# multiples of 4 columns (TMA pitch rule), ragged against the 128 x 32 tiling on purpose
SHAPES = [(256, 512), (300, 1200), (1024, 1024), (1024, 1024), (132, 260), (2048, 384)]


def _rel(a, b):
    return (a.double() - b.double()).norm().item() / max(b.double().norm().item(), 1e-30)


def _grads(shapes, dev, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = []
    for n, m in shapes:
        a = torch.randn(n, 12, generator=g) @ torch.randn(12, m, generator=g) + 0.1 * torch.randn(n, m, generator=g)
        out.append(a.to(dev))
    return out


@pytest.mark.parametrize("rank,iters,precision,tol", [(4, 2, "split", 1e-4), (2, 1, "split", 1e-4), (8, 2, "split", 2e-4),
                                                       (16, 2, "split", 1e-3), (4, 2, "tf32", 2e-2)])
@pytest.mark.parametrize("finalize", ["ffma", "tc"])
def test_tensor_core_products_match_torch_path(monkeypatch, rank, iters, precision, tol, finalize):
    monkeypatch.setenv("PSGD_B200_GEMM", "tc")
    monkeypatch.setenv("PSGD_B200_FINALIZE", finalize)
    monkeypatch.setenv("PSGD_B200_TC_PRECISION", precision)
    dev = torch.device("cuda:0")
    params = [torch.zeros(s, device=dev) for s in SHAPES]
    cfg = BasicConfig(rank=rank, num_iters_per_step=iters)
    ours = BasicPowerSGD(params, cfg, backend="native")
    oracle = BasicPowerSGD(params, cfg, backend="torch")
    ga = _grads(SHAPES, dev, 0)
    gb = [g.clone() for g in ga]
    for step in range(3):
        before = [g.clone() for g in ga]
        oa = [o.clone() for o in ours.aggregate(ga)]
        ob = oracle.aggregate(gb)
        torch.cuda.synchronize()
        assert ours._native.uses_tensor_cores
        assert ours._native._status.value == 0, "a bounded wait inside the tensor-core kernel ran out"
        for x, y, b, res in zip(oa, ob, before, ga):
            assert torch.isfinite(x).all()
            assert _rel(x, y) < tol, (step, tuple(x.shape), _rel(x, y))
            assert _rel(x + res, b) < 1e-6
        for x, y in zip(ga, gb):
            assert _rel(x, y) < tol, (step, tuple(x.shape), _rel(x, y))
            if precision == "split":
                # the compression error itself (norm of the residual) agrees to 1e-5 relative
                gap = abs(x.double().norm().item() - y.double().norm().item())
                assert gap <= (1e-5 if rank <= 8 else 1e-4) * y.double().norm().item(), (step, tuple(x.shape), gap)
        fresh = _grads(SHAPES, dev, 50 + step)
        for x, y, f in zip(ga, gb, fresh):
            x.add_(f)
            y.add_(f)


def test_long_accumulation_chains_keep_float32_accuracy(monkeypatch):
    """50 257 rows: every output of `M^T P` sums over chains far longer than one TMEM accumulation
    segment (512 rows), so the hand-over between the two accumulators and the FP32 running sum are
    what is under test. Compression error within 1e-5 relative of the float32 formulation."""
    monkeypatch.setenv("PSGD_B200_GEMM", "tc")
    monkeypatch.setenv("PSGD_B200_TC_PRECISION", "split")
    dev = torch.device("cuda:0")
    shapes = [(50257, 128), (4096, 256)]
    params = [torch.zeros(s, device=dev) for s in shapes]
    cfg = BasicConfig(rank=4, num_iters_per_step=2)
    ours = BasicPowerSGD(params, cfg, backend="native")
    oracle = BasicPowerSGD(params, cfg, backend="torch")
    ga = _grads(shapes, dev, 7)
    gb = [g.clone() for g in ga]
    for step in range(2):
        oa = [o.clone() for o in ours.aggregate(ga)]
        ob = oracle.aggregate(gb)
        torch.cuda.synchronize()
        assert ours._native.uses_tensor_cores and ours._native._status.value == 0
        for x, y in zip(oa, ob):
            assert _rel(x, y) < 1e-4, (step, tuple(x.shape), _rel(x, y))
        for x, y in zip(ga, gb):
            gap = abs(x.double().norm().item() - y.double().norm().item())
            assert gap <= 1e-5 * y.double().norm().item(), (step, tuple(x.shape), gap)
        fresh = _grads(shapes, dev, 70 + step)
        for x, y, f in zip(ga, gb, fresh):
            x.add_(f)
            y.add_(f)


def test_tensor_core_path_is_deterministic(monkeypatch):
    monkeypatch.setenv("PSGD_B200_GEMM", "tc")
    dev = torch.device("cuda:0")
    params = [torch.zeros(s, device=dev) for s in SHAPES]
    runs = []
    for _ in range(2):
        core = BasicPowerSGD(params, BasicConfig(rank=4, num_iters_per_step=2), backend="native")
        g = _grads(SHAPES, dev, 3)
        runs.append([t.clone() for t in core.aggregate(g)] + [t.clone() for t in g])
    for x, y in zip(*runs):
        assert torch.equal(x, y)


def test_tensor_core_fused_sgd_matches_torch_optimizer(monkeypatch):
    """Fused SGD through the tensor-core finalize kernel (TMA tile, TMEM update, coalesced RMW)."""
    from powersgd_b200 import Config, PowerSGD, optimizer_step

    monkeypatch.setenv("PSGD_B200_GEMM", "tc")
    monkeypatch.setenv("PSGD_B200_FINALIZE", "tc")
    dev = torch.device("cuda:0")

    def make():
        torch.manual_seed(2)
        return torch.nn.Sequential(torch.nn.Linear(256, 384), torch.nn.ReLU(), torch.nn.Linear(384, 132),
                                   torch.nn.ReLU(), torch.nn.Linear(132, 10)).to(dev)

    ma, mb = make(), make()
    kw = dict(lr=0.05, momentum=0.9, nesterov=True, weight_decay=1e-4)
    oa, ob = torch.optim.SGD(ma.parameters(), **kw), torch.optim.SGD(mb.parameters(), **kw)
    cfg = Config(rank=4, min_compression_rate=2, num_iters_per_step=2, start_compressing_after_num_steps=0)
    pa = PowerSGD(list(ma.parameters()), cfg, backend="native")
    pb = PowerSGD(list(mb.parameters()), cfg, backend="torch")
    x, y = torch.randn(64, 256, device=dev), torch.randint(0, 10, (64,), device=dev)
    for step in range(3):
        for m in (ma, mb):
            torch.nn.functional.cross_entropy(m(x), y).backward()
        optimizer_step(oa, pa)
        optimizer_step(ob, pb)
        torch.cuda.synchronize()
        native = pa._powersgd._native
        assert native.uses_tensor_cores and native._tiles_dev["fin"]["tc"][1] > 0
        assert native._status.value == 0
        for p, q in zip(ma.parameters(), mb.parameters()):
            assert _rel(p.detach(), q.detach()) < 1e-5, step
            assert _rel(p.grad, q.grad) < 5e-5 or q.grad.norm() == 0, step
