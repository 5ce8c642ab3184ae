"""Research-harness reducers on the native kernels against the UNMODIFIED upstream classes
(paper-code/gradient_reducers.py, copied under baseline/_ref/paper_code) on the same device."""
import importlib.util
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _upstream():
    path = os.path.join(ROOT, "baseline", "_ref", "paper_code", "gradient_reducers.py")
    if not os.path.exists(path):
        pytest.skip("upstream research code not installed under baseline/_ref/paper_code")
    sys.path.insert(0, os.path.dirname(path))
    spec = importlib.util.spec_from_file_location("_upstream_reducers", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class _Timer:
    def __call__(self, *a, **k):
        import contextlib

        return contextlib.nullcontext()


def _rel(a, b):
    return (a.double() - b.double()).norm().item() / max(b.double().norm().item(), 1e-30)


SHAPES = [(64, 3, 3, 3), (64, 64, 3, 3), (64, 64, 3, 3), (130, 650), (300, 1200), (10, 512), (64,), (10,), (2600, 650)]


def _inputs(dev, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for s in SHAPES:
        if len(s) == 1:
            out.append(torch.randn(s, generator=g).to(dev))
            continue
        n = s[0]
        m = int(torch.Size(s).numel() // n)
        k = min(6, n, m)
        a = torch.randn(n, k, generator=g) @ torch.randn(k, m, generator=g) + 0.1 * torch.randn(n, m, generator=g)
        out.append(a.view(s).to(dev))
    return out


@pytest.fixture
def single_rank_group(tmp_path):
    """The upstream reducers call torch.distributed collectives unconditionally: give them a
    process group of one rank."""
    import torch.distributed as dist

    dist.init_process_group("gloo", init_method=f"file://{tmp_path}/rdv", rank=0, world_size=1)
    yield
    dist.destroy_process_group()


def _plain_base_init(self, random_seed, device, timer):
    """The upstream base class draws a 512 MB table of random numbers that nothing reads (which
    also advances its random stream) and asks torch.distributed for the world size: set the same
    attributes without either."""
    import numpy as np

    self.rng = np.random.RandomState(random_seed)
    self.n_workers, self.rank = 1, 0
    self.device, self.timer = device, timer


@pytest.mark.parametrize("name,kwargs", [("RankKReducer", dict(rank=2, reuse_query=True)), ("RankKReducer", dict(rank=1, reuse_query=True)),
                                          ("RankKReducer", dict(rank=4, reuse_query=False)), ("HalfRankKReducer", dict(rank=2)),
                                          ("ExactReducer", dict())])
def test_native_reducers_match_upstream(name, kwargs, monkeypatch, single_rank_group):
    up = _upstream()
    from powersgd_b200.paper import reducers as ours_mod

    dev = torch.device("cuda:0")
    monkeypatch.setattr(up.Reducer, "__init__", _plain_base_init)
    theirs = getattr(up, name)(random_seed=5, device=dev, timer=_Timer(), **kwargs)
    ours = getattr(ours_mod, name)(random_seed=5, device=dev, **kwargs)
    mem_a = [torch.zeros(s, device=dev) for s in SHAPES]
    mem_b = [torch.zeros(s, device=dev) for s in SHAPES]
    for step in range(4):
        grads = _inputs(dev, 30 + step)
        send_a = [g + m for g, m in zip(grads, mem_a)]
        send_b = [g + m for g, m in zip(grads, mem_b)]
        keep = [t.clone() for t in send_a]
        out_a = [torch.full(s, float("nan"), device=dev) for s in SHAPES]
        out_b = [torch.zeros(s, device=dev) for s in SHAPES]
        bits_a = ours.reduce(send_a, out_a, mem_a)
        bits_b = theirs.reduce(send_b, out_b, mem_b)
        torch.cuda.synchronize()
        assert bits_a == bits_b, (step, bits_a, bits_b)
        for s, x, y, ma, mb, before, now in zip(SHAPES, out_a, out_b, mem_a, mem_b, keep, send_a):
            assert torch.equal(before, now), "inputs must not be modified"
            assert _rel(x, y) < 2e-5, (name, step, s, _rel(x, y))
            if float(mb.norm()) > 0:
                assert _rel(ma, mb) < 2e-5, (name, step, s, _rel(ma, mb))
                gap = abs(ma.double().norm().item() - mb.double().norm().item())
                assert gap <= 1e-5 * mb.double().norm().item(), (name, step, s, gap)
            else:
                assert float(ma.abs().max()) == 0.0
    if name != "ExactReducer":
        assert ours._native is not None and ours._native.launches > 0, "the native path did not run"
        # two product launches, two orthonormalisation launches, one decompression launch, one
        # flat launch for the 1-D tensors (a single worker)
        assert ours._native_launches_last <= 7, ours._native_launches_last
