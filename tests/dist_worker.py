"""Multi-rank scenarios, run as `python -m torch.distributed.run ... tests/dist_worker.py NAME`.

Every scenario prints `SCENARIO-OK` on rank 0 when its checks pass; the pytest wrappers look
for that line. Device scenarios use NCCL (one rank per GPU); host scenarios use gloo.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def _init(backend):
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if backend == "nccl":
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return rank, world, torch.device("cuda", local)
    dist.init_process_group("gloo")
    return rank, world, torch.device("cpu")


def _same_on_all_ranks(t, world):
    gathered = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(gathered, t.contiguous())
    return all(torch.equal(gathered[0], g) for g in gathered)


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30)).item()


# ------------------------------------------------------------------------------------------
def scenario_channel_allreduce():
    rank, world, dev = _init("nccl")
    from powersgd_b200.parallel.symm import Channel

    ch = Channel(1 << 20, timeout_ms=5000)
    for it, n in enumerate([1, 7, 1000, 4097, 1 << 16, 1 << 20, 333]):
        g = torch.Generator(device="cpu").manual_seed(100 * it + rank)
        x = torch.randn(n, generator=g).to(dev)
        ref = x.clone()
        dist.all_reduce(ref)
        ch.all_reduce_(x)
        torch.cuda.synchronize()
        ch.check()
        assert _rel(x, ref) < 1e-6, (n, _rel(x, ref))
        assert _same_on_all_ranks(x, world)
    # all-gather of 4-byte words (floats and integer bit patterns, NaN payloads included)
    for it, n in enumerate([1, 33, 4097, 1 << 18]):
        g = torch.Generator(device="cpu").manual_seed(500 * it + rank)
        words = torch.randint(-(2 ** 31), 2 ** 31 - 1, (n,), generator=g, dtype=torch.int64).to(torch.int32).to(dev)
        expect = [torch.empty_like(words) for _ in range(world)]
        dist.all_gather(expect, words)
        got = ch.all_gather(words)
        torch.cuda.synchronize()
        ch.check()
        assert got.shape == (world, n) and torch.equal(got, torch.stack(expect)), n
    # back-to-back launches without host synchronisation (epoch / double-buffer logic)
    x = torch.full((5000,), float(rank + 1), device=dev)
    for _ in range(50):
        ch.all_reduce_(x, scale=1.0 / world)
    torch.cuda.synchronize()
    ch.check()
    expect = sum(range(1, world + 1)) / world
    assert torch.allclose(x, torch.full_like(x, expect), rtol=1e-5), x[:4]
    dist.barrier()
    ch.close()
    # large messages: the two-shot kernel on a buffer in symmetric memory, several epochs in a row
    from powersgd_b200.parallel.symm import BulkAllReduce

    for n in (5, 3 * 4096 * world + 17, 1 << 21):
        bulk = BulkAllReduce(n, timeout_ms=5000)
        for it in range(3):
            g = torch.Generator(device="cpu").manual_seed(7 * it + rank + n)
            x = torch.randn(n, generator=g).to(dev)
            ref = x.clone()
            dist.all_reduce(ref)
            bulk.buffer.copy_(x)
            out = bulk.all_reduce_()
            torch.cuda.synchronize()
            bulk.check()
            assert _rel(out, ref) < 1e-6, (n, it, _rel(out, ref))
            assert _same_on_all_ranks(out, world)
        dist.barrier()
        bulk.close()
    if rank == 0:
        print("SCENARIO-OK")


def scenario_flat_twoshot():
    """Large uncompressed buffers take the two-shot (reduce-scatter + all-gather) peer-store path,
    plain floats with one flag per chunk. Compare it with the library all-reduce, with and
    without the fused SGD update, for 16-byte aligned tensors and for odd views."""
    rank, world, dev = _init("nccl")
    from powersgd_b200.cuda_path import NativeCompressor, NativeFlatAllReduce, _to_device

    os.environ["PSGD_B200_FLAT"] = "bulk"   # this scenario is about the two-shot kernels, whatever `auto` would take
    shapes = [(1000, 333), (7,), (513, 1025), (3, 3, 3, 3)]  # odd total: the padded tail is exercised

    def alloc(odd):
        # odd: views that start one float into their storage, so the element-wise kernels run
        if not odd:
            return [torch.zeros(*s, device=dev) for s in shapes]
        return [torch.zeros(1 + torch.Size(s).numel(), device=dev)[1:].view(*s) for s in shapes]

    def fresh(step, grads, odd):
        g = torch.Generator(device="cpu").manual_seed(1000 * step + rank)
        if grads is None:
            grads = alloc(odd)
        for t in grads:
            t.copy_(torch.randn(t.shape, generator=g))
        return grads

    def mean_of(grads):
        out = [t.clone() for t in grads]
        for t in out:
            dist.all_reduce(t)
            t.div_(world)
        return out

    for flavour, odd in (("aligned", False), ("odd", True)):
        red, grads = NativeFlatAllReduce(), None
        for step in range(4):
            grads = fresh(step, grads, odd)
            ref = mean_of(grads)
            out = red.aggregate(grads)
            torch.cuda.synchronize()
            assert red.path == "bulk" and red.launches == 4 and red._vec == (0 if odd else 1), (red.path, red.launches)
            red.comm.check()
            for o, r_, t in zip(out, ref, grads):
                assert _rel(o, r_) < 1e-6, (flavour, step, _rel(o, r_))
                assert _same_on_all_ranks(o, world)
                assert float(t.abs().max()) == 0.0  # inputs are zeroed like the reference's pack
        # fused SGD on the consumer side
        params = alloc(odd)
        for p_ in params:
            p_.copy_(torch.randn(p_.shape, device=dev))
            dist.broadcast(p_, 0)
        moms = alloc(odd)
        expect = [p_.clone() for p_ in params]
        hyper = NativeCompressor._default_hyper()
        hyper["lr"], hyper["momentum"], hyper["has_momentum"], hyper["one_minus_dampening"] = 0.1, 0.9, 1, 1.0
        hyper_dev = _to_device(hyper, dev)
        red2, grads, ref_moms = NativeFlatAllReduce(), None, None
        for step in range(3):
            grads = fresh(50 + step, grads, odd)
            mean = mean_of(grads)
            red2.aggregate_and_step(grads, params, moms, [0] * len(grads), hyper_dev)
            torch.cuda.synchronize()
            red2.comm.check()
            if ref_moms is None:
                ref_moms = [gm.clone() for gm in mean]
            else:
                for rm, gm in zip(ref_moms, mean):
                    rm.mul_(0.9).add_(gm)
            for e, rm in zip(expect, ref_moms):
                e.add_(rm, alpha=-0.1)
            for p_, e in zip(params, expect):
                assert _rel(p_, e) < 1e-5, (flavour, step, _rel(p_, e))
                assert _same_on_all_ranks(p_, world)
        dist.barrier()
        red.comm.close()
        red2.comm.close()
    if rank == 0:
        print("SCENARIO-OK")


def scenario_channel_timeout():
    """One rank stays away from a collective: the others' bounded waits give up, the kernels
    drain, the status word is set and the context stays usable."""
    rank, world, dev = _init("nccl")
    from powersgd_b200.parallel.symm import Channel, PowerSGDCommTimeout

    ch = Channel(4096, timeout_ms=300)
    x = torch.ones(1024, device=dev)
    raised = False
    if rank != world - 1:
        ch.all_reduce_(x)
        torch.cuda.synchronize()
        try:
            ch.check()
        except PowerSGDCommTimeout:
            raised = True
        assert raised, "expected a timeout status"
        # the device is still healthy
        y = torch.arange(10, device=dev).sum().item()
        assert y == 45
    dist.barrier()
    ch.close()
    if rank == 0:
        print("SCENARIO-OK")


def scenario_powersgd_native():
    rank, world, dev = _init("nccl")
    from powersgd_b200 import Config, PowerSGD

    shapes = [(64, 3, 3, 3), (64, 64, 3, 3), (64, 64, 3, 3), (10, 512), (130, 650), (64,), (10,), (300, 1200)]
    params = [torch.zeros(s, device=dev) for s in shapes]
    cfg = Config(rank=2, min_compression_rate=2, num_iters_per_step=2, start_compressing_after_num_steps=1)
    ours = PowerSGD(params, cfg, backend="native")
    oracle = PowerSGD(params, cfg, backend="torch")
    g = torch.Generator().manual_seed(rank)
    ga = [torch.randn(s, generator=g).to(dev) for s in shapes]
    gb = [x.clone() for x in ga]
    for step in range(4):
        mean_in = [x.clone() for x in ga]
        for x in mean_in:
            dist.all_reduce(x)
            x.div_(world)
        oa = [o.clone() for o in ours.aggregate(ga)]
        ob = oracle.aggregate(gb)
        torch.cuda.synchronize()
        for x, y in zip(oa, ob):
            assert _rel(x, y) < 5e-5, (step, x.shape, _rel(x, y))
            assert _same_on_all_ranks(x, world), "outputs differ between ranks"
        for x, y, keep in zip(ga, gb, ours.is_compressed_mask):
            if keep:
                assert _rel(x, y) < 5e-5
        # mean_i(residual_i) + output == mean_i(input_i)
        for res, out, m in zip(ga, oa, mean_in):
            r = res.clone()
            dist.all_reduce(r)
            r.div_(world)
            assert _rel(r + out, m) < 1e-5
        assert _same_on_all_ranks(ours._powersgd._ps_buffer, world)
        assert _same_on_all_ranks(ours._powersgd._qs_buffer, world)
        noise = [torch.randn(s, generator=g).to(dev) for s in shapes]
        for x, y, z in zip(ga, gb, noise):
            x.add_(z)
            y.add_(z)
    comm = ours._powersgd._native.comm
    if os.environ.get("PSGD_B200_COMM", "p2p") == "p2p":
        assert comm is not None, "expected the in-kernel all-reduce path"
        comm.check()
    else:
        assert comm is None
    dist.barrier()
    if rank == 0:
        print("SCENARIO-OK")


def scenario_powersgd_native_nccl():
    scenario_powersgd_native()


def scenario_train_step_graph():
    rank, world, dev = _init("nccl")
    from powersgd_b200 import Config, PowerSGD
    from powersgd_b200.engine import TrainStep
    from powersgd_b200.models import ResNet18

    torch.manual_seed(0)
    model = ResNet18().to(dev)
    params = list(model.parameters())
    opt = torch.optim.SGD(params, lr=0.05, momentum=0.9, nesterov=True, weight_decay=1e-4)
    agg = PowerSGD(params, Config(rank=2, num_iters_per_step=2, start_compressing_after_num_steps=0))
    step = TrainStep(model, torch.nn.functional.cross_entropy, opt, agg, cuda_graph=True)
    g = torch.Generator().manual_seed(10 + rank)
    losses = []
    for i in range(8):
        x = torch.randn(32, 3, 32, 32, generator=g).to(dev)
        y = torch.randint(0, 10, (32,), generator=g).to(dev)
        losses.append(float(step(x, y).item()))
    torch.cuda.synchronize()
    assert step._graphs, "the step was never captured"
    assert all(l == l for l in losses), losses
    for p in params:
        assert _same_on_all_ranks(p.detach(), world), "replicas drifted"
    dist.barrier()
    if rank == 0:
        print("SCENARIO-OK", losses[0], losses[-1])


def scenario_reducers_native():
    """RankK / HalfRankK / Exact reducers of the research harness on the native kernels (factors
    exchanged by the product kernels' peer pushes) against the unmodified upstream classes on the
    library all-reduce: outputs, memories and bit counts agree; outputs identical on all ranks."""
    import importlib.util

    rank, world, dev = _init("nccl")
    path = os.path.join(ROOT, "baseline", "_ref", "paper_code", "gradient_reducers.py")
    if not os.path.exists(path):
        if rank == 0:
            print("SCENARIO-OK (upstream research code not installed: nothing to compare)")
        return
    sys.path.insert(0, os.path.dirname(path))
    spec = importlib.util.spec_from_file_location("_upstream_reducers", path)
    up = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(up)
    import contextlib

    from powersgd_b200.paper import reducers as ours_mod

    class _Timer:
        def __call__(self, *a, **k):
            return contextlib.nullcontext()

    shapes = [(64, 3, 3, 3), (64, 64, 3, 3), (130, 650), (300, 1200), (10, 512), (64,), (10,)]
    for name, kwargs in (("RankKReducer", dict(rank=2, reuse_query=True)), ("HalfRankKReducer", dict(rank=2)), ("ExactReducer", dict())):
        theirs = getattr(up, name)(random_seed=5, device=dev, timer=_Timer(), **kwargs)
        # the upstream base class draws a 512 MB table nothing reads, advancing its random stream
        del theirs.precalc_numbers
        import numpy as np

        theirs.rng = np.random.RandomState(5)
        ours = getattr(ours_mod, name)(random_seed=5, device=dev, **kwargs)
        mem_a = [torch.zeros(s, device=dev) for s in shapes]
        mem_b = [torch.zeros(s, device=dev) for s in shapes]
        g = torch.Generator().manual_seed(100 + rank)
        for step in range(4):
            grads = []
            for s in shapes:
                if len(s) == 1:
                    grads.append(torch.randn(s, generator=g).to(dev))
                else:
                    n = s[0]
                    m = int(torch.Size(s).numel() // n)
                    a = torch.randn(n, 5, generator=g) @ torch.randn(5, m, generator=g) + 0.1 * torch.randn(n, m, generator=g)
                    grads.append(a.view(s).to(dev))
            send_a = [x + m for x, m in zip(grads, mem_a)]
            send_b = [x + m for x, m in zip(grads, mem_b)]
            out_a = [torch.full(s, float("nan"), device=dev) for s in shapes]
            out_b = [torch.zeros(s, device=dev) for s in shapes]
            bits_a = ours.reduce(send_a, out_a, mem_a)
            bits_b = theirs.reduce(send_b, out_b, mem_b)
            torch.cuda.synchronize()
            assert bits_a == bits_b, (name, step, bits_a, bits_b)
            for s, x, y, ma, mb in zip(shapes, out_a, out_b, mem_a, mem_b):
                assert _rel(x, y) < 3e-5, (name, step, s, _rel(x, y))
                assert _same_on_all_ranks(x, world), (name, "outputs differ between ranks")
                if float(mb.norm()) > 0:
                    assert _rel(ma, mb) < 3e-5, (name, step, s, _rel(ma, mb))
        native = getattr(ours, "_native", None)
        assert native is not None, name
        comm = native.comp.comm if hasattr(native, "comp") else native.comm
        assert comm is not None, "expected the in-kernel all-reduce path"
        comm.check()
        dist.barrier()
    if rank == 0:
        print("SCENARIO-OK")


def _check_mean_accumulator(rank, world, dev):
    """Count-weighted merge of nested accumulators with one collective over all leaves."""
    from powersgd_b200.utils import MeanAccumulator

    acc = MeanAccumulator()
    # rank r adds r + 1 samples; sample j of rank r is {"loss": r + j, "vec": [r, j, 1], "pair": [r, 2 j]}
    for j in range(rank + 1):
        acc.add({"loss": float(rank + j), "vec": torch.tensor([float(rank), float(j), 1.0], device=dev), "pair": [float(rank), 2.0 * j]})
    acc.reduce()
    got = acc.value()
    n_total = sum(r + 1 for r in range(world))
    want_loss = sum(float(r + j) for r in range(world) for j in range(r + 1)) / n_total
    want_vec = [sum(float(r) for r in range(world) for j in range(r + 1)) / n_total,
                sum(float(j) for r in range(world) for j in range(r + 1)) / n_total, 1.0]
    assert abs(got["loss"] - want_loss) < 1e-5, (got["loss"], want_loss)
    assert torch.allclose(got["vec"].cpu(), torch.tensor(want_vec), atol=1e-5), (got["vec"], want_vec)
    assert abs(got["pair"][0] - want_vec[0]) < 1e-5 and abs(got["pair"][1] - 2 * want_vec[1]) < 1e-5, got["pair"]
    assert abs(acc.average["loss"].counter - n_total) < 1e-6


def scenario_mean_accumulator_gloo():
    rank, world, dev = _init("gloo")
    _check_mean_accumulator(rank, world, dev)
    if rank == 0:
        print("SCENARIO-OK")


def scenario_sparse_reducers_native():
    """Top-k reducers (native select, in-kernel all-gather, cooperative scatter-combine) against the
    unmodified upstream classes; the metric accumulator on the in-kernel all-reduce."""
    import contextlib
    import importlib.util

    import numpy as np

    rank, world, dev = _init("nccl")
    _check_mean_accumulator(rank, world, dev)
    path = os.path.join(ROOT, "baseline", "_ref", "paper_code", "gradient_reducers.py")
    if not os.path.exists(path):
        if rank == 0:
            print("SCENARIO-OK (upstream research code not installed: nothing to compare)")
        return
    sys.path.insert(0, os.path.dirname(path))
    spec = importlib.util.spec_from_file_location("_upstream_reducers", path)
    up = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(up)
    from powersgd_b200.ops.topk import sparse_combine_status
    from powersgd_b200.paper import reducers as ours_mod

    class _Timer:
        def __call__(self, *a, **k):
            return contextlib.nullcontext()

    shapes = [(64, 3, 3, 3), (64, 64, 3, 3), (130, 650), (300, 1200), (10, 512), (64,), (1000,)]
    for name in ("TopKReducer", "GlobalTopKReducer"):
        theirs = getattr(up, name)(random_seed=5, device=dev, timer=_Timer(), compression=0.05)
        del theirs.precalc_numbers
        theirs.rng = np.random.RandomState(5)
        ours = getattr(ours_mod, name)(random_seed=5, device=dev, compression=0.05)
        g = torch.Generator().manual_seed(200 + rank)
        for step in range(3):
            # distinct magnitudes: no ties at the threshold, so both selections agree
            grads = [torch.randn(s, generator=g).to(dev) for s in shapes]
            out_a = [torch.full(s, float("nan"), device=dev) for s in shapes]
            out_b = [torch.zeros(s, device=dev) for s in shapes]
            mem_a = [torch.full(s, float("nan"), device=dev) for s in shapes]
            mem_b = [torch.zeros(s, device=dev) for s in shapes]
            bits_a = ours.reduce([x.clone() for x in grads], out_a, mem_a)
            bits_b = theirs.reduce([x.clone() for x in grads], out_b, mem_b)
            torch.cuda.synchronize()
            assert bits_a == bits_b, (name, step, bits_a, bits_b)
            for s, x, y, ma, mb in zip(shapes, out_a, out_b, mem_a, mem_b):
                assert torch.allclose(x, y, atol=1e-6), (name, step, s, (x - y).abs().max().item())
                assert torch.equal(ma, mb), (name, step, s)
                assert _same_on_all_ranks(x, world), (name, "outputs differ between ranks")
        assert sparse_combine_status(dev) == 0
        dist.barrier()
    # ATOMO: native SVD of the narrow matrices, payloads through the in-kernel all-gather of the staging buffer
    atomo = ours_mod.AtomoReducer(random_seed=5, device=dev, rank=2)
    small = [(24, 3, 3, 3), (16, 24), (10, 16), (24,)]
    g = torch.Generator().manual_seed(400 + rank)
    for step in range(2):
        grads = [torch.randn(s, generator=g).to(dev) for s in small]
        outs = [torch.full(s, float("nan"), device=dev) for s in small]
        mems = [torch.zeros(s, device=dev) for s in small]
        bits = atomo.reduce(grads, outs, mems)
        torch.cuda.synchronize()
        assert bits > 0
        for x in outs:
            assert bool(torch.isfinite(x).all()) and _same_on_all_ranks(x, world), "ATOMO outputs differ between ranks"
    dist.barrier()
    if rank == 0:
        print("SCENARIO-OK")


def scenario_nvls_allreduce():
    """In-switch all-reduce (multimem kernel between two bounded barriers) against the library
    all-reduce, directly and as the PSGD_B200_FLAT=nvls path of the flat aggregator. Never part of a
    failure test: every rank closes the buffer (collective) before leaving."""
    rank, world, dev = _init("nccl")
    from powersgd_b200.parallel.nvls import NvlsAllReduce, NvlsUnavailable

    g = torch.Generator().manual_seed(300 + rank)
    # barriers inside the launch / as two token all-reduces around it; memory bound by this package's
    # runtime / by PyTorch's symmetric-memory runtime
    for fused, runtime in (("1", "native"), ("0", "native"), ("1", "torch")):
        os.environ["PSGD_B200_NVLS_FUSED"] = fused
        os.environ["PSGD_B200_NVLS_RUNTIME"] = runtime
        try:
            red = NvlsAllReduce(3 * 1000 * 1000 + 5)
        except NvlsUnavailable as exc:
            if rank == 0:
                print(f"SCENARIO-OK (no NVLink multicast here: {exc})")
            return
        assert red.launches == (1 if fused == "1" else 3)
        assert red.runtime == runtime, f"asked for the {runtime} runtime, got {red.runtime}"
        for step in range(3):
            data = torch.randn(red.n_pad, generator=g).to(dev)
            red.buffer.copy_(data)
            red.all_reduce_()
            want = data.clone()
            dist.all_reduce(want)
            torch.cuda.synchronize()
            red.check()
            assert _rel(red.buffer, want) < 1e-6, (fused, step, _rel(red.buffer, want))
            assert _same_on_all_ranks(red.buffer, world), "replicas differ"
        red.close()
    del os.environ["PSGD_B200_NVLS_FUSED"], os.environ["PSGD_B200_NVLS_RUNTIME"]
    # the flat aggregator on the same path
    os.environ["PSGD_B200_FLAT"] = "nvls"
    from powersgd_b200.cuda_path import NativeFlatAllReduce

    flat = NativeFlatAllReduce()
    shapes = [(1000, 700), (300, 1200), (513,), (64, 3, 3, 3)]
    for step in range(2):
        grads = [torch.randn(s, generator=g).to(dev) for s in shapes]
        want = [x.clone() for x in grads]
        for w in want:
            dist.all_reduce(w)
            w.div_(world)
        got = flat.aggregate(grads)
        torch.cuda.synchronize()
        assert flat.path == "nvls", flat.path
        for a, b in zip(got, want):
            assert _rel(a, b) < 1e-6, (step, tuple(a.shape), _rel(a, b))
            assert _same_on_all_ranks(a, world)
    flat.close()
    del os.environ["PSGD_B200_FLAT"]
    dist.barrier()
    if rank == 0:
        print("SCENARIO-OK")


def scenario_paper_train_native():
    """The research training loop on GPUs (one rank each) for every family of reducers, a few
    batches of ResNet-18 on synthetic CIFAR: the native select / sign / low-rank / scatter-combine
    kernels, the in-kernel all-gather and all-reduce and the metric accumulator under a real model.
    Parameters stay bit-identical across ranks and finite."""
    import tempfile

    from powersgd_b200.paper import train

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    base = dict(train.config)
    cases = [("RankKReducer", dict(optimizer_reducer_rank=2)), ("HalfRankKReducer", dict(optimizer_reducer_rank=2)),
             ("ExactReducer", {}), ("TopKReducer", dict(optimizer_reducer_compression=0.01)),
             ("GlobalTopKReducer", dict(optimizer_reducer_compression=0.01)), ("SignSGDwithMajorityVoteReducer", {}),
             ("SignAndNormReducer", {}), ("RandomSparseReducer", dict(optimizer_reducer_rank=2))]
    for name, extra in cases:
        train.config.clear()
        train.config.update(base)
        train.config.update(num_epochs=1, optimizer_batch_size=32, max_batches_per_epoch=3, log_verbosity=0, train_size=512, test_size=64,
                            task_architecture="ResNet18", distributed_backend="nccl", optimizer_scale_lr_with_warmup_epochs=0,
                            optimizer_learning_rate=0.01, optimizer_conv_learning_rate=0.01, optimizer_reducer=name, **extra)
        train.output_dir = tempfile.mkdtemp(prefix=f"psgd_{name}_")
        task, reducer, bits = train.main()
        dev = task.state[0].device
        torch.cuda.synchronize()
        assert bits > 0, name
        for p in task.state:
            assert bool(torch.isfinite(p).all()), name
        flat = torch.cat([p.detach().reshape(-1).float() for p in task.state])
        assert _same_on_all_ranks(flat, world), (name, "replicas diverged")
        dist.barrier()
    if rank == 0:
        print("SCENARIO-OK")


def scenario_train_step_timeout():
    """A rank stays away from a training step: the others' bounded device-side waits give up, and
    their NEXT call of the training step raises (naming the step) instead of applying an update
    that is missing a contribution. Made on the host: nothing faults, traps or hangs a GPU, and
    the rank that stays away leaves nothing in flight."""
    import datetime

    rank, world, dev = _init("nccl")
    from powersgd_b200 import Config, PowerSGD
    from powersgd_b200.engine import TrainStep
    from powersgd_b200.parallel.symm import PowerSGDCommTimeout

    assert float(os.environ.get("PSGD_B200_COMM_TIMEOUT_MS", "0")) <= 1000, "run this scenario with a short limit"
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(128, 256), torch.nn.ReLU(), torch.nn.Linear(256, 10)).to(dev)
    params = list(model.parameters())
    opt = torch.optim.SGD(params, lr=0.05, momentum=0.9)
    agg = PowerSGD(params, Config(rank=2, num_iters_per_step=2, start_compressing_after_num_steps=0))
    step = TrainStep(model, torch.nn.functional.cross_entropy, opt, agg, cuda_graph=True)
    x, y = torch.randn(32, 128, device=dev), torch.randint(0, 10, (32,), device=dev)
    for _ in range(5):
        step(x, y).item()
    assert step._graphs
    torch.cuda.synchronize()
    dist.barrier()
    store = dist.distributed_c10d._get_default_store()
    if rank == world - 1:
        # stays away, between steps, with nothing of its own in flight
        store.wait(["timeout-observed"], datetime.timedelta(seconds=120))
    else:
        raised_after = None
        for extra in range(3):
            try:
                step(x, y).item()
            except PowerSGDCommTimeout as exc:
                raised_after = extra
                assert "training step" in str(exc)
                break
        assert raised_after is not None and raised_after <= 2, raised_after
        # the device still answers
        assert torch.arange(10, device=dev).sum().item() == 45
        if rank == 0:
            store.set("timeout-observed", "1")
    dist.barrier()
    agg.close()
    if rank == 0:
        print("SCENARIO-OK")


def scenario_plan_mismatch_gloo():
    """Ranks that were set up differently are told so at construction, on every rank."""
    rank, world, dev = _init("gloo")
    from powersgd_b200.parallel.symm import PowerSGDConfigMismatch, assert_same_on_all_ranks
    from powersgd_b200.plan import CompressionPlan

    assert_same_on_all_ranks((CompressionPlan.build([(64, 27), (10, 512)], rank=2).signature(), 2, 2), "plan")
    shapes = [(64, 27), (10, 512)] if rank == 0 else [(64, 27), (12, 512)]
    raised = False
    try:
        assert_same_on_all_ranks((CompressionPlan.build(shapes, rank=2).signature(), 2, 2), "PowerSGD compression plan")
    except PowerSGDConfigMismatch as exc:
        raised = "compression plan" in str(exc)
    assert raised
    dist.barrier()
    if rank == 0:
        print("SCENARIO-OK")


def scenario_mlp_gloo():
    """The plumbing configuration: 2-layer MLP on CPU ranks; parameters stay bit-identical."""
    rank, world, dev = _init("gloo")
    from powersgd_b200 import Config, PowerSGD, optimizer_step

    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(784, 256), torch.nn.ReLU(), torch.nn.Linear(256, 10))
    params = list(model.parameters())
    opt = torch.optim.SGD(params, lr=0.1, momentum=0.9)
    agg = PowerSGD(params, Config(rank=1, min_compression_rate=10, num_iters_per_step=2, start_compressing_after_num_steps=0))
    assert agg.is_compressed_mask == [True, False, False, False]
    g = torch.Generator().manual_seed(1 + rank)
    first = last = None
    for step in range(20):
        x = torch.randn(64, 784, generator=g)
        y = torch.randint(0, 10, (64,), generator=g)
        loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        optimizer_step(opt, agg)
        first = loss.item() if first is None else first
        last = loss.item()
    for p in params:
        assert _same_on_all_ranks(p.detach(), world)
    assert _same_on_all_ranks(agg._powersgd._ps_buffer, world)
    dist.barrier()
    if rank == 0:
        print("SCENARIO-OK", first, last)


def scenario_ef_identity_gloo():
    rank, world, dev = _init("gloo")
    from powersgd_b200 import Config, PowerSGD
    from powersgd_b200.ops.emulate import emulated_aggregate

    shapes = [(20, 30), (20, 30), (16, 3, 3, 3), (7,)]
    params = [torch.zeros(s) for s in shapes]
    agg = PowerSGD(params, Config(rank=2, min_compression_rate=1.5, num_iters_per_step=3, start_compressing_after_num_steps=0))
    g = torch.Generator().manual_seed(rank)
    grads = [torch.randn(s, generator=g) for s in shapes]
    mean_in = [x.clone() for x in grads]
    for x in mean_in:
        dist.all_reduce(x)
        x.div_(world)
    # the kernel pipeline's algebra, with a gloo all-reduce in place of the peer pushes
    core = agg._powersgd
    twin = [x.clone() for x, keep in zip(grads, agg.is_compressed_mask) if keep]
    import copy

    core_twin = copy.deepcopy(core)
    out_twin = emulated_aggregate(core_twin, twin, allreduce=dist.all_reduce)
    out = agg.aggregate(grads)
    k = 0
    for o, keep in zip(out, agg.is_compressed_mask):
        if keep:
            assert _rel(out_twin[k], o) < 1e-4, _rel(out_twin[k], o)
            k += 1
    for o, res, m in zip(out, grads, mean_in):
        assert _same_on_all_ranks(o, world)
        r = res.clone()
        dist.all_reduce(r)
        r.div_(world)
        assert torch.allclose(r + o, m, atol=1e-5)
    dist.barrier()
    if rank == 0:
        print("SCENARIO-OK")


def scenario_rank_failure_gloo():
    """A rank that raises before a collective: the others' next collective ends with an error
    (short process-group timeout) instead of hanging."""
    import datetime

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=3))
    from powersgd_b200 import AllReduce

    ok = AllReduce().aggregate([torch.ones(4)])
    assert torch.allclose(ok[0], torch.ones(4))
    if rank == world - 1:
        print("SCENARIO-OK-FAILING-RANK-LEFT")
        os._exit(0)  # leaves between steps, nothing in flight
    failed = False
    try:
        AllReduce().aggregate([torch.ones(4)])
    except Exception:
        failed = True
    assert failed, "expected the collective to fail once a rank is gone"
    if rank == 0:
        print("SCENARIO-OK")
    os._exit(0)


def scenario_ddp_hooks_gloo():
    """The DDP comparison harness with each built-in hook, two CPU ranks."""
    import datetime

    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=60))
    from powersgd_b200.paper import train_ddp

    for hook in ("allreduce", "PowerSGD"):
        train_ddp.config.update(distributed_backend="gloo", device="cpu", num_epochs=1, max_batches_per_epoch=3,
                                optimizer_batch_size=8, task_architecture="LeNet", train_size=64, test_size=32,
                                log_verbosity=0, optimizer_reducer=hook, start_powerSGD_iter=2,
                                rank=dist.get_rank(), n_workers=dist.get_world_size())
        task, bits = train_ddp.main()
        assert bits >= 0
        for p in task.state:
            assert torch.isfinite(p).all()
            assert _same_on_all_ranks(p.detach(), dist.get_world_size())
    if dist.get_rank() == 0:
        print("SCENARIO-OK")


def scenario_preflight_gloo():
    """The node preflight as CPU ranks: library all-reduce smoke test, one JSON report."""
    from powersgd_b200.paper import environment

    report = environment.main(backend="gloo")
    assert report["ok"] and report["checks"]["library_all_reduce"] and report["world"] == dist.get_world_size()
    if dist.get_rank() == 0:
        print("SCENARIO-OK")


def scenario_preflight():
    """The node preflight on GPUs: adds peer access and the in-kernel all-reduce."""
    from powersgd_b200.paper import environment

    report = environment.main()
    assert report["ok"] and report["checks"]["in_kernel_all_reduce"] and report["device"]["peer_access_to_all"]
    if dist.get_rank() == 0:
        print("SCENARIO-OK")


if __name__ == "__main__":
    globals()["scenario_" + sys.argv[1]]()
    if dist.is_initialized():
        dist.destroy_process_group()
