"""`batch.reduce` of the research harness: this package's gradient reducers against the unmodified
upstream classes (paper-code/gradient_reducers.py) on the gradient shapes of ResNet-18.

The training loop of the harness spends its communication time in one call per step,
`reducer.reduce(send_buffers, grads, memories)` (paper-code/train.py:184-186, timer label
`batch.reduce`). This script times exactly that call on synthetic gradients of the 62 parameter
shapes of ResNet-18 with the CIFAR stem, for both implementations, on 1..N GPUs:

    python bench_reducers.py --steps 20
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29681 bench_reducers.py --steps 20

CUDA events around each call after warm-up, a 252 MB buffer rewritten between calls (the 44.7 MB of
gradients fit L2), mean over steps, max over ranks. One JSON line per reducer on rank 0; `rel_diff`
is the largest relative difference between the two implementations' outputs on the last step (same
inputs, same starting state).
"""
from __future__ import annotations

import argparse
import contextlib
import importlib.util
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


class _NoTimer:
    def __call__(self, *args, **kwargs):
        return contextlib.nullcontext()


def upstream_module():
    path = os.path.join(ROOT, "baseline", "_ref", "paper_code", "gradient_reducers.py")
    if not os.path.exists(path):
        return None
    sys.path.insert(0, os.path.dirname(path))
    spec = importlib.util.spec_from_file_location("_upstream_reducers", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def resnet18_shapes():
    from powersgd_b200.models import ResNet18

    return [tuple(p.shape) for p in ResNet18().parameters()]


def gradients(shapes, device, seed):
    g = torch.Generator().manual_seed(seed)
    out = []
    for s in shapes:
        if len(s) == 1:
            out.append(torch.randn(s, generator=g).to(device))
        else:
            n, m = s[0], int(np.prod(s[1:]))
            low = torch.randn(n, 4, generator=g) @ torch.randn(4, m, generator=g)
            out.append((low + 0.1 * torch.randn(n, m, generator=g)).view(s).to(device))
    return out


def time_reducer(reducer, grads, steps, warmup, flush, world):
    memories = [torch.zeros_like(g) for g in grads]
    outs = [torch.zeros_like(g) for g in grads]
    send = [torch.empty_like(g) for g in grads]   # persistent, as the harness keeps them (train.py:139-142)
    times = []
    bits = 0
    for i in range(warmup + steps):
        for s, g, m in zip(send, grads, memories):
            torch.add(g, m, out=s)   # train.py:179-182
        flush.add_(1.0)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        bits = reducer.reduce(send, outs, memories)
        b.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(a.elapsed_time(b))
    ms = sum(times) / len(times)
    if world > 1:
        t = torch.tensor([ms], device=grads[0].device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms, bits, outs


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--reducers", default="RankKReducer,HalfRankKReducer,ExactReducer,TopKReducer,GlobalTopKReducer,SignSGDwithMajorityVoteReducer")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    # the upstream classes ask the process group for its size, also in a single-process run
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29682")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    from powersgd_b200.paper import reducers as ours_mod

    up = upstream_module()
    shapes = resnet18_shapes()
    grads = gradients(shapes, device, 100 + rank)
    flush = torch.zeros(63 * 1000 * 1000, device=device)
    kwargs = {
        "RankKReducer": dict(rank=2, reuse_query=True), "HalfRankKReducer": dict(rank=2), "ExactReducer": {},
        "TopKReducer": dict(compression=1 / 244), "GlobalTopKReducer": dict(compression=1 / 244),
        "SignSGDwithMajorityVoteReducer": {}, "SignAndNormReducer": {}, "SignReducer": {},
        "RandomSparseReducer": dict(rank=2), "RandomSparseBlockReducer": dict(rank=2),
        "UniformRandomSparseReducer": dict(compression=1 / 244), "UniformRandomSparseBlockReducer": dict(compression=1 / 244),
    }
    for name in args.reducers.split(","):
        kw = kwargs.get(name, {})
        ours = getattr(ours_mod, name)(random_seed=5, device=device, **kw)
        ours_ms, ours_bits, ours_out = time_reducer(ours, grads, args.steps, args.warmup, flush, world)
        row = {"reducer": name, "n_gpus": world, "tensors": len(shapes), "mbytes": sum(g.numel() for g in grads) * 4 / 1e6,
               "ours_ms": ours_ms, "bits": int(ours_bits), "l2": "flush between calls"}
        if up is not None and hasattr(up, name):
            theirs = getattr(up, name)(random_seed=5, device=device, timer=_NoTimer(), **kw)
            theirs.rng = np.random.RandomState(5)  # the base class draws an unused table first; same stream as ours
            try:
                ref_ms, ref_bits, ref_out = time_reducer(theirs, grads, args.steps, args.warmup, flush, world)
            except NameError as exc:   # the sign reducers need the external bit2byte extension (same on every rank)
                row["upstream"] = f"unavailable: {exc}"
            else:
                diff = max(float((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-30)) for a, b in zip(ours_out, ref_out))
                row.update({"upstream_ms": ref_ms, "speedup": ref_ms / ours_ms, "upstream_bits": int(ref_bits), "rel_diff": diff})
            del theirs
        if rank == 0:
            print(json.dumps(row), flush=True)
        close = getattr(ours, "close", None)
        if close is not None:
            close()
        del ours
        torch.cuda.empty_cache()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
