#!/usr/bin/env python3
"""Compression micro-benchmark (the second benchmark configuration).

For float32 gradient matrices of the named shapes — each drawn as a rank-8 product of N(0,1)
factors plus N(0, 1e-3) noise — time one `aggregate()` (compress + reduce + decompress +
error feedback) of this library's native kernels against

  * the reference formulation (batched `torch.bmm` / `torch.linalg.qr` + NCCL all-reduce; the
    unmodified upstream package when it is installed under baseline/_ref, else this
    repository's PyTorch restatement of it), and
  * an uncompressed all-reduce of the same gradients (multi-GPU runs),

and report the relative compression error of both. Device-timed with CUDA events per
iteration after warm-up, max over ranks; a buffer larger than L2 is rewritten between timed
iterations when the gradients themselves are smaller than L2.

    python bench_compress.py --shapes 1024x1024,4096x1024 --ranks 1,4 --iters 2 --batch 4
    python -m torch.distributed.run --nproc-per-node 2 ... bench_compress.py ...

One JSON line per (shape, rank, iters) on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 << 20


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="1024x1024,4096x1024,4096x4096,50257x1024")
    ap.add_argument("--ranks", default="1,2,4,8,16")
    ap.add_argument("--iters", default="1,2")
    ap.add_argument("--batch", type=int, default=4, help="matrices per shape (one shape group)")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--skip-reference", action="store_true")
    ap.add_argument("--only-ours", action="store_true", help="time only the native path (used for profiler captures)")
    ap.add_argument("--stages", action="store_true", help="add per-phase device times of the native path to every row")
    ap.add_argument("--model", choices=["resnet18", "lstm"], default=None,
                    help="instead of --shapes: the compressed gradient matrices of this model (ResNet-18 with the CIFAR "
                         "stem: 21 matrices in 12 shape groups; LSTM language model: 33278x650 and 6 x 2600x650), "
                         "per-phase device times with the product kernels on CUDA cores and on tensor cores")
    ap.add_argument("--read-floor", action="store_true",
                    help="add to every row the time of a plain read-only streaming pass over the same gradients "
                         "(the floor of any kernel that reads them once), cold, CUDA events")
    ap.add_argument("--flat-stages", action="store_true",
                    help="multi-GPU: per-stage device times of the uncompressed peer-store all-reduce (pack, "
                         "scatter + reduce, unpack) next to the library all-reduce, then exit")
    return ap.parse_args()


def make_gradients(n, m, batch, device, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    out = []
    for _ in range(batch):
        a = torch.randn(n, 8, generator=g).to(device) @ torch.randn(8, m, generator=g).to(device)
        a.add_(torch.randn(n, m, generator=g).to(device), alpha=1e-3 ** 0.5)
        out.append(a)
    return out


def reference_module():
    ref_root = os.path.join(ROOT, "baseline", "_ref")
    if os.path.isdir(os.path.join(ref_root, "powersgd")):
        sys.path.insert(0, ref_root)
        import powersgd

        return powersgd
    return None


def time_aggregate(make_agg, grads, steps, warmup, flush, world, device, stages=None):
    """`stages`: a dict that receives the mean device time of every named phase of the native
    path (CUDA-event pairs between its launches), max over ranks."""
    from powersgd_b200.cuda_path import _Range

    agg = make_agg()
    work = [g.clone() for g in grads]
    times = []
    out = None
    phase = {}
    for i in range(warmup + steps):
        _Range.events = [] if (stages is not None and i >= warmup) else None
        for w, g in zip(work, grads):
            w.copy_(g)  # same input every iteration: the timing does not depend on the residual
        if flush is not None:
            flush.add_(1.0)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        out = agg.aggregate(work)
        b.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(a.elapsed_time(b))
            for name, ea, eb in _Range.events or []:
                phase[name] = phase.get(name, 0.0) + ea.elapsed_time(eb) / steps
    _Range.events = None
    if stages is not None and phase:
        names = sorted(phase)
        t = torch.tensor([phase[k] for k in names], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        stages.update({k: round(float(v), 5) for k, v in zip(names, t)})
    ms = sum(times) / len(times)
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    err = sum(float(w.double().norm() ** 2) for w in work) ** 0.5
    close = getattr(agg, "close", None)
    if close is not None:
        close()  # symmetric arenas are returned now, not when the collector gets to them
    return ms, err, out


def flat_stages(args, world, rank, device):
    """Device time of each stage of NativeFlatAllReduce's two-shot path, max over ranks."""
    import ctypes

    from powersgd_b200.cuda_path import NativeFlatAllReduce, _stream_ptr
    from powersgd_b200.ops import native

    def timed(stages, before):
        acc = [0.0] * len(stages)
        for it in range(args.warmup + args.steps):
            before()
            dist.barrier()
            torch.cuda.synchronize()
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(len(stages) + 1)]
            evs[0].record()
            for i, stage in enumerate(stages):
                stage()
                evs[i + 1].record()
            torch.cuda.synchronize()
            if it >= args.warmup:
                for i in range(len(stages)):
                    acc[i] += evs[i].elapsed_time(evs[i + 1]) / args.steps
        t = torch.tensor(acc, device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    for shape in args.shapes.split(","):
        n, m = (int(v) for v in shape.lower().split("x"))
        grads = [torch.randn(n, m, device=device) for _ in range(args.batch)]
        refill = lambda: [g.normal_() for g in grads]  # noqa: E731
        red = NativeFlatAllReduce()
        red._bind(grads)
        row = {"shape": [n, m], "batch": args.batch, "n_gpus": world, "path": red.path, "mbytes": 4e-6 * n * m * args.batch}
        if red.path == "bulk":
            hyper = red._hyper_dev
            middle = lambda: native.check(  # noqa: E731
                red.lib.psgd_bulk_allreduce_launch(red.comm.ptr, ctypes.c_longlong(red.n_pad), world, _stream_ptr()), "bulk")
            t = timed([lambda: red._launch(0, hyper, float(world)), middle, lambda: red._launch(12, hyper, 1.0)], refill)
            red.comm.check()
            row.update({"pack_ms": t[0], "scatter_reduce_ms": t[1], "unpack_ms": t[2], "whole_path_ms": sum(t)})
        else:
            t = timed([lambda: red.aggregate(grads)], refill)
            row["whole_path_ms"] = t[0]
        red.close()
        flat = torch.cat([g.reshape(-1) for g in grads])
        row["library_allreduce_ms"] = timed([lambda: dist.all_reduce(flat)], lambda: None)[0]
        if rank == 0:
            print(json.dumps(row), flush=True)
        del grads, flat
        torch.cuda.empty_cache()


def read_floor_ms(grads, flush, steps, device) -> float:
    """Best-of-`steps` device time of one read-only streaming pass over all gradient tensors (one
    launch each, back to back, between one CUDA-event pair), caches flushed before every sample."""
    import ctypes

    from powersgd_b200.ops import native

    lib = native.lib()
    sink = torch.zeros(1, device=device)
    scratch = flush if flush is not None else torch.zeros(2 * L2_BYTES // 4, device=device)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    best = float("inf")
    for _ in range(max(steps, 3)):
        scratch.add_(1.0)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for g in grads:
            native.check(lib.psgd_read_pass_launch(ctypes.c_void_p(g.data_ptr()), ctypes.c_longlong(g.numel()), ctypes.c_void_p(sink.data_ptr()),
                                                   148 * 8, stream), "psgd_read_pass_launch")
        b.record()
        torch.cuda.synchronize()
        best = min(best, a.elapsed_time(b))
    return best


def model_table(args, world, rank, device):
    """Per-phase device times of one aggregate() on the gradient shapes of a whole model, once with
    the CUDA-core product kernels and once with the tensor-core ones wherever TMA can address the
    matrix (CUDA-event pairs between the launches, L2 flushed between iterations, max over ranks)."""
    from powersgd_b200 import BasicConfig, BasicPowerSGD, Config
    from powersgd_b200.plan import should_compress

    if args.model == "resnet18":
        from powersgd_b200.models import ResNet18

        net, r, iters = ResNet18(), 2, 2
    else:
        from powersgd_b200.models import wikitext2_lstm

        net, r, iters = wikitext2_lstm(33278), 4, 1
    cfg = Config(rank=r, min_compression_rate=2, num_iters_per_step=iters, start_compressing_after_num_steps=0)
    seen, shapes = set(), []
    for p in net.parameters():
        if id(p) in seen:
            continue  # tied weights
        seen.add(id(p))
        if should_compress(p.shape, cfg):
            shapes.append(tuple(p.shape))
    g = torch.Generator(device="cpu").manual_seed(3 + rank)
    grads = []
    for s_ in shapes:
        n = s_[0]
        m = int(torch.Size(s_).numel() // n)
        a = torch.randn(n, 8, generator=g).to(device) @ torch.randn(8, m, generator=g).to(device)
        a.add_(torch.randn(n, m, generator=g).to(device), alpha=1e-3 ** 0.5)
        grads.append(a.view(s_))
    nbytes = 4 * sum(t.numel() for t in grads)
    flush = torch.zeros(2 * L2_BYTES // 4, device=device)
    for mode in ("ffma", "tc"):
        os.environ["PSGD_B200_GEMM"] = mode
        stages = {}
        ms, err, _ = time_aggregate(lambda: BasicPowerSGD(grads, BasicConfig(rank=r, num_iters_per_step=iters), backend="native"),
                                    grads, args.steps, args.warmup, flush, world, device, stages=stages)
        if rank == 0:
            print(json.dumps({"model": args.model, "matrices": len(grads), "mbytes": nbytes / 1e6, "rank": r, "iters": iters,
                              "n_gpus": world, "products": mode, "ours_ms": ms, "ours_phase_ms": stages,
                              "l2": "flush between iterations"}), flush=True)
    os.environ.pop("PSGD_B200_GEMM", None)


def main():
    args = parse()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    from powersgd_b200 import BasicConfig, BasicPowerSGD

    if args.flat_stages:
        if world < 2:
            raise SystemExit("--flat-stages needs at least two ranks")
        flat_stages(args, world, rank, device)
        dist.destroy_process_group()
        return

    if args.model:
        model_table(args, world, rank, device)
        if world > 1:
            dist.destroy_process_group()
        return

    ref = None if (args.skip_reference or args.only_ours) else reference_module()
    peaks = {}
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        with open(peaks_path) as fp:
            peaks = json.load(fp)
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    hbm_label = "of measured" if peaks else "of fallback"

    for shape in args.shapes.split(","):
        n, m = (int(v) for v in shape.lower().split("x"))
        grads = make_gradients(n, m, args.batch, device, seed=1 + rank)
        nbytes = 4 * n * m * args.batch
        flush = torch.zeros(2 * L2_BYTES // 4, device=device) if nbytes < 2 * L2_BYTES else None
        norm_in = sum(float(g.double().norm() ** 2) for g in grads) ** 0.5
        for r in (int(v) for v in args.ranks.split(",")):
            for iters in (int(v) for v in args.iters.split(",")):
                cfg = BasicConfig(rank=r, num_iters_per_step=iters)
                stages = {} if args.stages else None
                ours_ms, ours_err, _ = time_aggregate(
                    lambda: BasicPowerSGD(grads, cfg, backend="native"), grads, args.steps, args.warmup, flush, world, device,
                    stages=stages,
                )
                row = {
                    "shape": [n, m], "batch": args.batch, "rank": r, "iters": iters, "n_gpus": world,
                    "ours_ms": ours_ms, "ours_rel_error": ours_err / norm_in,
                    "l2": "flush between iterations" if flush is not None else "inputs larger than L2",
                }
                if stages:
                    row["ours_phase_ms"] = stages
                if args.read_floor:
                    row["read_pass_ms"] = read_floor_ms(grads, flush, args.steps, device)
                    row["read_pass_gbs"] = nbytes / (row["read_pass_ms"] * 1e-3) / 1e9
                # algorithmic traffic: `iters` reads of M, then read M + write residual + write update
                traffic = (iters + 3) * nbytes
                row["ours_gbs"] = traffic / (ours_ms * 1e-3) / 1e9
                row["ours_hbm_fraction"] = f"{row['ours_gbs'] / hbm:.3f} {hbm_label} {hbm:.0f} GB/s"
                if not args.only_ours:
                    if ref is not None:
                        make_ref = lambda: ref.powersgd.BasicPowerSGD(grads, ref.powersgd.BasicConfig(rank=r, num_iters_per_step=iters))  # noqa: E731
                        label = "upstream package"
                    else:
                        make_ref = lambda: BasicPowerSGD(grads, cfg, backend="torch")  # noqa: E731
                        label = "PyTorch restatement"
                    ref_ms, ref_err, _ = time_aggregate(make_ref, grads, args.steps, args.warmup, flush, world, device)
                    row.update({"reference_ms": ref_ms, "reference_rel_error": ref_err / norm_in, "reference_impl": label,
                                "speedup": ref_ms / ours_ms,
                                "rel_error_gap": abs(ours_err - ref_err) / max(ref_err, 1e-30)})
                    if world > 1:
                        flat = torch.cat([g.reshape(-1) for g in grads])
                        ts = []
                        for i in range(args.warmup + args.steps):
                            dist.barrier()
                            torch.cuda.synchronize()
                            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                            a.record()
                            dist.all_reduce(flat)
                            b.record()
                            torch.cuda.synchronize()
                            if i >= args.warmup:
                                ts.append(a.elapsed_time(b))
                        t = torch.tensor([sum(ts) / len(ts)], device=device, dtype=torch.float64)
                        dist.all_reduce(t, op=dist.ReduceOp.MAX)
                        row["uncompressed_allreduce_ms"] = float(t.item())
                        # the same mean through this library's peer-store kernels (pack + push, owner
                        # sum + push, consume), which can be recorded in a CUDA graph
                        from powersgd_b200.cuda_path import NativeFlatAllReduce

                        class _Flat:
                            def __init__(self):
                                self.red = NativeFlatAllReduce()

                            def aggregate(self, tensors):
                                return self.red.aggregate(tensors)

                            def close(self):
                                self.red.close()

                        flat_ms, _, _ = time_aggregate(_Flat, grads, args.steps, args.warmup, flush, world, device)
                        row["uncompressed_peer_store_allreduce_ms"] = flat_ms
                        if ref is not None:
                            # the upstream package's own uncompressed aggregator: pack (torch.cat), NCCL
                            # all-reduce, divide, unpack - the like-for-like of the line above
                            up_ms, _, _ = time_aggregate(lambda: ref.powersgd.AllReduce(), grads, args.steps, args.warmup, flush, world, device)
                            row["uncompressed_upstream_aggregator_ms"] = up_ms
                if rank == 0:
                    print(json.dumps(row), flush=True)
        del grads, flush
        torch.cuda.empty_cache()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
