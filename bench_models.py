#!/usr/bin/env python3
"""Throughput of the other benchmark configurations (the LSTM and GPT-2 configurations), same
protocol and JSON line as bench.py (device-timed K steps after W warm-up steps, max over ranks,
plus the end-to-end figure with pinned H2D input copies and a D2H loss read every step).

    python bench_models.py --model lstm   [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python bench_models.py --model gpt2   ...

lstm: 3 x LSTM(650) tied-embedding language model, vocabulary 33 278, dropout 0.4, float32,
      synthetic Zipf(1) tokens, BPTT 30, batch 64 per GPU, PowerSGD rank 4, SGD lr 1.25,
      gradient-norm clipping 0.4 as in the paper's task. Metric: tokens/s.
gpt2: GPT-2 medium (24 layers, d 1024, 16 heads, vocabulary 50 257, sequence 1024), bf16
      autocast with float32 parameters and gradients, synthetic Zipf(1) tokens, batch 8 per GPU,
      PowerSGD rank 4 x 2 half-iterations, min_compression_rate 10, SGD lr 0.01 momentum 0.9.
      Metric: tokens/s.
The reference arm runs the unmodified upstream package with the same model modules (the
upstream repository has no GPT-2; for the LSTM the upstream model class is used).
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

import bench as headline

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


class LMStep(nn.Module):
    """Language model with its carried hidden state kept in buffers, so that a whole BPTT
    window (forward, loss) is a pure function of the token batch and can be graph-captured."""

    def __init__(self, lm, batch: int):
        super().__init__()
        self.lm = lm
        h, c = lm.init_hidden(batch)
        self.register_buffer("h", h)
        self.register_buffer("c", c)

    def forward(self, tokens):
        logits, (h, c) = self.lm(tokens, (self.h.clone(), self.c.clone()))
        with torch.no_grad():
            self.h.copy_(h)
            self.c.copy_(c)
        return logits.view(-1, logits.size(-1))


class Autocast(nn.Module):
    def __init__(self, inner):
        super().__init__()
        self.inner = inner

    def forward(self, tokens):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            logits = self.inner(tokens)
        return logits.view(-1, logits.size(-1)).float()


def flat_ce(logits, targets):
    return F.cross_entropy(logits, targets.reshape(-1))


def build(model_name: str, impl: str, device, use_graph: bool):
    from powersgd_b200 import Config, PowerSGD
    from powersgd_b200.engine import TrainStep
    from powersgd_b200.models import GPT2, GPT2Config, wikitext2_lstm
    from powersgd_b200.paper.tasks.utils import zipf_tokens

    torch.manual_seed(0)
    if model_name == "lstm":
        batch, seq, vocab = 64, 30, 33278
        if impl == "reference":
            path = os.path.join(ROOT, "baseline", "_ref", "paper_code", "tasks", "language_modeling", "model.py")
            spec = importlib.util.spec_from_file_location("_ref_lm", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            lm = mod.RNNModel("LSTM", vocab, 650, 650, 3, dropout=0.4, tie_weights=True)
        else:
            lm = wikitext2_lstm(vocab)
        model = LMStep(lm.to(device), batch).to(device)
        cfg = dict(rank=4, min_compression_rate=2, num_iters_per_step=1, start_compressing_after_num_steps=0)
        opt_kw = dict(lr=1.25, momentum=0.0)
        shape, tokens_per_step, clip = (seq, batch), seq * batch, 0.4
    else:
        batch, seq, vocab = 8, 1024, 50257
        model = Autocast(GPT2(GPT2Config.medium())).to(device)
        cfg = dict(rank=4, min_compression_rate=10, num_iters_per_step=2, start_compressing_after_num_steps=0)
        opt_kw = dict(lr=0.01, momentum=0.9)
        shape, tokens_per_step, clip = (batch, seq), seq * batch, None
    params = [p for p in model.parameters()]
    optimizer = torch.optim.SGD(params, **opt_kw)
    rank = int(os.environ.get("RANK", "0"))
    stream = zipf_tokens(8 * (tokens_per_step + 1), vocab, seed=77 + rank)
    xs = [stream[i * tokens_per_step : (i + 1) * tokens_per_step].view(shape).pin_memory() for i in range(8)]
    ys = [stream[i * tokens_per_step + 1 : (i + 1) * tokens_per_step + 1].view(shape).pin_memory() for i in range(8)]

    if impl == "ours":
        agg = PowerSGD(params, Config(**cfg))
        step = TrainStep(model, flat_ce, optimizer, agg, cuda_graph=use_graph, grad_clip=clip)
    else:
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        import powersgd as ref

        agg = ref.PowerSGD(params, ref.Config(**cfg))

        class Step:
            launches_per_step = 0
            time_aggregate = False   # switched on for the separate aggregate-timing pass only
            _pair = None

            @property
            def aggregate_ms(self):
                if self._pair is None:
                    return None
                a, b = self._pair
                b.synchronize()
                return a.elapsed_time(b)

            def __call__(self, x, y):
                loss = flat_ce(model(x), y)
                loss.backward()
                if self.time_aggregate:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                if clip is not None:
                    torch.nn.utils.clip_grad_norm_(params, clip)
                ref.optimizer_step(optimizer, agg)
                if self.time_aggregate:
                    b.record()
                    self._pair = (a, b)
                return loss.detach()

        step = Step()
    return step, xs, ys, tokens_per_step, cfg, opt_kw


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=["lstm", "gpt2"], required=True)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "powersgd")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"}))
        return 0
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return 0
    local, world = headline.setup_dist(args.gpus)
    device = torch.device("cuda", local)
    rank = int(os.environ.get("RANK", "0"))
    step, xs_host, ys_host, tokens_per_step, cfg, opt_kw = build(args.model, args.impl, device, not args.no_graph)
    xs_dev, ys_dev = [x.to(device) for x in xs_host], [y.to(device) for y in ys_host]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # at least 3 untimed steps: two run eagerly (cuDNN autotuning, lazy buffers), the third records the graph
    for i in range(max(args.warmup, 3)):
        step(xs_dev[i % 8], ys_dev[i % 8])
    barrier()
    sampler = headline.ClockSampler(local, enabled=rank == 0)
    sampler.start()
    time.sleep(0.3)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    a.record()
    for i in range(args.steps):
        loss = step(xs_dev[i % 8], ys_dev[i % 8])
    b.record()
    barrier()
    dev_ms = max_over_ranks(a.elapsed_time(b))
    x_stage, y_stage = torch.empty_like(xs_dev[0]), torch.empty_like(ys_dev[0])
    barrier()
    c, d = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c.record()
    last = 0.0
    for i in range(args.steps):
        x_stage.copy_(xs_host[i % 8], non_blocking=True)
        y_stage.copy_(ys_host[i % 8], non_blocking=True)
        last = float(step(x_stage, y_stage).item())
    d.record()
    barrier()
    e2e_ms = max_over_ranks(c.elapsed_time(d))
    clocks = sampler.stop()
    agg_ms, agg_how = headline.measure_aggregate(step, xs_dev, ys_dev, args.impl == "reference", max_over_ranks,
                                                 graph=args.impl == "ours" and not args.no_graph, bursts=8, burst_len=5)
    barrier()
    tokens = tokens_per_step * world * args.steps
    if rank == 0:
        print(json.dumps({
            "metric": f"{args.model} tokens/s", "impl": args.impl, "value": tokens / (dev_ms / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "fp32" if args.model == "lstm" else "bf16 autocast, fp32 parameters and gradients",
            "data": "synthetic Zipf(s=1) tokens, random-init weights",
            "config": {"model": args.model, "tokens_per_step_per_gpu": tokens_per_step, "parallelism": f"dp{world}",
                       "powersgd": cfg, "optimizer": opt_kw,
                       "l2": "per-step working set exceeds L2; no explicit flush"},
            "engine": {"cuda_graph": bool(args.impl == "ours" and not args.no_graph), "host_cpus": os.cpu_count()},
            "clocks": clocks,
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": 2 * 8 * tokens_per_step, "d2h_bytes_per_step": 4, "last_loss": last},
            "gpu_launches": getattr(step, "launches_per_step", 0) * args.steps,
            "aggregate_ms_per_step": agg_ms,
            "aggregate_how": agg_how,
        }))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
