"""Training-step engine: forward, backward, gradient aggregation and optimizer update as one
replayable CUDA graph.

The reference leaves the step to the user's Python loop (README.md:23-43): a few hundred
eager launches for a CIFAR ResNet plus several hundred more inside `aggregate()`. On a B200
that loop is bound by launch latency, not by the GPU. `TrainStep` keeps the same semantics
(`loss.backward()` accumulates onto the residual left in `.grad`; no `zero_grad`) but records
the whole step once and replays it:

    step = TrainStep(model, loss_fn, optimizer, aggregator)
    for x, y in loader:
        loss = step(x, y)          # tensor on the device; call .item() when you need it

Everything that changes between steps lives in device memory that the graph reads at replay
time: the input batch (copied into static buffers), the learning-rate table (refreshed from
pinned memory), the warm-start factors and the residuals. Steps that are structurally
different run eagerly or get their own graph: the un-compressed warm-up phase, the first
steps (cuDNN autotuning, lazy momentum buffers), and — for an odd `num_iters_per_step` — the
two parities of the power iteration.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from .optim import optimizer_step
from .utils import same_layout


class TrainStep:
    def __init__(
        self,
        model: torch.nn.Module,
        loss_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
        optimizer: torch.optim.Optimizer,
        aggregator,
        cuda_graph: bool = True,
        eager_steps: int = 2,
        channels_last: bool = True,
        grad_clip: Optional[float] = None,
        autotune: bool = True,
        time_aggregate: bool = True,
    ):
        self.model = model
        self.loss_fn = loss_fn
        self.optimizer = optimizer
        self.aggregator = aggregator
        self.device = next(model.parameters()).device
        self.use_graph = bool(cuda_graph) and self.device.type == "cuda"
        self.eager_steps = max(int(eager_steps), 2)
        # 4-D inputs are fed in NHWC (cuDNN's tensor-core convolutions run ~1.7x faster on B200 that
        # way) and 4-D weights, their gradients and momentum buffers are stored channels_last too.
        self.channels_last = bool(channels_last) and self.device.type == "cuda"
        if self.channels_last:
            self._weights_to_channels_last()
        # optional global gradient-norm clipping before aggregation (the LSTM task clips at 0.4)
        self.grad_clip = grad_clip
        # Shapes are static (the step is recorded once and replayed), so the library's
        # convolution algorithms can be picked by measurement during the eager steps instead of
        # by heuristics. Process-wide PyTorch switch; pass autotune=False to leave it alone.
        if autotune and self.device.type == "cuda":
            torch.backends.cudnn.benchmark = True
        self._gather_norm_counters()
        self._steps_done = 0
        self._graphs: Dict[int, torch.cuda.CUDAGraph] = {}
        self._graph_keep: Dict[int, list] = {}
        self._static_x: Optional[torch.Tensor] = None
        self._static_y: Optional[torch.Tensor] = None
        self._static_loss: Optional[torch.Tensor] = None
        self._pool = None
        self._agg_events = None
        # Device time between the end of backward and the end of the parameter update. Eager steps
        # bracket it with ordinary events; a recorded step carries two event-record nodes
        # ("external" events, which a graph replays), so every replay refreshes the pair.
        self.time_aggregate = bool(time_aggregate) and self.device.type == "cuda"
        self._graph_events: Dict[int, tuple] = {}
        self.launches_per_step = 0
        # residuals detached from p.grad for the duration of backward: (parameter, residual)
        self._held: list = []
        self._accumulate = None
        # Overlap with the tail of backward: the compressed tensors whose gradients are complete
        # first (the last layers) form the "early bucket". Their residuals stay in p.grad, so autograd
        # accumulates onto them as it goes; a post-accumulate hook counts them, and when the bucket
        # is full its share of the step's first product is launched on the aggregator's side stream
        # while backward goes on for the earlier layers (in a recorded step: a parallel branch of
        # the graph). PSGD_B200_OVERLAP=0 switches it off.
        import os

        self._overlap = os.environ.get("PSGD_B200_OVERLAP", "1") != "0" and self.device.type == "cuda" and grad_clip is None
        self._hook_order: list = []        # parameter ids in the order their gradients completed (first compressed step)
        self._hook_recording = False
        self._bucket: dict = {}            # id(parameter) -> parameter, the early bucket
        self._bucket_seen = 0
        self._hooks_installed = False
        self._bucket_decided = False

    # ------------------------------------------------------------------------------------
    def _weights_to_channels_last(self) -> None:
        """Store 4-D weights the way the NHWC convolutions read them. With contiguous weights the
        library converts every filter before each forward / backward and converts every weight
        gradient back (three small copy kernels per convolution and step). The aggregation
        kernels take either layout: a channels_last weight is the same [out, in*kh*kw] matrix
        with permuted columns."""
        fmt = torch.channels_last
        for p in self._params():
            if p.dim() != 4 or p.is_contiguous(memory_format=fmt):
                continue
            p.data = p.data.contiguous(memory_format=fmt)
            if p.grad is not None:
                p.grad = p.grad.contiguous(memory_format=fmt)
            buf = self.optimizer.state.get(p, {}).get("momentum_buffer")
            if buf is not None:
                self.optimizer.state[p]["momentum_buffer"] = buf.contiguous(memory_format=fmt)

    def _gather_norm_counters(self) -> None:
        """Every BatchNorm layer bumps its own `num_batches_tracked` with a one-element kernel per
        forward (20 launches, ~38 us of a ResNet-18 step on B200). The counters become views of ONE
        tensor that the step bumps with a single launch; while the model runs, the layers see no
        counter (they only need it when `momentum` is None, and those layers are left alone).
        `state_dict()` / `load_state_dict()` keep working: the buffers are still there, per layer."""
        self._norm_layers, self._norm_counters = [], None
        if self.device.type != "cuda":
            return
        layers = [m for m in self.model.modules()
                  if isinstance(m, torch.nn.modules.batchnorm._BatchNorm) and m.track_running_stats
                  and m.momentum is not None and isinstance(m._buffers.get("num_batches_tracked"), torch.Tensor)]
        if len(layers) < 2:
            return
        counters = torch.stack([m._buffers["num_batches_tracked"].to(self.device, torch.long).reshape(()) for m in layers])
        for i, m in enumerate(layers):
            m._buffers["num_batches_tracked"] = counters[i]
        self._norm_layers, self._norm_counters = layers, counters

    def _forward(self, x: torch.Tensor) -> torch.Tensor:
        """The model's forward with the normalisation layers' step counters bumped by one launch."""
        layers = self._norm_layers
        if not layers or not self.model.training:
            return self.model(x)
        views = [m._buffers["num_batches_tracked"] for m in layers]
        for m in layers:
            m._buffers["num_batches_tracked"] = None
        try:
            out = self.model(x)
        finally:
            for m, v in zip(layers, views):
                m._buffers["num_batches_tracked"] = v
        if all(v._base is self._norm_counters for v in views):
            self._norm_counters.add_(1)
        else:  # a checkpoint load or .to() replaced the buffers: bump what is there
            torch._foreach_add_(views, 1)
        return out

    def _format(self, x: torch.Tensor) -> torch.Tensor:
        if self.channels_last and x.dim() == 4:
            return x.contiguous(memory_format=torch.channels_last)
        return x

    def _clip(self) -> None:
        if self.grad_clip is not None:
            # foreach implementation: no host synchronisation, capturable
            torch.nn.utils.clip_grad_norm_(self._params(), self.grad_clip, foreach=True)

    def _params(self):
        return [p for g in self.optimizer.param_groups for p in g["params"]]

    def _begin(self) -> None:
        begin = getattr(self.aggregator, "begin_step", None)
        if begin is not None:
            begin()
        # Tensors that are all-reduced uncompressed leave no residual (their .grad is all zeros
        # after a step), so autograd does not need to ACCUMULATE onto it: dropping the zero tensor
        # lets it adopt the fresh gradient and saves one small add kernel per such tensor.
        # Compressed tensors do leave a residual. It is detached for the duration of backward
        # (autograd then adopts the fresh gradients without arithmetic) and `_fold` adds all
        # fresh gradients onto their residuals in one launch instead of one add per parameter.
        self._held = []
        self._bucket_seen = 0
        self._bucket_live = False
        mask = getattr(self.aggregator, "is_compressed_mask", None)
        if self._overlap and mask is not None and getattr(self.aggregator, "compressing", False):
            self._install_hooks()
            if not self._bucket_decided:
                self._hook_order = []
                self._hook_recording = True   # this backward tells in which order gradients complete
        if mask is not None and getattr(self.aggregator, "compressing", False):
            fold = self.device.type == "cuda" and getattr(self.aggregator, "supports_fused_step", lambda _o: False)(self.optimizer)
            for p, keep in zip(self._params(), mask):
                if not keep:
                    p.grad = None
                elif fold and p.grad is not None:
                    if id(p) in self._bucket:
                        self._bucket_live = True   # stays attached: autograd accumulates onto the residual
                        continue
                    self._held.append((p, p.grad))
                    p.grad = None

    # -- overlap with backward -------------------------------------------------------------
    def _install_hooks(self) -> None:
        if self._hooks_installed or not self._overlap:
            return
        mask = getattr(self.aggregator, "is_compressed_mask", None)
        if mask is None:
            return
        self._hooks_installed = True
        for p, keep in zip(self._params(), mask):
            if keep:
                p.register_post_accumulate_grad_hook(self._on_grad_ready)

    def _on_grad_ready(self, p: torch.Tensor) -> None:
        """Post-accumulate hook of a compressed parameter (fires once per backward per parameter,
        however many times the parameter is used)."""
        if self._hook_recording:
            self._hook_order.append(id(p))
            return
        if id(p) in self._bucket and self._bucket_live:
            self._bucket_seen += 1
            if self._bucket_seen == len(self._bucket):
                self._launch_early()

    def _choose_bucket(self) -> None:
        """Early bucket = the compressed parameters that completed first in the recorded backward,
        up to ~60 % of the compressed elements (for a ResNet: the last stage and the classifier)."""
        core = getattr(self.aggregator, "_powersgd", None)
        native = getattr(core, "_native", None)
        if native is None or not self._hook_order:
            return
        params = self._params()
        by_id = {id(p): p for p in params}
        compressed = [p for p, keep in zip(params, self.aggregator.is_compressed_mask) if keep]
        position = {id(p): i for i, p in enumerate(compressed)}
        total = sum(p.numel() for p in compressed)
        picked, acc = [], 0
        on_tensor_cores = getattr(native, "tensor_core_positions", frozenset())
        for pid in self._hook_order:
            if pid not in position or acc >= 0.6 * total or position[pid] in on_tensor_cores:
                continue
            picked.append(pid)
            acc += by_id[pid].numel()
        if len(picked) == len(compressed) or not picked:
            return  # nothing would be left for after backward / nothing early: no split
        self._bucket = {pid: by_id[pid] for pid in picked}
        native.set_early_bucket([position[pid] for pid in picked])

    def _launch_early(self) -> None:
        """All gradients of the early bucket are complete (autograd has added them onto the
        residuals): start their share of the first product on the side stream. Uses descriptor
        tables bound in an earlier step; nothing is allocated or uploaded here."""
        native = getattr(self.aggregator._powersgd, "_native", None)
        if native is not None:
            native.early_product()

    def _fold(self) -> None:
        """p.grad <- residual + fresh gradient for the parameters detached by `_begin`."""
        held, self._held = self._held, []
        self._fold_launches = 0
        if not held:
            return
        live = [(p, r) for p, r in held if p.grad is not None]
        same = all(same_layout(p.grad, r) and p.grad.dtype == r.dtype for p, r in live)
        if live and same and all(r.dtype == torch.float32 for _p, r in live):
            if self._accumulate is None:
                from .cuda_path import MultiTensorAccumulate

                self._accumulate = MultiTensorAccumulate()
            fused = getattr(self.aggregator, "_fused", None)
            if fused is not None:
                fused.fold(self._accumulate, [r for _p, r in live], [p.grad for p, _r in live])
            else:
                self._accumulate([r for _p, r in live], [p.grad for p, _r in live])
            self._fold_launches += 1
        else:
            for p, r in live:
                r.add_(p.grad)
        for p, r in held:
            p.grad = r  # parameters that received no gradient keep their residual as it was

    def _eager(self, x: torch.Tensor, y: torch.Tensor, time_aggregate: bool = False) -> torch.Tensor:
        self._begin()
        loss = self.loss_fn(self._forward(self._format(x)), y)
        loss.backward()
        if time_aggregate and self.time_aggregate:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            self._fold()
            self._clip()
            optimizer_step(self.optimizer, self.aggregator)
            b.record()
            self._agg_events = (a, b)
        else:
            self._fold()
            self._clip()
            optimizer_step(self.optimizer, self.aggregator)
            self._agg_events = None
        fused = getattr(self.aggregator, "_fused", None)
        if fused is not None:
            self.launches_per_step = getattr(fused, "launches", 0) + getattr(self, "_fold_launches", 0)
        if self._hook_recording:
            self._hook_recording = False
            if fused is not None and getattr(self.aggregator._powersgd, "_native", None) is not None:
                self._choose_bucket()   # may leave the bucket empty: then nothing is launched early
                self._bucket_decided = True
        return loss.detach()

    @property
    def aggregate_ms(self) -> Optional[float]:
        """Device time of the aggregation + optimizer part (everything after backward) of the LAST
        step, recorded or eager; synchronises on that step's end. None if it was not timed."""
        if self._agg_events is None:
            return None
        a, b = self._agg_events
        b.synchronize()
        return a.elapsed_time(b)

    def _parity(self) -> int:
        core = getattr(self.aggregator, "_powersgd", None)
        if core is None:
            return 0
        return (core.step_counter * core.config.num_iters_per_step) % 2

    def _graphable_now(self) -> bool:
        if not self.use_graph or self._steps_done < self.eager_steps:
            return False
        if self._graphs:
            return True
        compressing = getattr(self.aggregator, "compressing", True)
        fused_ok = getattr(self.aggregator, "supports_fused_step", lambda _o: False)(self.optimizer)
        return bool(compressing) and bool(fused_ok)

    def _bump_counters(self) -> None:
        agg = self.aggregator
        agg.step_counter += 1
        core = getattr(agg, "_powersgd", None)
        if core is not None and core.params:
            core.step_counter += 1
        self.optimizer._opt_called = True  # what a learning-rate scheduler checks

    def _capture(self, parity: int) -> None:
        agg = self.aggregator
        saved = (agg.step_counter, agg._powersgd.step_counter)
        from .cuda_path import capture_scope

        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        # relaxed: descriptor tables rebuilt during capture allocate pinned staging memory
        with capture_scope() as keep, torch.cuda.graph(graph, pool=self._pool, capture_error_mode="relaxed"):
            self._begin()
            loss = self.loss_fn(self._forward(self._static_x), self._static_y)
            loss.backward()
            if self.time_aggregate:
                ev = (torch.cuda.Event(enable_timing=True, external=True), torch.cuda.Event(enable_timing=True, external=True))
                ev[0].record()
            self._fold()
            self._clip()
            agg.fused_step(self.optimizer, prepared=True)
            if self.time_aggregate:
                ev[1].record()
                self._graph_events[parity] = ev
            if self._static_loss is None:
                self._static_loss = loss.detach()
            else:
                self._static_loss.copy_(loss.detach())
        if self._pool is None:
            self._pool = graph.pool()
        # capturing ran the host side of the step (counters) but not the kernels: rewind
        agg.step_counter, agg._powersgd.step_counter = saved
        self._graphs[parity] = graph
        self._graph_keep[parity] = keep  # tables the graph's copy nodes read: same lifetime as the graph

    def __call__(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        if not self._graphable_now():
            loss = self._eager(x, y, time_aggregate=True)
            self._steps_done += 1
            return loss
        if self._static_x is None:
            self._static_x = self._format(torch.empty_like(x, device=self.device))
            self._static_y = torch.empty_like(y, device=self.device)
        if x.shape != self._static_x.shape or y.shape != self._static_y.shape:
            loss = self._eager(x, y)  # ragged last batch etc.
            self._steps_done += 1
            return loss
        self._static_x.copy_(x, non_blocking=True)
        self._static_y.copy_(y, non_blocking=True)
        parity = self._parity()
        if parity not in self._graphs:
            self._capture(parity)
        # a bounded device-side wait that gave up during an earlier step (a peer that stayed away)
        # left zeros where data should be: stop here, with the step number, instead of training on
        fused = self.aggregator._fused
        try:
            fused.check()
        except RuntimeError as exc:
            raise type(exc)(f"training step {self._steps_done}: {exc}") from None
        # host-side refresh of what the graph reads from memory (learning rates etc.)
        fused.prepare(self.optimizer)
        self._graphs[parity].replay()
        self._agg_events = self._graph_events.get(parity)
        self._bump_counters()
        self._steps_done += 1
        return self._static_loss
