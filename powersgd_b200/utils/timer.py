"""Phase timers.

`Timer` keeps the interface of the research harness (paper-code/timer.py:12-132): a
context manager keyed by label with a verbosity gate, the first occurrence of each label
dropped, a text summary and a JSON dump. It brackets the region with a device
synchronisation, so it serialises the GPU exactly like the original.

`DeviceTimer` is the variant used by the benchmarks: CUDA events on the current stream,
resolved lazily, so that timing a phase does not stall the pipeline.
"""
from __future__ import annotations

import json
import time
from contextlib import contextmanager
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np
import torch


class Timer:
    def __init__(self, verbosity_level: int = 1, log_fn: Optional[Callable] = None, skip_first: bool = True):
        self.verbosity_level = verbosity_level
        self.log_fn = log_fn if log_fn is not None else self._print_event
        self.skip_first = skip_first
        self.reset()

    def reset(self) -> None:
        self.totals: Dict[str, float] = {}
        self.first_time: Dict[str, float] = {}
        self.last_time: Dict[str, float] = {}
        self.call_counts: Dict[str, int] = {}

    def report(self, label: str, start: float, end: float) -> None:
        seen = label in self.totals
        if not seen and self.skip_first:
            # the first sample of a label usually holds one-off costs (allocation, autotune)
            self.totals[label] = 0.0
            self.call_counts[label] = 0
            self.last_time[label] = end
            return
        self.first_time.setdefault(label, start)
        self.last_time[label] = end
        self.totals[label] = self.totals.get(label, 0.0) + (end - start)
        self.call_counts[label] = self.call_counts.get(label, 0) + 1

    @contextmanager
    def __call__(self, label: str, epoch: float = -1.0, verbosity: int = 1):
        if verbosity > self.verbosity_level:
            yield
            return
        self._sync()
        start = time.perf_counter()
        yield
        self._sync()
        end = time.perf_counter()
        self.report(label, start, end)
        count = self.call_counts[label]
        if count > 0 and np.random.rand() < 1.0 / count:
            self.log_fn("timer", {"epoch": float(epoch), "value": end - start}, {"event": label})

    def _rows(self) -> List[Tuple[str, int, float, float]]:
        rows = []
        for label in sorted(self.totals):
            count = self.call_counts[label]
            if count == 0:
                continue
            total = self.totals[label]
            span = max(self.last_time[label] - self.first_time[label], 1e-12)
            rows.append((label, count, total / count, 100.0 * total / span))
        return rows

    def summary(self) -> str:
        lines = [
            "--- Timer summary -----------------------------------------------",
            "  Event                          |  Count | Average time |  Frac.",
        ]
        for label, count, avg, frac in self._rows():
            lines.append(f"- {label:30s} | {count:6d} | {avg:11.5f}s | {frac:5.1f}%")
        lines.append("-----------------------------------------------------------------")
        return "\n".join(lines) + "\n"

    def save_summary(self, json_file_path: str) -> None:
        data = {
            label: {
                "label": label,
                "average_duration": avg,
                "n_events": count,
                "total_time": avg * count,
            }
            for label, count, avg, _ in self._rows()
        }
        with open(json_file_path, "w") as fp:
            json.dump(data, fp)

    @staticmethod
    def _sync() -> None:
        if torch.cuda.is_available():
            torch.cuda.synchronize()

    @staticmethod
    def _print_event(_, values, tags) -> None:
        print(f"Timer: {tags['event']:30s} @ {values['epoch']:4.1f} - {values['value']:8.5f}s")


class DeviceTimer:
    """Label-keyed CUDA-event timer that never synchronises inside the timed region.

    Each `with timer(label)` records an event pair on the current stream. Durations are
    read in `resolve()` (called by `summary()` / `totals_ms()`), which synchronises once.
    On a machine without CUDA it falls back to the host clock.
    """

    def __init__(self, skip_first: bool = False):
        self.skip_first = skip_first
        self._pending: List[Tuple[str, object, object]] = []
        self._ms: Dict[str, List[float]] = {}
        self._seen: Dict[str, int] = {}
        self._cuda = torch.cuda.is_available()

    @contextmanager
    def __call__(self, label: str, epoch: float = -1.0, verbosity: int = 1):
        if self._cuda:
            start = torch.cuda.Event(enable_timing=True)
            stop = torch.cuda.Event(enable_timing=True)
            start.record()
            yield
            stop.record()
            self._pending.append((label, start, stop))
        else:
            t0 = time.perf_counter()
            yield
            self._record(label, (time.perf_counter() - t0) * 1e3)

    def _record(self, label: str, ms: float) -> None:
        seen = self._seen.get(label, 0)
        self._seen[label] = seen + 1
        if self.skip_first and seen == 0:
            return
        self._ms.setdefault(label, []).append(ms)

    def resolve(self) -> None:
        if not self._pending:
            return
        torch.cuda.synchronize()
        for label, start, stop in self._pending:
            self._record(label, start.elapsed_time(stop))
        self._pending.clear()

    def totals_ms(self) -> Dict[str, float]:
        self.resolve()
        return {k: float(sum(v)) for k, v in self._ms.items()}

    def mean_ms(self) -> Dict[str, float]:
        self.resolve()
        return {k: float(sum(v) / len(v)) for k, v in self._ms.items() if v}

    def summary(self) -> str:
        means = self.mean_ms()
        lines = ["--- Device timer (CUDA events) ----------------------------------"]
        for label in sorted(means):
            lines.append(f"- {label:30s} | {len(self._ms[label]):6d} | {means[label]:10.4f} ms")
        return "\n".join(lines) + "\n"
