"""Step timing and memory tracking.

``step_perf`` brackets one training step; ``.mark(name)`` closes a phase
(``clip`` / ``noise`` / ``optimizer``).  On CUDA every mark records a CUDA event
on the current stream and the durations are read *on the device* when the
context exits (one synchronise per step, none per mark); on CPU it falls back
to ``perf_counter``.  ``PerfState`` folds steps (the first ``warmup_steps`` are
excluded from throughput), ``PerfTracker`` keeps one state per stage, and
``sync(PerfState)`` reduces across ranks as time = max, samples = sum,
peak memory = max.  ``trace_range`` names a phase for the PyTorch profiler (and NVTX when enabled), ``trace`` collects
a Chrome trace of a few steps.

Parity: packages/opaque-engine/src/opaque/api/engine/profiling/_memory.py:374-436, :689;
_distributed.py.
"""
from __future__ import annotations

import contextlib
import dataclasses
import time
from typing import Any

import torch


@dataclasses.dataclass(frozen=True)
class MemoryStats:
    allocated_bytes: int = 0
    reserved_bytes: int = 0
    peak_allocated_bytes: int = 0
    peak_reserved_bytes: int = 0

    @property
    def peak_gb(self) -> float:
        return self.peak_allocated_bytes / 2 ** 30

    @property
    def allocated_gb(self) -> float:
        return self.allocated_bytes / 2 ** 30

    @property
    def reserved_gb(self) -> float:
        return self.reserved_bytes / 2 ** 30

    def to_dict(self) -> dict[str, float]:
        return {"allocated_gb": self.allocated_gb, "reserved_gb": self.reserved_gb, "peak_gb": self.peak_gb,
                "peak_reserved_gb": self.peak_reserved_bytes / 2 ** 30}


_NVTX = {"on": None}      # None: decided by the environment variable OPAQUE_B200_NVTX on first use


def enable_nvtx(on: bool = True) -> None:
    """Also emit NVTX ranges from :func:`trace_range` (visible in Nsight Systems / Nsight Compute timelines)."""
    _NVTX["on"] = bool(on)


def _nvtx_on() -> bool:
    if _NVTX["on"] is None:
        import os
        _NVTX["on"] = os.environ.get("OPAQUE_B200_NVTX", "0") not in ("0", "", "false", "False")
    return bool(_NVTX["on"]) and torch.cuda.is_available()


@contextlib.contextmanager
def trace_range(name: str):
    """A named range around a phase: a ``torch.profiler.record_function`` range always (free when no profiler is attached),
    plus an NVTX range when enabled (``enable_nvtx()`` or ``OPAQUE_B200_NVTX=1``).  The functional API's own ranges
    (``opaque::clipped_grad``, ``opaque::gaussian_noise``, ``opaque::mf_gaussian_noise``, …) and the fused engine's
    (``opaque::fused/microbatch``, ``/clip``, ``/shard_step``) all come through here or ``record_function``."""
    nvtx = _nvtx_on()
    if nvtx:
        torch.cuda.nvtx.range_push(name)
    try:
        with torch.profiler.record_function(name):
            yield
    finally:
        if nvtx:
            torch.cuda.nvtx.range_pop()


@contextlib.contextmanager
def trace(path: str | None = None, *, with_stack: bool = False, record_shapes: bool = False):
    """Collect a ``torch.profiler`` trace of the enclosed steps (CPU activity always, CUDA when available); on exit the
    Chrome-trace JSON goes to ``path`` when given.  Yields the profiler (``key_averages()`` for a table).  Timings under
    a profiler are for reading the timeline, never for reporting throughput."""
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    with torch.profiler.profile(activities=acts, with_stack=with_stack, record_shapes=record_shapes) as prof:
        yield prof
    if path:
        prof.export_chrome_trace(path)


def _is_cuda(device: Any) -> bool:
    return torch.device(device).type == "cuda" and torch.cuda.is_available()


def get_memory_stats(device: Any = None) -> MemoryStats:
    """Current / peak allocated and reserved device memory in bytes."""
    if device is None or not _is_cuda(device):
        return MemoryStats()
    return MemoryStats(torch.cuda.memory_allocated(device), torch.cuda.memory_reserved(device),
                       torch.cuda.max_memory_allocated(device), torch.cuda.max_memory_reserved(device))


def reset_peak_memory(device: Any = None) -> None:
    """Reset the allocator's peak-memory counters."""
    if device is not None and _is_cuda(device):
        torch.cuda.reset_peak_memory_stats(device)


def empty_cache(device: Any = None) -> None:
    """Release cached device memory held by the allocator (no-op without a GPU)."""
    if device is not None and _is_cuda(device):
        torch.cuda.empty_cache()


def print_memory(device: Any = None, label: str = "", *, prefix: str = "") -> MemoryStats:
    """Print ``get_memory_stats`` in GiB behind an optional ``[label]`` (or a literal ``prefix``) and return the stats."""
    s = get_memory_stats(device)
    prefix = f"[{label}] " if label else prefix
    print(f"{prefix}allocated={s.allocated_bytes / 2**30:.2f}GiB reserved={s.reserved_bytes / 2**30:.2f}GiB "
          f"peak={s.peak_allocated_bytes / 2**30:.2f}GiB")
    return s


@dataclasses.dataclass(frozen=True)
class StepPerf:
    """One step: total seconds, per-phase seconds, samples, peak memory."""
    seconds: float
    phases: dict[str, float]
    batch_size: int
    peak_memory_bytes: int = 0
    device_timed: bool = False

    # the reference's field names, as read-only views
    @property
    def step_time_sec(self) -> float:
        return self.seconds

    @property
    def samples_per_second(self) -> float:
        return self.batch_size / self.seconds if self.seconds > 0 else 0.0

    @property
    def memory_peak_gb(self) -> float:
        return self.peak_memory_bytes / 2 ** 30

    @property
    def marks(self) -> dict[str, float]:
        return self.phases

    def to_dict(self) -> dict[str, Any]:
        """JSON-ready: seconds, samples per second, peak memory in GB, and ``time/<phase>`` per mark."""
        return {"step_time_sec": self.seconds, "samples_per_second": self.samples_per_second, "batch_size": self.batch_size,
                "memory_peak_gb": self.memory_peak_gb, **{f"time/{k}": v for k, v in self.phases.items()}}


class _StepTimer:
    def __init__(self, device: Any, batch_size: int, track_memory: bool):
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.batch_size = batch_size
        self.track_memory = track_memory
        self.cuda = _is_cuda(self.device)
        self._marks: list[tuple[str, Any]] = []
        self.result: StepPerf | None = None

    def _stamp(self):
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(self.device))
            return ev
        return time.perf_counter()

    def start(self):
        if self.cuda and self.track_memory:
            torch.cuda.reset_peak_memory_stats(self.device)
        self._t0 = self._stamp()

    def mark(self, name: str) -> None:
        self._marks.append((name, self._stamp()))

    def finish(self):
        end = self._stamp()
        phases: dict[str, float] = {}
        if self.cuda:
            end.synchronize()
            prev = self._t0
            for name, ev in self._marks:
                phases[name] = phases.get(name, 0.0) + prev.elapsed_time(ev) / 1e3
                prev = ev
            total = self._t0.elapsed_time(end) / 1e3
            peak = torch.cuda.max_memory_allocated(self.device) if self.track_memory else 0
        else:
            prev = self._t0
            for name, t in self._marks:
                phases[name] = phases.get(name, 0.0) + (t - prev)
                prev = t
            total = end - self._t0
            peak = 0
        self.result = StepPerf(total, phases, self.batch_size, peak, self.cuda)


@contextlib.contextmanager
def step_perf(device: Any = None, *, batch_size: int = 0, track_memory: bool = True):
    """Time one step; read ``.result`` (a :class:`StepPerf`) after the block."""
    timer = _StepTimer(device, batch_size, track_memory)
    timer.start()
    try:
        yield timer
    finally:
        timer.finish()


@dataclasses.dataclass(frozen=True)
class PerfState:
    """Running totals over steps; warm-up steps count toward ``steps`` only."""
    steps: int = 0
    timed_steps: int = 0
    seconds: float = 0.0
    samples: int = 0
    peak_memory_bytes: int = 0
    phases: dict[str, float] = dataclasses.field(default_factory=dict)
    warmup_steps: int = 1

    def add(self, step: StepPerf) -> "PerfState":
        peak = max(self.peak_memory_bytes, step.peak_memory_bytes)
        if self.steps < self.warmup_steps:
            return dataclasses.replace(self, steps=self.steps + 1, peak_memory_bytes=peak)
        phases = dict(self.phases)
        for k, v in step.phases.items():
            phases[k] = phases.get(k, 0.0) + v
        return dataclasses.replace(self, steps=self.steps + 1, timed_steps=self.timed_steps + 1,
                                   seconds=self.seconds + step.seconds,
                                   samples=self.samples + step.batch_size,
                                   peak_memory_bytes=peak, phases=phases)

    @property
    def samples_per_second(self) -> float:
        return self.samples / self.seconds if self.seconds > 0 else 0.0

    @property
    def seconds_per_step(self) -> float:
        return self.seconds / self.timed_steps if self.timed_steps else 0.0

    # the reference's field names, as read-only views ("stable" = after the warm-up steps)
    @property
    def num_steps(self) -> int:
        return self.steps

    @property
    def num_steps_stable(self) -> int:
        return self.timed_steps

    @property
    def total_time_stable(self) -> float:
        return self.seconds

    @property
    def total_samples_stable(self) -> int:
        return self.samples

    @property
    def max_peak_memory_gb(self) -> float:
        return self.peak_memory_bytes / 2 ** 30

    @property
    def avg_step_time_stable(self) -> float:
        return self.seconds_per_step

    avg_step_time = avg_step_time_stable                 # warm-up steps are not timed into the totals here

    @property
    def avg_samples_per_second_stable(self) -> float:
        return self.samples_per_second

    avg_samples_per_second = avg_samples_per_second_stable

    def to_dict(self) -> dict[str, Any]:
        """JSON-ready summary of the stage (rates over the steps after warm-up)."""
        return {"num_steps": self.steps, "num_steps_stable": self.timed_steps, "total_time_stable": self.seconds,
                "total_samples_stable": self.samples, "avg_step_time_stable": self.seconds_per_step,
                "avg_samples_per_second_stable": self.samples_per_second, "max_peak_memory_gb": self.max_peak_memory_gb,
                **{f"time/{k}": v / max(self.timed_steps, 1) for k, v in self.phases.items()}}


PerfStage = str


class PerfTracker:
    """One :class:`PerfState` per stage (``train`` / ``eval`` / ``test``)."""

    def __init__(self, device: Any = None, warmup_steps: int = 1):
        self.device = device
        self.warmup_steps = warmup_steps
        self.stages: dict[str, PerfState] = {}

    def step(self, stage: str = "train", *, batch_size: int = 0, track_memory: bool = True):
        tracker = self

        @contextlib.contextmanager
        def ctx():
            with step_perf(tracker.device, batch_size=batch_size, track_memory=track_memory) as t:
                yield t
            state = tracker.stages.get(stage, PerfState(warmup_steps=tracker.warmup_steps))
            tracker.stages[stage] = state.add(t.result)
        return ctx()

    def state(self, stage: str = "train") -> PerfState:
        return self.stages.get(stage, PerfState(warmup_steps=self.warmup_steps))

    def summary(self) -> dict[str, dict[str, float]]:
        return {k: {"samples_per_second": s.samples_per_second, "seconds_per_step": s.seconds_per_step,
                    "peak_memory_gb": s.peak_memory_bytes / 2 ** 30, "steps": s.steps}
                for k, s in self.stages.items()}


def perf_tracker(device: Any = None, warmup_steps: int = 1) -> PerfTracker:
    """A ``PerfTracker`` that accumulates named step timings, samples and tokens."""
    return PerfTracker(device, warmup_steps)


def sync_perf_state(state: PerfState) -> PerfState:
    """Cross-rank fold: seconds = max, samples = sum, peak = max."""
    from ..distributed import is_distributed, reduce_scalar
    if not is_distributed():
        return state
    phases = {k: reduce_scalar(v, "max") for k, v in sorted(state.phases.items())}
    return dataclasses.replace(
        state, seconds=reduce_scalar(state.seconds, "max"), samples=int(reduce_scalar(state.samples, "sum")),
        peak_memory_bytes=int(reduce_scalar(state.peak_memory_bytes, "max")), phases=phases)


__all__ = ["MemoryStats", "PerfStage", "PerfState", "PerfTracker", "StepPerf", "empty_cache", "enable_nvtx",
           "get_memory_stats", "perf_tracker", "print_memory", "reset_peak_memory", "step_perf",
           "sync_perf_state", "trace", "trace_range"]

from ..utils.namespaces import submodule as _sub  # noqa: E402

_sub(__name__, "types", "Classes of the profiling façade.", {n: globals()[n] for n in ("MemoryStats", "PerfStage", "PerfState", "PerfTracker", "StepPerf")},
     bind=False)
