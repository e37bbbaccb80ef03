"""Stage timing, NVTX ranges, request metrics and a device-memory monitor.

Three levels, as in the reference's ``cpp/profiling`` (``timer.h``: pooled CUDA-event pairs per stage behind a
global switch, ``TIME_STAGE``; ``nvtx_wrapper.h``: scoped ranges compiled out unless enabled; ``metrics.h``: prefill /
generation / speculative metrics structs) and ``examples/cpp/common/memoryMonitor.cpp`` (50 ms sampling of device
memory).  Stage times are device times (CUDA events on the launching stream); on CPU the timer falls back to the
host clock so the same call sites work in tests.
"""
from __future__ import annotations

import contextlib
import os
import threading
import time
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional

import torch

_ENABLED = os.environ.get("TELB_PROFILE", "0") == "1"
_NVTX = os.environ.get("TELB_ENABLE_NVTX", "0") == "1"

# stage names shared with the range names of the reference's scheduler and decoders
IFB_PLAN, IFB_EXECUTE, IFB_COMMIT = "IFB_PLAN", "IFB_EXECUTE", "IFB_COMMIT"
PREFILL, VANILLA_DECODING, SAMPLING = "LLM_PREFILL", "VANILLA_DECODING", "SAMPLING"
SPEC_DRAFT, SPEC_VERIFY, SPEC_ACCEPT = "SPEC_DECODE_DRAFT", "SPEC_DECODE_VERIFY", "SPEC_DECODE_ACCEPT"


def set_profiling_enabled(on: bool) -> None:
    global _ENABLED
    _ENABLED = bool(on)


def profiling_enabled() -> bool:
    return _ENABLED


def set_nvtx_enabled(on: bool) -> None:
    global _NVTX
    _NVTX = bool(on)


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range around a host region; free when NVTX is off or there is no CUDA runtime."""
    if not _NVTX or not torch.cuda.is_available():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


@dataclass
class TimingSample:
    stage: str
    ms: float
    batch: int = 0
    tokens: int = 0


class StageTimer:
    """Per-thread collector of stage durations.  ``with timer.stage("X", batch=…, tokens=…):`` records a CUDA-event pair
    on the current stream (events come from a pool and are read back lazily by :meth:`samples`, so timing adds no
    synchronisation to the timed region)."""

    def __init__(self, device: Optional[torch.device] = None):
        self.device = device
        self._pool: List[torch.cuda.Event] = []
        self._pending: List[tuple] = []
        self._done: List[TimingSample] = []

    def _event(self):
        return self._pool.pop() if self._pool else torch.cuda.Event(enable_timing=True)

    @contextlib.contextmanager
    def stage(self, name: str, batch: int = 0, tokens: int = 0):
        if not _ENABLED:
            with nvtx_range(name):
                yield
            return
        cuda = torch.cuda.is_available() and (self.device is None or self.device.type == "cuda")
        with nvtx_range(name):
            if cuda:
                e0, e1 = self._event(), self._event()
                e0.record()
                try:
                    yield
                finally:
                    e1.record()
                    self._pending.append((name, e0, e1, batch, tokens))
            else:
                t0 = time.perf_counter()
                try:
                    yield
                finally:
                    self._done.append(TimingSample(name, (time.perf_counter() - t0) * 1e3, batch, tokens))

    def begin(self, name: str, batch: int = 0, tokens: int = 0):
        """Open a stage without a ``with`` block; pass the result to :meth:`end`."""
        cm = self.stage(name, batch, tokens)
        cm.__enter__()
        return cm

    @staticmethod
    def end(handle) -> None:
        handle.__exit__(None, None, None)

    def samples(self) -> List[TimingSample]:
        if self._pending:
            torch.cuda.synchronize()
            for name, e0, e1, batch, tokens in self._pending:
                self._done.append(TimingSample(name, e0.elapsed_time(e1), batch, tokens))
                self._pool += [e0, e1]
            self._pending = []
        return list(self._done)

    def reset(self) -> None:
        self.samples()
        self._done = []

    def summary(self) -> Dict[str, Dict[str, float]]:
        out: Dict[str, Dict[str, float]] = {}
        for s in self.samples():
            d = out.setdefault(s.stage, {"count": 0, "total_ms": 0.0, "tokens": 0, "max_ms": 0.0})
            d["count"] += 1
            d["total_ms"] += s.ms
            d["tokens"] += s.tokens
            d["max_ms"] = max(d["max_ms"], s.ms)
        for d in out.values():
            d["mean_ms"] = d["total_ms"] / max(d["count"], 1)
        return out

    def format(self) -> str:
        rows = ["stage                      count   total ms    mean ms     max ms     tokens"]
        for k, d in sorted(self.summary().items(), key=lambda kv: -kv[1]["total_ms"]):
            rows.append(f"{k:<26}{d['count']:>6}{d['total_ms']:>11.3f}{d['mean_ms']:>11.3f}{d['max_ms']:>11.3f}{d['tokens']:>11}")
        return "\n".join(rows)


_TLS = threading.local()


def timer() -> StageTimer:
    """The calling thread's timer (the engine's actor thread and a benchmark's main thread do not share one)."""
    t = getattr(_TLS, "timer", None)
    if t is None:
        t = _TLS.timer = StageTimer()
    return t


def time_stage(name: str, batch: int = 0, tokens: int = 0):
    return timer().stage(name, batch, tokens)


# ---- metrics structs -------------------------------------------------------------------------------------------------

@dataclass
class PrefillMetrics:
    reused_tokens: int = 0
    computed_tokens: int = 0
    pruned_tokens: int = 0
    time_ms: float = 0.0

    @property
    def tokens_per_second(self) -> float:
        return self.computed_tokens / (self.time_ms / 1e3) if self.time_ms > 0 else 0.0


@dataclass
class GenerationMetrics:
    generated_tokens: int = 0
    decode_steps: int = 0
    time_ms: float = 0.0

    @property
    def tokens_per_second(self) -> float:
        return self.generated_tokens / (self.time_ms / 1e3) if self.time_ms > 0 else 0.0


@dataclass
class SpecDecodeMetrics:
    rounds: int = 0
    draft_tokens: int = 0
    accepted_tokens: int = 0
    acceptance_lengths: List[int] = field(default_factory=list)

    @property
    def mean_acceptance_length(self) -> float:
        return sum(self.acceptance_lengths) / len(self.acceptance_lengths) if self.acceptance_lengths else 0.0


def metrics_dict(m) -> dict:
    d = asdict(m)
    for k in ("tokens_per_second", "mean_acceptance_length"):
        if hasattr(m, k):
            d[k] = getattr(m, k)
    return d


# ---- device memory monitor -------------------------------------------------------------------------------------------

class MemoryMonitor:
    """Samples this process's device memory every ``interval_s`` on a helper thread and keeps the peak.

    Sources, in order: NVML's per-process figure (when the ``pynvml`` module and the library are present), else the
    drop in free device memory since :meth:`start` (``cudaMemGetInfo``), else torch's allocator statistics.  ``probe``
    may be replaced by a callable returning bytes, which is how the CPU tests drive it."""

    def __init__(self, device: int = 0, interval_s: float = 0.05, probe=None):
        self.device, self.interval_s = device, interval_s
        self._probe = probe or self._make_probe()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.peak_bytes = 0
        self.samples = 0
        self.source = getattr(self._probe, "source", "custom")

    def _make_probe(self):
        if torch.cuda.is_available():
            try:
                import pynvml
                pynvml.nvmlInit()
                h = pynvml.nvmlDeviceGetHandleByIndex(self.device)
                pid = os.getpid()

                def nvml_probe():
                    for p in pynvml.nvmlDeviceGetComputeRunningProcesses(h):
                        if p.pid == pid and p.usedGpuMemory:
                            return int(p.usedGpuMemory)
                    return 0
                if nvml_probe() > 0:
                    nvml_probe.source = "nvml"
                    return nvml_probe
            except Exception:          # no NVML in this container: fall through to the runtime's own view
                pass
            free0, _ = torch.cuda.mem_get_info(self.device)

            def info_probe():
                free, _ = torch.cuda.mem_get_info(self.device)
                return max(free0 - free, torch.cuda.memory_reserved(self.device))
            info_probe.source = "mem_get_info"
            return info_probe

        def none_probe():
            return 0
        none_probe.source = "none"
        return none_probe

    def _run(self):
        while not self._stop.is_set():
            try:
                self.peak_bytes = max(self.peak_bytes, int(self._probe()))
                self.samples += 1
            except Exception:          # a failing probe must not take the measured program down
                pass
            self._stop.wait(self.interval_s)

    def start(self) -> "MemoryMonitor":
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, name="telb-memory-monitor", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> int:
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None
            self.peak_bytes = max(self.peak_bytes, int(self._probe()))
        return self.peak_bytes

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
