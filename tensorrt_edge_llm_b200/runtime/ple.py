"""Per-layer-embedding store: file-resident table, device row cache, per-step gather.

``PleStore.gather(token_ids)`` returns ``[T, layers, dim]`` rows for the step's tokens.  The native side
(``csrc/runtime/ple.{h,cpp}``) plans hits / misses, coalesces file runs, applies the IO budget and copies the
missing rows into a pinned staging tensor on worker threads; this module uploads the staging rows, scatters them
into the device cache (``index_copy_``) and gathers the step's rows with the embedding-gather kernel.

Parity: ``cpp/runtime/embedding/ple*.cpp`` with the ``pleGatherPlugin`` / ``pleGather.cu`` / ``pleScatter.cu``
kernels, and the server's ``PleRuntimeConfig`` (``tensorrt_edgellm/server/config.py``)."""
from __future__ import annotations

from typing import Optional, Sequence

import torch

from .. import ops
from . import native as rt

_DTYPES = {0: torch.float16, 1: torch.bfloat16, 2: torch.float32}
_CODES = {v: k for k, v in _DTYPES.items()}


def write_ple_table(path: str, table: torch.Tensor, layers: int) -> None:
    """``table [vocab, layers · dim]`` (fp16 / bf16 / fp32) → a PLE table file."""
    if table.dim() != 2 or table.shape[1] % layers:
        raise ValueError("expected [vocab, layers * dim]")
    t = table.contiguous().cpu()
    raw = t.view(torch.uint8).numpy() if t.dtype != torch.bfloat16 else t.view(torch.int16).view(torch.uint8).numpy()
    rt.PleTable.write(path, raw, layers, _CODES[table.dtype])


class PleStore:
    def __init__(self, path: str, cache_rows: int, device="cpu", io_bytes_per_step: int = 0, read_threads: int = 2,
                 max_step_rows: int = 8192):
        self.table = rt.PleTable(path)
        self.dtype = _DTYPES[self.table.dtype]
        self.layers = self.table.layers
        self.row_elems = self.table.row_bytes // torch.empty((), dtype=self.dtype).element_size()
        self.dim = self.row_elems // self.layers
        self.device = torch.device(device)
        self.cache = rt.PleCache(cache_rows)
        self.budget = rt.PleIoBudget(io_bytes_per_step) if io_bytes_per_step else None
        self.executor = rt.PleReadExecutor(read_threads)
        self.device_cache = torch.zeros(cache_rows, self.row_elems, dtype=self.dtype, device=self.device)
        self.staging = torch.empty(max_step_rows, self.row_elems, dtype=self.dtype)
        if self.device.type == "cuda":
            self.staging = self.staging.pin_memory()
        self.deferred_rows = 0
        self.bytes_read = 0

    @torch.no_grad()
    def gather(self, token_ids: Sequence[int]) -> torch.Tensor:
        """Rows of ``token_ids`` as ``[T, layers, dim]``.  A token whose row the IO budget deferred gets zeros this
        step (its contribution is skipped rather than stalling the step) and is read on a later one."""
        ids = [int(t) for t in token_ids]
        plan = self.cache.plan(ids, self.table.row_bytes, self.budget)
        n_miss = len(plan.miss_rows)
        if n_miss > self.staging.shape[0]:
            raise ValueError(f"{n_miss} rows to read exceed the staging buffer ({self.staging.shape[0]})")
        if n_miss:
            self.executor.read(self.table, plan, self.staging.data_ptr())
            fresh = self.staging[:n_miss].to(self.device, non_blocking=True)
            self.device_cache.index_copy_(0, torch.tensor(plan.miss_slots, dtype=torch.int64, device=self.device), fresh)
            self.bytes_read += plan.bytes
        self.deferred_rows += plan.deferred
        slots = torch.tensor(plan.slots, dtype=torch.int32, device=self.device)
        rows = ops.embedding(slots.clamp(min=0), self.device_cache)
        if plan.deferred:
            rows = rows * (slots >= 0)[:, None].to(rows.dtype)
        return rows.view(len(ids), self.layers, self.dim)

    @property
    def hit_rate(self) -> float:
        tot = self.cache.hits + self.cache.misses
        return self.cache.hits / tot if tot else 0.0
