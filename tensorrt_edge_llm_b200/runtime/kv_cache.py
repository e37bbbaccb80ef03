"""Paged KV-cache pool and the host-truth page table.

One device tensor ``[layers, pages, 2, Hkv, page_size, D]`` holds every attention layer's keys
and values; a (page, K|V, head) slab is contiguous (``page_size × D`` elements), which is the
tile the attention kernels fetch with one TMA copy.  A logical page of a sequence maps to the
same physical page index in every layer, so one ``[seats, max_pages]`` table serves the model.

Parity: ``cpp/runtime/kvCacheManager.{h,cpp}`` (per-layer pools ``[2, numPages, 128, Hkv, D]``),
``cpp/runtime/state/kvPageTable.{h,cpp}`` (host-truth table, −1 = unused, dirty-row upload) and
``cpp/common/pagedKvTypes.h`` (page size 128; here it is a runtime parameter, 64 by default).
Page accounting is delegated to the native allocator when the runtime extension is built.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from ..config import ModelConfig, LAYER_ATTENTION


class PageAllocator:
    """Free-list page allocator with reference counts (shared prefix pages)."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))
        self._ref = [0] * num_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n > len(self._free):
            raise MemoryError(f"KV pool exhausted: want {n} pages, {len(self._free)} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._ref[p] = 1
        return out

    def retain(self, pages: Sequence[int]) -> None:
        for p in pages:
            if self._ref[p] <= 0:
                raise ValueError(f"retain of free page {p}")
            self._ref[p] += 1

    def release(self, pages: Sequence[int]) -> None:
        for p in pages:
            if self._ref[p] <= 0:
                raise ValueError(f"double free of page {p}")
            self._ref[p] -= 1
            if self._ref[p] == 0:
                self._free.append(p)


class KVCacheManager:
    """Owns the pool tensor, the allocator and the per-seat page table."""

    def __init__(self, cfg: ModelConfig, num_pages: int, page_size: int = 64, max_seats: int = 64,
                 max_pages_per_seq: int = 64, device="cpu", dtype: Optional[torch.dtype] = None,
                 num_layers: Optional[int] = None, bounded_swa: Optional[bool] = None, kv_dtype: Optional[str] = None):
        """``kv_dtype``: ``"fp8"`` stores keys and values as E4M3 bytes (half the bytes per cached token; the attention layers
        work on a 16-bit staging copy of the pages a step touches, see ``csrc/kernels/kv_fp8.cu``); ``None`` / ``"auto"`` follows
        the checkpoint's ``kv_cache_quant`` setting; ``"fp16"`` / ``"bf16"`` / ``"model"`` keep the compute type."""
        self.cfg = cfg
        # Bounded sliding-window storage (``cpp/runtime/state/boundedSwaKVPageManager.cpp`` in the reference): every
        # attention layer of the model looks back at most `sliding_window` tokens, so pages that lie wholly before the
        # window are handed back to the pool as the sequence grows.  Both attention kernels start their KV loop at a
        # 128-token tile boundary at or below `past - window + 1`; the retire boundary is rounded down the same way.
        win = getattr(cfg, "sliding_window", None)
        per_layer = getattr(cfg, "layer_windows", None)
        if per_layer:                            # mixed stacks: one full-attention layer keeps every page alive
            win = max(per_layer) if all(per_layer) else 0
        self.window = int(win) if win else 0
        self.bounded_swa = bool(self.window) if bounded_swa is None else (bool(bounded_swa) and bool(self.window))
        self.retired_pages = 0
        self.page_size = page_size
        self.max_seats = max_seats
        self.max_pages_per_seq = max_pages_per_seq
        self.num_layers = num_layers if num_layers is not None else sum(t == LAYER_ATTENTION for t in cfg.layer_types)
        hkv = max(cfg.num_key_value_heads // cfg.tp_size, 1)
        self.dtype = dtype or cfg.compute_dtype
        if kv_dtype in (None, "auto"):
            kv_dtype = getattr(cfg.quant, "kv_cache_quant", None)
        self.kv_fp8 = str(kv_dtype).lower() in ("fp8", "fp8_e4m3", "e4m3") and dtype is None
        if self.kv_fp8:
            if cfg.head_dim % 16:
                raise ValueError("an FP8 KV cache needs a head_dim that is a multiple of 16")
            self.dtype = torch.float8_e4m3fn
        self.pool = torch.zeros(self.num_layers, num_pages, 2, hkv, page_size, cfg.head_dim, dtype=self.dtype, device=device)
        # hybrid models: model layer index → attention pool index, plus the recurrent state pools
        self._attn_index = {}
        for i, t in enumerate(cfg.layer_types):
            if t == LAYER_ATTENTION:
                self._attn_index[i] = len(self._attn_index)
        self.recurrent = None
        if cfg.is_hybrid:
            from ..models.nemotron_h import RecurrentState
            self.recurrent = RecurrentState(cfg, max_seats, device, cfg.compute_dtype if self.kv_fp8 else self.dtype)
        self.alloc = PageAllocator(num_pages)
        self.table = torch.full((max_seats, max_pages_per_seq), -1, dtype=torch.int32)   # host truth
        self.lengths = [0] * max_seats
        self._pages: Dict[int, List[int]] = {}
        self.table_version = 0       # bumped whenever a row of `table` changes (device copies compare it to know they are stale)
        # Page accounting lives in the native table when the runtime module is built; the Python
        # structures above mirror it so callers can read `lengths` / `table` directly.
        try:
            from . import native as _rt
            self.native = _rt.KVPageTable(num_pages, page_size, max_seats, max_pages_per_seq)
        except ImportError:
            self.native = None

    def kv_layer(self, model_layer: int) -> torch.Tensor:
        """KV pool of attention layer ``model_layer`` (index into the model's layer list)."""
        return self.pool[self._attn_index[model_layer]]

    @property
    def bytes_per_token(self) -> int:
        return self.pool[:, 0, :, :, 0].numel() * self.pool.element_size()

    def capacity_tokens(self, seat: int) -> int:
        return len(self._pages.get(seat, [])) * self.page_size

    def reserve(self, seat: int, total_tokens: int) -> None:
        """Grow ``seat``'s page list so it can hold ``total_tokens``."""
        need = (total_tokens + self.page_size - 1) // self.page_size
        have = self._pages.setdefault(seat, [])
        if need > self.max_pages_per_seq:
            raise ValueError(f"sequence of {total_tokens} tokens exceeds {self.max_pages_per_seq} pages")
        if need > len(have):
            if self.native is not None:
                self.native.reserve(seat, total_tokens)
                pages = list(self.native.pages(seat))
                new = pages[len(have):]
            else:
                new = self.alloc.alloc(need - len(have))
            self.table[seat, len(have):need] = torch.tensor(new, dtype=torch.int32)
            have.extend(new)
            self.table_version += 1

    def adopt_prefix(self, seat: int, pages: Sequence[int], tokens: int) -> None:
        """Share already-filled pages (prefix reuse); the seat must be empty."""
        assert not self._pages.get(seat)
        if self.native is not None:
            self.native.adopt_prefix(seat, list(pages), tokens)
        else:
            self.alloc.retain(pages)
        self._pages[seat] = list(pages)
        self.table[seat, :len(pages)] = torch.tensor(list(pages), dtype=torch.int32)
        self.lengths[seat] = tokens
        self.table_version += 1

    def commit(self, seat: int, new_tokens: int) -> None:
        self.lengths[seat] += new_tokens
        if self.native is not None:
            self.native.commit(seat, new_tokens)
        if self.bounded_swa:
            self._retire(seat)

    SWA_TILE = 128          # KV tile of the attention kernels: the first tile they touch starts at a multiple of this

    def first_live_token(self, length: int) -> int:
        return max(0, (length - self.window + 1) // self.SWA_TILE * self.SWA_TILE)

    def swa_live_pages_bound(self, step_tokens: int) -> int:
        """Most pages one sequence can hold at once when each step appends at most ``step_tokens``."""
        p = self.page_size
        return min((self.window + self.SWA_TILE + step_tokens + p - 1) // p + 1, self.max_pages_per_seq)

    def _retire(self, seat: int) -> None:
        first = self.first_live_token(self.lengths[seat])
        have = self._pages.get(seat, [])
        upto = min(len(have), first // self.page_size)
        if upto == 0 or all(pg < 0 for pg in have[:upto]):
            return
        if self.native is not None:
            self.retired_pages += self.native.retire_before(seat, first)
        else:
            gone = [pg for pg in have[:upto] if pg >= 0]
            self.alloc.release(gone)
            self.retired_pages += len(gone)
        for i in range(upto):
            have[i] = -1
        self.table[seat, :upto] = -1
        self.table_version += 1

    def live_pages(self, seat: int) -> int:
        return sum(pg >= 0 for pg in self._pages.get(seat, []))

    def rewind(self, seat: int, length: int) -> None:
        """Drop everything after ``length`` tokens (speculative rejection); pages are kept."""
        assert length <= self.lengths[seat]
        self.lengths[seat] = length
        if self.native is not None:
            self.native.rewind(seat, length)

    def free(self, seat: int) -> None:
        pages = self._pages.pop(seat, [])
        if self.native is not None:
            self.native.free_seat(seat)
        else:
            self.alloc.release([pg for pg in pages if pg >= 0])
        self.table[seat].fill_(-1)
        self.lengths[seat] = 0
        self.table_version += 1

    def pages_of(self, seat: int) -> List[int]:
        return list(self._pages.get(seat, []))

    def table_rows(self, seats: Sequence[int]) -> torch.Tensor:
        return self.table[list(seats)]
