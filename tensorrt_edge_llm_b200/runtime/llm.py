"""Offline generation API: ``LLM(...).generate(prompts, SamplingParams)``.

Parity: ``tensorrt_edgellm.server.LLM`` / ``SamplingParams``
(``tensorrt_edgellm/server/runtime/engine.py:920-2167``; usage in
``docs/source/user_guide/examples/server.md:27-64``).  Construction takes a checkpoint directory
or a :class:`ModelConfig` (random-init weights, for benchmarks without network access).
"""
from __future__ import annotations

import dataclasses
import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Union

import torch

from ..config import (QUANT_NVFP4, Mapping, ModelConfig, QuantConfig)
from ..model import AutoModel
from .kv_cache import KVCacheManager
from .runner import ModelRunner, SamplingParams


@dataclass
class RequestOutput:
    prompt_token_ids: List[int]
    token_ids: List[int]
    text: Optional[str] = None
    finish_reason: str = "length"
    ttft_s: float = 0.0
    decode_s: float = 0.0


class LLM:
    def __init__(self, model: Union[str, ModelConfig], *, device: Optional[str] = None, comm=None,
                 max_batch_size: int = 64, max_input_len: int = 2048, max_kv_cache_capacity: int = 2304,
                 page_size: int = 64, max_num_tokens: int = 8192, random_init_seed: Optional[int] = 0,
                 tokenizer=None, kv_pages: Optional[int] = None):
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        self.device = torch.device(device)
        if isinstance(model, ModelConfig):
            self.model = AutoModel.from_config(model, comm=comm, device=self.device, random_init=random_init_seed)
        else:
            self.model = AutoModel.from_pretrained(model, comm=comm, device=self.device)
        self.cfg = self.model.cfg
        self.tokenizer = tokenizer
        self.max_batch_size = max_batch_size
        self.max_input_len = max_input_len
        pages_per_seq = (max_kv_cache_capacity + page_size - 1) // page_size
        total_pages = kv_pages or (pages_per_seq * max_batch_size + 1)
        self.kv = KVCacheManager(self.cfg, total_pages, page_size, max_seats=max_batch_size,
                                 max_pages_per_seq=pages_per_seq, device=self.device)
        self.runner = ModelRunner(self.model, self.kv, self.device, max_num_tokens=max_num_tokens)

    # ------------------------------------------------------------------------------------------
    def _encode(self, prompts) -> List[List[int]]:
        out = []
        for p in prompts:
            if isinstance(p, str):
                if self.tokenizer is None:
                    raise ValueError("text prompts need a tokenizer")
                out.append(list(self.tokenizer.encode(p)))
            else:
                out.append([int(t) for t in p])
        return out

    @torch.no_grad()
    def generate(self, prompts: Sequence[Union[str, Sequence[int]]], sampling_params: Optional[SamplingParams] = None
                 ) -> List[RequestOutput]:
        """Generate for a batch of prompts (static batch: one prefill wave, then decode)."""
        sp = sampling_params or SamplingParams()
        if isinstance(prompts, torch.Tensor):
            outs = []
            for b0 in range(0, prompts.shape[0], self.max_batch_size):
                outs.extend(self._generate_batch(prompts[b0:b0 + self.max_batch_size], sp))
            return outs
        ids = self._encode(prompts)
        outs: List[RequestOutput] = []
        for b0 in range(0, len(ids), self.max_batch_size):
            outs.extend(self._generate_batch(ids[b0:b0 + self.max_batch_size], sp))
        return outs

    def _generate_batch(self, ids: List[List[int]], sp: SamplingParams) -> List[RequestOutput]:
        n = len(ids)
        seats = list(range(n))
        for s in seats:
            self.kv.free(s)
        for s, p in zip(seats, ids):
            if len(p) > self.max_input_len:
                raise ValueError(f"prompt of {len(p)} tokens exceeds max_input_len {self.max_input_len}")
            self.kv.reserve(s, len(p) + sp.max_tokens)
        t0 = time.perf_counter()
        if isinstance(ids, torch.Tensor):
            logits = self.runner.prefill_tensor(seats, ids)      # pinned host tensor → one H2D copy per chunk
        else:
            logits = self.runner.prefill(seats, ids)
        first = self.runner.sample(logits, sp, step=0)
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        t1 = time.perf_counter()
        if sp.max_tokens > 1:
            if sp.temperature < 1e-3:
                rest = self.runner.decode_greedy(seats, first, sp.max_tokens - 1)
            else:
                rest = self.runner.decode_sampled(seats, first, sp.max_tokens - 1, sp)
            toks = torch.cat([first[:, None].to(rest.device), rest], dim=1)
        else:
            toks = first[:, None]
        toks_host = toks.to("cpu")          # device → host read of the step's result
        t2 = time.perf_counter()
        outs = []
        eos = self.cfg.eos_token_id
        eos_set = set(eos if isinstance(eos, (list, tuple)) else [eos]) if eos is not None else set()
        eos_set |= set(sp.stop_token_ids)
        for i in range(n):
            row = toks_host[i].tolist()
            reason = "length"
            if not sp.ignore_eos and eos_set:
                for j, t in enumerate(row):
                    if t in eos_set:
                        row = row[:j + 1]
                        reason = "stop"
                        break
            text = self.tokenizer.decode(row) if self.tokenizer is not None else None
            outs.append(RequestOutput(ids[i].tolist() if isinstance(ids, torch.Tensor) else ids[i], row, text, reason,
                                      t1 - t0, t2 - t1))
        for s in seats:
            self.kv.free(s)
        return outs

    def close(self):
        self.runner = None
        self.kv = None
        self.model = None
