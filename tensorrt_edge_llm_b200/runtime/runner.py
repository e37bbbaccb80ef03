"""Model runner: executes ragged steps (prefill chunks, decode rows, mixed) on one rank.

This is the counterpart of the reference's ``EngineExecutor`` + ``LLMRankRuntime`` step
functions (``cpp/runtime/exec/engineExecutor.h:94-271``, ``cpp/runtime/llmRankRuntime.cpp``
``runBaseModelPrefill`` :4758, ``captureDecodingCUDAGraph`` :5326, vanilla decode
``cpp/runtime/decoding/vanillaDecoder.cpp:67-181,304-404``) without a TensorRT engine: the
"engine" is the PyTorch module whose leaves are sm_100a kernels.  Prefill runs eagerly;
all-resident decode steps replay a CUDA graph per batch size, with device-resident step state
(lengths, positions, token feedback) so a run of decode steps needs no host round trip.
"""
from __future__ import annotations

import contextlib
import os

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from ..ops.meta import StepMeta, build_step_meta
from .. import profiling as prof
from .kv_cache import KVCacheManager


@dataclass
class SamplingParams:
    """Per-request sampling controls (``cpp/sampler/sampling.h:36-100`` semantics)."""

    max_tokens: int = 128
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 42
    ignore_eos: bool = False
    stop_token_ids: Sequence[int] = ()
    logprobs: Optional[int] = None          # None = off; k = report the chosen token's log-probability and the k most likely
    logit_bias: Optional[dict] = None       # token id → additive bias on its logit
    guided: Optional[object] = None         # runtime.guided.GuidedDecodingParams
    disable_spec_decode: bool = False       # on a speculative deployment: decode this request token by token
    lora_name: Optional[str] = None         # adapter (loaded with LLM.load_lora) applied to this request's rows
    context_cache_lookup: bool = True       # False = bypass the prefix cache for this request
    context_cache_commit: str = "prefill_state_only"     # "none" | "prefill_state_only" | "including_generated_tokens"
    max_denoising_steps: int = 0            # block-diffusion checkpoints: denoise passes per block (0 = the checkpoint's default)

    @property
    def needs_logits_processing(self) -> bool:
        return self.logprobs is not None or bool(self.logit_bias) or self.guided is not None


class ModelRunner:
    def __init__(self, model, kv: KVCacheManager, device=None, max_num_tokens: int = 8192):
        self.model = model
        self.kv = kv
        self.device = torch.device(device) if device is not None else kv.pool.device
        pool_dev = kv.pool.device
        if self.device.type != pool_dev.type or (self.device.index or 0) != (pool_dev.index or 0):
            raise ValueError(f"runner device {self.device} differs from the KV pool's device {pool_dev}")
        self.device = pool_dev
        self.max_num_tokens = max_num_tokens
        self._graphs: Dict[int, "_DecodeGraph"] = {}
        # EDGELLM_DISABLE_CUDA_GRAPH=1 (the reference's switch, cpp/runtime/multiDevice/runtimeCoordinator.cpp:680) keeps decode eager
        self.use_cuda_graphs = self.device.type == "cuda" and os.environ.get("EDGELLM_DISABLE_CUDA_GRAPH", "0") != "1"
        # hybrid models address attention pools and recurrent state pools through the manager itself
        self.cache = kv if getattr(model, "needs_cache_set", False) else kv.pool
        # reduced-vocabulary LM head: logits cover `vocab_map.numel()` columns, column c is token vocab_map[c]
        self.vocab_map: Optional[torch.Tensor] = None
        self.rope_delta: dict = {}          # seat → multimodal RoPE position offset of its decode rows

    # ---- eager ragged step -----------------------------------------------------------------
    def _meta(self, seats: Sequence[int], q_lens: Sequence[int], logits_all=False, tree_mask=None,
              positions=None) -> StepMeta:
        past = [self.kv.lengths[s] for s in seats]
        for s, q, p in zip(seats, q_lens, past):
            if p == 0:
                self.rope_delta.pop(s, None)          # a fresh sequence on this seat
            self.kv.reserve(s, p + q)
        meta = build_step_meta(q_lens, past, self.kv.table_rows(seats), self.kv.page_size, slot_ids=seats,
                               logits_all=logits_all, device=self.device, tree_mask=tree_mask, positions=positions)
        table = getattr(self.model.cfg, "skip_softmax_prefill_table", None)
        if table and tree_mask is None and max(q_lens, default=0) > 1:
            # skip-softmax deployment: every sequence of a prefill-size step votes with the threshold of its own length
            from ..skip_softmax import thresholds_log2
            meta.skip_thr = thresholds_log2(table, [p + q for p, q in zip(past, q_lens)], device=self.device)
        return meta

    def rope_delta_empty(self) -> bool:
        """No resident sequence carries a multimodal position offset (captured passes take positions as given)."""
        return not any(self.rope_delta.values())

    @torch.no_grad()
    def step(self, seats: Sequence[int], token_lists: Sequence[Sequence[int]], logits_all=False,
             commit=True, tree_mask=None, positions=None) -> torch.Tensor:
        """Run one ragged step; returns logits ``[L, V]`` (last row of each sequence unless
        ``logits_all``).  KV lengths advance by the rows fed when ``commit``."""
        q_lens = [len(t) for t in token_lists]
        for s in seats:
            if self.kv.lengths[s] == 0:
                self.rope_delta.pop(s, None)          # a fresh sequence on this seat
        if positions is None and self.rope_delta and any(self.rope_delta.get(s) for s in seats):
            # sequences whose prompt held images: text positions run ahead of / behind the cache length by a fixed offset
            positions = [self.kv.lengths[s] + self.rope_delta.get(s, 0) + j for s, q in zip(seats, q_lens) for j in range(q)]
        meta = self._meta(seats, q_lens, logits_all, tree_mask, positions)
        flat = [t for ts in token_lists for t in ts]
        if self.device.type == "cuda":
            host = torch.tensor(flat, dtype=torch.int32).pin_memory()
            ids = host.to(self.device, non_blocking=True)
        else:
            ids = torch.tensor(flat, dtype=torch.int32)
        logits = self.model(ids, meta, self.cache)
        if commit:
            for s, q in zip(seats, q_lens):
                self.kv.commit(s, q)
        return logits

    @torch.no_grad()
    def prefill(self, seats: Sequence[int], prompts: Sequence[Sequence[int]]) -> torch.Tensor:
        """Chunked prefill of whole prompts; returns the last-token logits ``[N, V]``.

        Sequences are packed into steps of at most ``max_num_tokens`` rows; a prompt longer than
        the budget is split on page boundaries (``cpp/scheduler/stepPlanner.cpp`` rule)."""
        n = len(seats)
        with prof.time_stage(prof.PREFILL, batch=n, tokens=sum(len(x) for x in prompts)):
            return self._prefill(seats, prompts)

    def _prefill(self, seats, prompts) -> torch.Tensor:
        n = len(seats)
        done = [0] * n
        out: List[Optional[torch.Tensor]] = [None] * n
        p = self.kv.page_size
        while any(done[i] < len(prompts[i]) for i in range(n)):
            budget = self.max_num_tokens
            step_seats, step_tokens, finishing = [], [], []
            for i in range(n):
                rem = len(prompts[i]) - done[i]
                if rem == 0 or budget == 0:
                    continue
                take = min(rem, budget)
                if take < rem:
                    take = (take // p) * p
                    if take == 0:
                        continue
                step_seats.append(seats[i])
                step_tokens.append(prompts[i][done[i]:done[i] + take])
                finishing.append((i, done[i] + take == len(prompts[i])))
                done[i] += take
                budget -= take
            logits = self.step(step_seats, step_tokens)
            for row, (i, fin) in enumerate(finishing):
                if fin:
                    out[i] = logits[row]
        return torch.stack(out)  # type: ignore[arg-type]

    @torch.no_grad()
    def prefill_embeds(self, seats: Sequence[int], embeds: Sequence[torch.Tensor], positions3: Optional[Sequence[torch.Tensor]] = None,
                       rope_deltas: Optional[Sequence[int]] = None, deepstack: Optional[dict] = None) -> torch.Tensor:
        """Prefill from embedding rows instead of token ids (multimodal prompts: text rows with the image / audio
        rows already merged in).  One step; returns last-row logits ``[N, V]``.

        ``positions3`` (one ``[3, T_i]`` tensor per sequence, see ``ops.reference.mrope_positions``) switches the step to
        multimodal RoPE; ``rope_deltas`` are remembered per seat and added to the position of every later decode row."""
        q_lens = [int(e.shape[0]) for e in embeds]
        meta = self._meta(seats, q_lens)
        if deepstack:
            # {layer: (row indices into the packed step, features)}: intermediate vision levels joining the early layers
            meta.deepstack = {int(k): (torch.as_tensor(r, dtype=torch.int64, device=self.device), f.to(self.device)) for k, (r, f) in deepstack.items()}
        if positions3 is not None:
            meta.positions3 = torch.cat([p.to(torch.int32) for p in positions3], dim=1).to(self.device)
            for s, d in zip(seats, rope_deltas or [0] * len(seats)):
                self.rope_delta[s] = int(d)
        x = torch.cat([e.to(self.device) for e in embeds], dim=0).to(self.model.cfg.compute_dtype)
        logits = self.model(None, meta, self.cache, inputs_embeds=x)
        for s, q in zip(seats, q_lens):
            self.kv.commit(s, q)
        return logits

    @torch.no_grad()
    def step_embeds(self, seats: Sequence[int], embeds: Sequence[torch.Tensor], positions3: Optional[Sequence[Optional[torch.Tensor]]] = None,
                    deepstack: Optional[dict] = None) -> torch.Tensor:
        """One ragged step whose rows are embedding rows: prompt chunks of multimodal requests next to ordinary prompt chunks
        and decode rows (already embedded by the caller).  ``positions3[i]`` is the ``[3, T_i]`` position block of sequence
        ``i`` or ``None`` for text-like rows, which take ``cache length + decode offset + j`` on all three components.
        ``deepstack`` indexes rows of the packed step.  Commits every row; returns last-row logits ``[N, V]``."""
        q_lens = [int(e.shape[0]) for e in embeds]
        for s in seats:
            if self.kv.lengths[s] == 0:
                self.rope_delta.pop(s, None)              # a fresh sequence on this seat
        base = [self.kv.lengths[s] + self.rope_delta.get(s, 0) for s in seats]
        flat_pos = [b + j for b, q in zip(base, q_lens) for j in range(q)]
        meta = self._meta(seats, q_lens, positions=flat_pos)
        if positions3 is not None and any(p is not None for p in positions3):
            blocks = []
            for p3, b, q in zip(positions3, base, q_lens):
                blocks.append(p3.to(torch.int32) if p3 is not None else torch.arange(b, b + q, dtype=torch.int32)[None, :].expand(3, q))
            meta.positions3 = torch.cat(blocks, dim=1).to(self.device)
        if deepstack:
            meta.deepstack = {int(k): (torch.as_tensor(r, dtype=torch.int64, device=self.device), f.to(self.device)) for k, (r, f) in deepstack.items()}
        x = torch.cat([e.to(self.device) for e in embeds], dim=0).to(self.model.cfg.compute_dtype)
        logits = self.model(None, meta, self.cache, inputs_embeds=x)
        for s, q in zip(seats, q_lens):
            self.kv.commit(s, q)
        return logits

    def embed_tokens(self, ids: Sequence[int]) -> torch.Tensor:
        t = torch.tensor(list(ids), dtype=torch.int32, device=self.device)
        e = ops.embedding(t, self.model.model.embed_tokens.weight)
        scale = getattr(self.model.model, "embed_scale", 1.0)      # Gemma multiplies looked-up rows (1.0 once folded into the table)
        return e if scale == 1.0 else (e * torch.tensor(scale, dtype=e.dtype)).to(e.dtype)

    @torch.no_grad()
    def prefill_tensor(self, seats: Sequence[int], ids: torch.Tensor) -> torch.Tensor:
        """Prefill equal-length prompts given as one tensor ``[N, S]`` (pinned host or device
        memory); chunks hold whole sequences.  Returns last-token logits ``[N, V]``."""
        n, s_len = ids.shape
        per = max(1, self.max_num_tokens // s_len)
        outs = []
        for b0 in range(0, n, per):
            grp = list(seats[b0:b0 + per])
            meta = self._meta(grp, [s_len] * len(grp))
            chunk = ids[b0:b0 + per].reshape(-1)
            if chunk.device != self.device:
                chunk = chunk.to(self.device, non_blocking=True)
            outs.append(self.model(chunk.to(torch.int32), meta, self.cache))
            for sidx in grp:
                self.kv.commit(sidx, s_len)
        return torch.cat(outs, dim=0)

    # ---- sampling --------------------------------------------------------------------------
    def sample(self, logits: torch.Tensor, sp: SamplingParams, step: int = 0) -> torch.Tensor:
        """Next token per row.  Greedy when ``temperature < 1e-3``; otherwise per-row top-k/top-p
        with a counter-based uniform per (seed, row, step) so draws do not depend on batch position."""
        if sp.temperature < 1e-3:
            return self.pick(logits)
        n = logits.shape[0]
        dev = logits.device
        # uniforms: one generator stream per (seed, step), as before, but drawn for 64 steps at a time and uploaded in one copy;
        # the per-row sampling parameters are constant over a generation and live on the device
        blk, off = divmod(int(step), 64)
        key = (sp.seed, n, blk, str(dev))
        cache = self.__dict__.setdefault("_uniform_cache", {})
        if key not in cache:
            if len(cache) > 8:
                cache.clear()
            rows = [torch.rand(n, generator=torch.Generator(device="cpu").manual_seed(sp.seed * 1000003 + blk * 64 + j)) for j in range(64)]
            cache[key] = torch.stack(rows).to(dev)
        u = cache[key][off]
        pkey = (n, float(sp.temperature), int(sp.top_k), float(sp.top_p), str(dev))
        params = self.__dict__.setdefault("_sample_params", {})
        if pkey not in params:
            if len(params) > 16:
                params.clear()
            params[pkey] = (torch.full((n,), sp.temperature, device=dev), torch.full((n,), sp.top_k, device=dev, dtype=torch.int32),
                            torch.full((n,), sp.top_p, device=dev))
        t, k, p = params[pkey]
        return self.to_full_vocab(ops.sample(logits, t, k, p, u))

    def to_full_vocab(self, cols: torch.Tensor) -> torch.Tensor:
        return cols if self.vocab_map is None else self.vocab_map[cols.long()]

    def pick(self, logits: torch.Tensor) -> torch.Tensor:
        """Greedy token per row, as ids of the full vocabulary."""
        return self.to_full_vocab(ops.argmax(logits))

    def greedy_step(self, ids: torch.Tensor, meta: StepMeta) -> torch.Tensor:
        """One model step that ends in the greedy token of every logits row.  Models with a vocabulary-sharded head
        exchange per-shard candidates instead of gathering the logits (``CausalLM.greedy_tokens``)."""
        g = getattr(self.model, "greedy_tokens", None)
        if g is None:
            return self.pick(self.model(ids, meta, self.cache))
        return self.to_full_vocab(g(ids, meta, self.cache))

    def _candidate_k(self, sp: SamplingParams) -> int:
        """Candidates per vocabulary shard that make sampling over them exact, or 0 when the sampler needs every logit (no
        top-k and no top-p cut) or the model's head is not sharded."""
        comm = getattr(self.model, "comm", None)
        if comm is None or getattr(comm, "world_size", 1) <= 1 or not hasattr(self.model, "candidates_from_hidden"):
            return 0
        if not self.model.supports_candidate_sampling() or self.vocab_map is not None:
            return 0
        if sp.top_k and sp.top_k > 0:
            return min(int(sp.top_k), 1024)
        return 1024 if sp.top_p < 1.0 else 0             # top-p alone: the sampler's own candidate cap

    @torch.no_grad()
    def step_candidates(self, seats: Sequence[int], token_lists: Sequence[Sequence[int]], k: int):
        """One ragged decode step that ends in per-shard candidates instead of logits (tensor-parallel sampling without the
        full-vocabulary gather): ``(values [B, world · k], token ids [B, world · k])``."""
        q_lens = [len(t) for t in token_lists]
        positions = None
        if self.rope_delta and any(self.rope_delta.get(s) for s in seats):
            positions = [self.kv.lengths[s] + self.rope_delta.get(s, 0) + j for s, q in zip(seats, q_lens) for j in range(q)]
        meta = self._meta(seats, q_lens, False, None, positions)
        ids = torch.tensor([t for ts in token_lists for t in ts], dtype=torch.int32).to(self.device)
        x = self.model.hidden_states(ids, meta, self.cache)
        out = self.model.candidates_from_hidden(x, meta, k)
        for s, q in zip(seats, q_lens):
            self.kv.commit(s, q)
        return out

    @torch.no_grad()
    def decode_sampled(self, seats, first_tokens, steps, sp: SamplingParams) -> torch.Tensor:
        toks = first_tokens.to(torch.int32)
        cols = []
        kc = self._candidate_k(sp)
        for i in range(steps):
            feed = [[int(t)] for t in toks.tolist()]
            if kc:
                # vocabulary-sharded head: sample over the exchanged per-shard candidates, then map the pick back to its token
                vals, ids = self.step_candidates(seats, feed, kc)
                pick = self.sample(vals, sp, step=i + 1).long()
                toks = ids.gather(1, pick[:, None])[:, 0].to(torch.int32)
            else:
                toks = self.sample(self.step(seats, feed), sp, step=i + 1)
            cols.append(toks)
        return torch.stack(cols, dim=1)

    # ---- decode ----------------------------------------------------------------------------
    def can_graph_step(self, seats: Sequence[int]) -> bool:
        """Whether one all-resident greedy decode step of these seats may run from the captured graph."""
        return (self.use_cuda_graphs and not self.kv.bounded_swa and len(seats) > 0
                and not any(self.rope_delta.get(s) for s in seats))

    @torch.no_grad()
    def decode_step_graph(self, seats: Sequence[int], tokens: Sequence[int]) -> List[int]:
        """One all-resident greedy decode step from the captured graph of this batch size: feeds ``tokens[i]`` to seat
        ``seats[i]``, commits one KV position per seat and returns the next tokens (one device → host read).

        This is the in-flight-batching form of ``decode_greedy``: the request engine calls it step by step.  While the
        same seats decode back to back and feed the tokens the graph itself produced, the step state (lengths,
        positions, page-table rows, token feedback) already sits on the device and the step is a replay plus the read;
        any other step (a new or departed sequence, an eager step in between, a grown page table) reloads the state first.
        Reference: the all-resident decode steps of ``docs/source/developer_guide/software-design/in-flight-batching.md:351-372``
        and ``cpp/runtime/decoding/vanillaDecoder.cpp:446-491`` replay a captured graph the same way."""
        n = len(seats)
        nb = self.graph_bucket(n)
        g = self._graphs.get(nb)
        if g is None:
            g = self._graphs[nb] = _DecodeGraph(self, nb)
        seats, tokens = list(seats), [int(t) for t in tokens]
        # rows up to the bucket size repeat the last real row (same seat, same token, same position): they recompute and
        # rewrite exactly what that row writes, and their outputs are dropped
        seats += [seats[-1]] * (nb - n)
        tokens += [tokens[-1]] * (nb - n)
        with prof.time_stage(prof.VANILLA_DECODING, batch=n, tokens=n):
            return g.step(seats, tokens, n)

    def graph_bucket(self, n: int) -> int:
        """Batch size of the graph that serves ``n`` decode rows.  A serving run sees every batch size between 1 and the
        seat count; one capture per size would be dozens of captures, so sizes above 8 share the graph of the next
        multiple of 8 (the extra rows repeat the last row).  Models with recurrent layers keep exact sizes: a repeated
        row would advance that sequence's state twice."""
        if n <= 8 or getattr(self.model.cfg, "is_hybrid", False):
            return n
        return min((n + 7) // 8 * 8, max(self.kv.max_seats, n))

    @torch.no_grad()
    def decode_greedy(self, seats: Sequence[int], first_tokens: torch.Tensor, steps: int) -> torch.Tensor:
        """Greedy decode ``steps`` tokens for every seat starting from ``first_tokens [N]``;
        returns ``[N, steps]`` int32 (the tokens *generated*, not including ``first_tokens``).

        On CUDA the steps replay one captured graph whose device-side state advances by itself;
        the host copies the token matrix back once at the end."""
        with prof.time_stage(prof.VANILLA_DECODING, batch=len(seats), tokens=len(seats) * steps):
            return self._decode_greedy(seats, first_tokens, steps)

    def _decode_greedy(self, seats, first_tokens, steps) -> torch.Tensor:
        n = len(seats)
        for s in seats:
            self.kv.reserve(s, self.kv.lengths[s] + steps)
        if self.use_cuda_graphs and not any(self.rope_delta.get(s) for s in seats):
            g = self._graphs.get(n)
            if g is None:
                g = self._graphs[n] = _DecodeGraph(self, n)
            out = g.run(seats, first_tokens, steps)
        else:
            toks = first_tokens.to(torch.int32)
            cols = []
            for _ in range(steps):
                logits = self.step(seats, [[int(t)] for t in toks.tolist()])
                toks = self.pick(logits)
                cols.append(toks)
            return torch.stack(cols, dim=1)
        for s in seats:
            self.kv.commit(s, steps)
        return out


@contextlib.contextmanager
def capture_guard():
    """No cyclic garbage collection while a stream is capturing: a collected object that owns a CUDA graph (an old decoder,
    a runner of an earlier model) destroys it from this thread, which the capture treats as a prohibited call and dies of."""
    import gc
    was = gc.isenabled()
    gc.collect()
    gc.disable()
    try:
        yield
    finally:
        if was:
            gc.enable()


class _DecodeGraph:
    """A captured all-resident decode step for a fixed batch size.

    Static device state: ``ids`` (fed back from the sampler), ``past_len`` / ``positions``
    (advanced by the captured increment), the page-table rows and the output token ring."""

    MAX_STEPS = 4096

    def __init__(self, runner: ModelRunner, n: int):
        self.r = runner
        self.n = n
        dev = runner.device
        kv = runner.kv
        i32 = dict(dtype=torch.int32, device=dev)
        self.ids = torch.zeros(n, **i32)
        self.meta = StepMeta(
            q_start=torch.arange(n + 1, **i32), q_len=torch.ones(n, **i32), past_len=torch.zeros(n, **i32),
            positions=torch.zeros(n, **i32), seq_ids=torch.arange(n, **i32),
            page_table=torch.full((n, kv.max_pages_per_seq), -1, **i32), slot_ids=torch.zeros(n, **i32),
            logits_idx=torch.arange(n, **i32), page_size=kv.page_size, num_seqs=n, num_tokens=n,
            max_q_len=1, max_seq_len=kv.max_pages_per_seq * kv.page_size)
        self.out = torch.zeros(self.MAX_STEPS, n, **i32)
        self.step_idx = torch.zeros(1, dtype=torch.int64, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._pin = torch.empty(n * (kv.max_pages_per_seq + 3), dtype=torch.int32, pin_memory=True)
        # stepped use (in-flight batching): what the device-side state currently describes, as the host knows it
        self._tok_pin = torch.empty(n, dtype=torch.int32, pin_memory=True)
        self._tok_event = torch.cuda.Event()
        self._key: Optional[tuple] = None
        self._host_len: List[int] = []
        self._last_tokens: List[int] = []
        self._table_version = -1
        self._ring_used = 0
        self.reloads = 0              # times a step had to rebuild the device state (diagnostics / tests)

    def _body(self):
        m = self.meta
        tok = self.r.greedy_step(self.ids, m)
        self.ids.copy_(tok)
        self.out.index_copy_(0, self.step_idx, tok.unsqueeze(0))
        self.step_idx.add_(1)
        m.past_len.add_(1)
        m.positions.add_(1)

    def _load_state(self, seats, first_tokens):
        kv = self.r.kv
        n, mp = self.n, kv.max_pages_per_seq
        host = self._pin
        host[:n] = torch.tensor([kv.lengths[s] for s in seats], dtype=torch.int32)
        host[n:2 * n] = torch.tensor(list(seats), dtype=torch.int32)
        host[2 * n:3 * n] = first_tokens.to("cpu", torch.int32) if first_tokens.device.type != "cpu" else first_tokens.to(torch.int32)
        host[3 * n:] = kv.table_rows(seats).reshape(-1)
        devbuf = host.to(self.r.device, non_blocking=True)
        self.meta.past_len.copy_(devbuf[:n])
        self.meta.positions.copy_(devbuf[:n])
        self.meta.slot_ids.copy_(devbuf[n:2 * n])
        self.ids.copy_(devbuf[2 * n:3 * n])
        self.meta.page_table.copy_(devbuf[3 * n:].view(n, mp))
        self.step_idx.zero_()

    def step(self, seats: List[int], tokens: List[int], n_real: Optional[int] = None) -> List[int]:
        kv = self.r.kv
        n_real = len(seats) if n_real is None else n_real
        lens = [kv.lengths[s] for s in seats]
        for s, ln in zip(seats, lens):
            if kv.capacity_tokens(s) < ln + 1:
                kv.reserve(s, ln + 1)                      # bumps kv.table_version: the state below is rebuilt
        stale = (self.graph is None or self._key != tuple(seats) or self._host_len != lens or self._last_tokens != tokens
                 or self._table_version != kv.table_version or self._ring_used >= self.MAX_STEPS - 1)
        if stale:
            first = torch.tensor(tokens, dtype=torch.int32)
            self._load_state(seats, first)
            self._ensure_graph(seats, first)
            self._key, self._table_version, self._ring_used = tuple(seats), kv.table_version, 0
            self.reloads += 1
        from ..ops import cuda as _cu
        self.graph.replay()
        _cu.LAUNCHES += self.launches_per_replay
        self._tok_pin.copy_(self.ids, non_blocking=True)
        self._tok_event.record()
        self._tok_event.synchronize()
        out = self._tok_pin.tolist()
        self._ring_used += 1
        self._host_len = [ln + 1 for ln in lens]
        self._last_tokens = out
        for s in seats[:n_real]:
            kv.commit(s, 1)
        return out[:n_real]

    def _ensure_graph(self, seats, first_tokens):
        if self.graph is None:
            self.run(seats, first_tokens, 0)

    def run(self, seats, first_tokens, steps):
        assert steps <= self.MAX_STEPS
        self._key = None                  # a whole run leaves the stepped bookkeeping behind
        self._load_state(seats, first_tokens)
        if self.graph is None:
            # warm up once eagerly (allocator, lazy kernels), restore state, then capture
            s = torch.cuda.Stream(device=self.r.device)
            s.wait_stream(torch.cuda.current_stream(self.r.device))
            with torch.cuda.stream(s):
                self._body()
            torch.cuda.current_stream(self.r.device).wait_stream(s)
            self._load_state(seats, first_tokens)
            from ..ops import cuda as _cu
            before = _cu.LAUNCHES
            g = torch.cuda.CUDAGraph()
            # thread-local capture mode: other threads of a server (media encoders, tokenisation) may call into CUDA meanwhile
            with capture_guard(), torch.cuda.graph(g, capture_error_mode="thread_local"):
                self._body()
            self.graph = g
            self.launches_per_replay = _cu.LAUNCHES - before
            _cu.LAUNCHES = before
            self._load_state(seats, first_tokens)
        from ..ops import cuda as _cu
        for _ in range(steps):
            self.graph.replay()
        _cu.LAUNCHES += steps * self.launches_per_replay
        return self.out[:steps].t().contiguous()
