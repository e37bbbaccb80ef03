"""The model-side implementation of the scheduler's ``RuntimeSession`` seam.

The native ``RequestEngine`` plans steps (chunked prefill + decode rows, compact layout) and
calls ``execute(plan)``; this session turns a plan into one ragged model step through
``ModelRunner``, samples the rows that produce tokens and reports deltas.  KV pages come from
the native ``KVPageTable``; with ``enable_prefix_cache`` full prompt pages are shared between
requests through the native ``PrefixCache``.

Parity: ``RankRuntimeSession`` (``cpp/runtime/runtimeSession.{h,cpp}``: admit :325, execute :628,
executeContext/Decode/Compact) and the context-cache request flow
(``cpp/runtime/contextCacheRequest.*``).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Optional

import torch

from .. import ops
from .. import profiling as prof
from ..ops.meta import build_step_meta
from . import logits as lp
from . import native as rt
from .runner import ModelRunner, SamplingParams


class _Seq:
    __slots__ = ("req", "request_id", "tokens", "generated", "last_token", "finished", "row_state", "plain", "feed", "mm")

    def __init__(self, req, request_id):
        self.req, self.request_id = req, request_id
        self.tokens: List[int] = list(req.prompt_ids)
        self.generated = 0
        self.last_token: Optional[int] = None
        self.finished = False
        self.row_state = None            # logits.RowState when the request biases, constrains or reports log-probabilities
        self.feed: List[int] = []        # emitted tokens whose KV is not written yet, when more than the last one (jump-forward)
        self.mm: Optional[dict] = None   # multimodal prompt: embedding rows, 3-D positions, decode offset, deepstack levels


class ModelSession(rt.RuntimeSession):
    def __init__(self, runner: ModelRunner, eos_ids=(), enable_prefix_cache: bool = False, max_input_len: int = 2048,
                 guided_vocab=None, max_snapshots: int = 64, max_records: int = 4096, spec_decoder=None, mirror=None):
        super().__init__()
        self.runner = runner
        self.guided_vocab = guided_vocab
        # Speculative decoding under in-flight batching: resident decode rows advance by one draft → verify round per
        # step (several tokens per delta), whole prompts are prefilled through the decoder so the draft sees them too.
        # tensor parallelism: operations that touch the model are broadcast to the follower ranks first (parallel/tp_serving.py)
        self.mirror = mirror
        if mirror is not None:
            if spec_decoder is not None:
                raise ValueError("speculative decoding is not mirrored to follower ranks")
            if runner.model.cfg.is_hybrid:
                enable_prefix_cache = False    # recurrent-state snapshots are not mirrored to follower ranks
        self.spec = spec_decoder
        if spec_decoder is not None:
            enable_prefix_cache = False        # the draft's own KV has no shared prefix pages
        self.kv = runner.kv
        self.eos = set(int(e) for e in eos_ids if e is not None)
        self.max_input_len = max_input_len
        self.slots = rt.ResidentSlotPool(self.kv.max_seats)
        self.seqs: Dict[int, _Seq] = {}
        # retired sliding-window pages cannot be shared, so bounded storage and the prefix cache exclude each other
        self.prefix = rt.PrefixCache(self.kv.native.allocator(), self.kv.page_size, max_records) if (
            enable_prefix_cache and getattr(self.kv, "native", None) is not None and not self.kv.bounded_swa) else None
        self._swa_bound = self.kv.swa_live_pages_bound(runner.max_num_tokens) if self.kv.bounded_swa else 0
        # Hybrid models: shared KV pages alone do not restore a prefix, the recurrent rows at that boundary are needed
        # too.  Snapshots are taken at page-aligned prefill boundaries and keyed by the same chained block hash as the
        # page index (``cpp/runtime/state/contextCache/hybridSnapshotStorage.*`` in the reference).
        self.hybrid = bool(runner.model.cfg.is_hybrid)
        self.snapshots: "OrderedDict[int, list]" = OrderedDict()
        self.max_snapshots = max_snapshots
        self.snapshot_hits = 0
        self.jump_forward_tokens = 0       # tokens appended because a grammar left no choice (no forward pass of their own)
        self.graph_steps = 0               # all-resident decode steps that replayed a captured graph
        # multimodal prompts wait here between `register_embeds` (caller's thread) and admission (engine thread)
        self.mm_store: Dict[int, dict] = {}
        self._mm_next = 1

    def register_embeds(self, ids, emb: torch.Tensor, positions3=None, delta: int = 0, deepstack: Optional[dict] = None) -> int:
        """Park a multimodal prompt (placeholder ids, embedding rows with the media spliced in, optional 3-D positions,
        decode offset and deepstack levels); the returned key goes into ``GenerationRequest.embeds_key``."""
        if emb.shape[0] != len(ids):
            raise ValueError("one embedding row per prompt token is needed")
        key = self._mm_next
        self._mm_next += 1
        self.mm_store[key] = {"emb": emb, "pos3": positions3, "delta": int(delta or 0),
                              "deepstack": {int(k): (torch.as_tensor(r, dtype=torch.int64), f) for k, (r, f) in (deepstack or {}).items()}}
        return key

    def _prefix_seed(self, req) -> int:
        """Start of a request's block-hash chain: 0 for the base model, else a hash of the adapter's name and load
        generation (``BlockKeyExtras.adapter`` in ``cpp/runtime/state/contextCache/blockHash.h``).  K/V written under
        one adapter (LoRA wraps the QKV projection) is never adopted by the base model or by another adapter, and
        an adapter reloaded under the same name starts a new chain."""
        name = getattr(req, "lora_name", "") or ""
        epoch = int(getattr(self.runner, "weights_epoch", 0))       # bumped by a refit: K/V of the old weights is never adopted
        if not name:
            return int(rt.PrefixCache.extras_seed("", epoch, "weights")) if epoch else 0
        lora = getattr(self.runner, "lora", None)
        gen = lora.generation(name) if lora is not None and hasattr(lora, "generation") else 0
        return int(rt.PrefixCache.extras_seed(name, int(gen), f"weights{epoch}" if epoch else ""))

    # ---- seam ------------------------------------------------------------------------------------
    def capabilities(self):
        c = rt.SessionCapabilities()
        c.compact = True
        c.max_batch_size = self.kv.max_seats
        c.max_input_length = self.max_input_len
        c.kv_page_size = self.kv.page_size
        c.max_kv_tokens = self.kv.max_pages_per_seq * self.kv.page_size
        return c

    def admit(self, request_id, req):
        r = rt.AdmissionResult()
        n = len(req.prompt_ids)
        need = n + req.max_tokens
        if n > self.max_input_len or need > self.kv.max_pages_per_seq * self.kv.page_size:
            r.admitted, r.retry_later, r.reason = False, False, "EDGELLM_INPUT_TOO_LONG: prompt + max_tokens exceed the KV capacity"
            return r
        row_state = None
        plain = True
        if self.spec is not None:
            # sampled, constrained or opted-out requests are decoded token by token next to the speculative ones
            plain = bool(req.disable_spec_decode or req.temperature >= 1e-3 or req.guided_type or req.logit_bias_ids or req.num_logprobs >= 0)
            if not plain:
                need += self.spec.spec.verify_tokens + 8       # head room of one verification tree
        if req.guided_type or req.logit_bias_ids or req.num_logprobs >= 0:
            try:
                if req.guided_type and self.runner.vocab_map is not None:
                    raise ValueError("guided decoding is not combined with a reduced vocabulary")
                row_state = lp.make_row_state(
                    self.guided_vocab, guided=lp.guided_from_wire(req.guided_type, req.guided_spec),
                    logit_bias=dict(zip(req.logit_bias_ids, req.logit_bias_values)) or None,
                    num_logprobs=req.num_logprobs if req.num_logprobs >= 0 else None, vocab_size=self.runner.model.cfg.vocab_size)
            except ValueError as e:
                r.admitted, r.retry_later, r.reason = False, False, f"EDGELLM_BAD_REQUEST: {e}"
                return r
        mm = None
        if req.embeds_key:
            mm = self.mm_store.get(int(req.embeds_key))
            if mm is None or mm["emb"].shape[0] != n:
                r.admitted, r.retry_later, r.reason = False, False, "EDGELLM_BAD_REQUEST: unknown or mismatched multimodal prompt key"
                return r
        slot = self.slots.acquire()
        if slot < 0:
            r.admitted, r.retry_later, r.reason = False, True, "no free seat"
            return r
        reused = 0
        looked_up = None                  # prompt ids when the prefix cache was consulted: follower ranks repeat the lookup
        try:
            if self.prefix is not None and req.cache_lookup and mm is None:      # placeholder ids say nothing about the media
                looked_up = list(req.prompt_ids)
                seed = self._prefix_seed(req)
                m = self.prefix.lookup(list(req.prompt_ids), seed)
                pages, tokens = list(m.pages), m.tokens
                if tokens and self.hybrid:
                    pages, tokens = self._restore_snapshot(slot, req.prompt_ids, pages, seed)
                if tokens:
                    self.kv.adopt_prefix(slot, pages, tokens)
                    reused = tokens
            if self.kv.bounded_swa:
                # pages are taken step by step and handed back as the window moves on; admission keeps the sum of the
                # residents' worst-case live pages inside the pool, so a later step cannot run out
                if (len(self.seqs) + 1) * self._swa_bound > self.kv.pool.shape[1]:
                    raise MemoryError("sliding-window page budget is taken")
            else:
                self.kv.reserve(slot, need)               # capacity is reserved at seat time: no eviction later
                if self.mirror is not None:
                    # followers repeat lookup → adopt → reserve on their own page table and prefix index (same operations in
                    # the same order keep their state identical to this rank's)
                    self.mirror.send(("admit", slot, looked_up, need, True, self._prefix_seed(req)) if self.prefix is not None
                                     else ("reserve", slot, need))
        except (MemoryError, RuntimeError) as e:
            self.kv.free(slot)
            self.slots.release(slot)
            if self.mirror is not None and self.prefix is not None:
                self.mirror.send(("admit", slot, looked_up, need, False, self._prefix_seed(req)))
            if self.prefix is not None and self.prefix.evict(8):
                r.admitted, r.retry_later, r.reason = False, True, "KV pool full (evicted cached prefixes)"
            else:
                r.admitted, r.retry_later, r.reason = False, True, f"KV pool full: {e}"
            return r
        self.seqs[slot] = _Seq(req, request_id)
        self.seqs[slot].row_state = row_state
        self.seqs[slot].plain = plain
        if mm is not None:
            self.seqs[slot].mm = mm
            self.seqs[slot].plain = True              # on a speculative deployment media prompts decode token by token
            self.mm_store.pop(int(req.embeds_key), None)
        r.admitted, r.slot, r.reused_tokens = True, slot, reused
        return r

    def execute(self, plan):
        with prof.time_stage(prof.IFB_EXECUTE, batch=len(plan.seqs), tokens=plan.total_tokens):
            return self._execute(plan)

    # ---- hybrid prefix snapshots ---------------------------------------------------------------
    def _chain_hashes(self, tokens, n_pages: int, seed: int = 0):
        p, h, out = self.kv.page_size, seed, []
        for i in range(n_pages):
            h = rt.PrefixCache.hash_block(h, list(tokens[i * p:(i + 1) * p]))
            out.append(h)
        return out

    def _restore_snapshot(self, slot: int, prompt_ids, pages, seed: int = 0):
        """Longest page prefix of ``pages`` that also has a recurrent snapshot: its rows go into the seat's state."""
        hashes = self._chain_hashes(prompt_ids, len(pages), seed)
        for k in range(len(pages), 0, -1):
            snap = self.snapshots.get(hashes[k - 1])
            if snap is not None:
                self.snapshots.move_to_end(hashes[k - 1])
                self.kv.recurrent.restore([slot], snap)
                self.snapshot_hits += 1
                return pages[:k], k * self.kv.page_size
        return [], 0

    def _take_snapshot(self, slot: int, q, upto_tokens: int) -> None:
        h = self._chain_hashes(q.req.prompt_ids, upto_tokens // self.kv.page_size, self._prefix_seed(q.req))[-1]
        if h in self.snapshots:
            self.snapshots.move_to_end(h)
            return
        self.snapshots[h] = self.kv.recurrent.snapshot([slot])
        while len(self.snapshots) > self.max_snapshots:
            self.snapshots.popitem(last=False)

    def _execute(self, plan):
        seqs = list(plan.seqs)                            # the binding hands out copies: edit and use this one list
        if self.spec is not None:
            fast = [s for s in seqs if not self.seqs[s.slot].plain]
            slow = [s for s in seqs if self.seqs[s.slot].plain]
            out = self._execute_speculative(fast) if fast else rt.StepResult()
            if slow:
                out.deltas = list(out.deltas) + list(self._execute_plan(slow).deltas)
            return out
        if self.hybrid and self.prefix is not None:
            self._prefill_to_page_boundary(seqs)
        return self._execute_plan(seqs)

    def _prefill_to_page_boundary(self, seqs) -> None:
        """A prompt's last chunk is cut at the last page boundary: the part before it runs first, the recurrent rows
        there are saved for later requests with the same prefix, and the plan keeps only the rest."""
        p = self.kv.page_size
        head_seats, head_tokens, cut = [], [], []
        for s in seqs:
            if s.kind != rt.WorkKind.Context:
                continue
            q = self.seqs[s.slot]
            end = s.start + s.length
            boundary = end // p * p
            if s.last_chunk and s.start < boundary < end:
                head_seats.append(s.slot)
                head_tokens.append(q.tokens[s.start:boundary])
                cut.append((s, boundary))
            elif not s.last_chunk and end % p == 0:
                cut.append((s, None))                     # ends on a boundary by itself: snapshot after the main step
        if head_seats:
            self.runner.step(head_seats, head_tokens)
        self._snap_after = []
        for s, boundary in cut:
            if boundary is None:
                self._snap_after.append((s.slot, s.start + s.length))
            else:
                self._take_snapshot(s.slot, self.seqs[s.slot], boundary)
                s.length -= boundary - s.start
                s.start = boundary

    def _execute_speculative(self, seqs):
        ctx = [s for s in seqs if s.kind == rt.WorkKind.Context]
        dec = [s for s in seqs if s.kind != rt.WorkKind.Context]
        deltas = []

        def emit(slot, tokens):
            q = self.seqs[slot]
            d = rt.TokenDelta()
            d.slot = slot
            keep = []
            for t in tokens[:max(q.req.max_tokens - q.generated, 0)]:
                keep.append(int(t))
                if not q.req.ignore_eos and (t in self.eos or t in q.req.stop_token_ids):
                    d.finished = True
                    d.reason = rt.FinishReason.EndId if t in self.eos else rt.FinishReason.StopWords
                    break
            q.generated += len(keep)
            q.tokens += keep
            if keep:
                q.last_token = keep[-1]
            d.tokens = keep
            deltas.append(d)
        if ctx:
            for s in ctx:
                if s.start != 0 or not s.last_chunk:
                    raise RuntimeError("speculative decoding prefills whole prompts: raise max_chunk_tokens to the longest prompt")
            slots = [s.slot for s in ctx]
            first = self.spec.prefill(slots, [self.seqs[x].tokens[:] for x in slots])
            for slot, t in zip(slots, first):
                emit(slot, [t])
        if dec:
            slots = [s.slot for s in dec]
            for slot, toks in zip(slots, self.spec.round(slots)):
                emit(slot, toks)
        out = rt.StepResult()
        out.deltas = deltas
        return out

    def _execute_plan(self, seqs):
        seats, token_lists, producers = [], [], []
        for s in seqs:
            q = self.seqs[s.slot]
            if s.kind == rt.WorkKind.Context:
                toks = q.tokens[s.start:s.start + s.length]
                produces = s.last_chunk
            else:
                toks = q.feed or [q.last_token]
                q.feed = []
                produces = True
            if self.kv.bounded_swa:
                self.kv.reserve(s.slot, self.kv.lengths[s.slot] + len(toks))
            seats.append(s.slot)
            token_lists.append(toks)
            producers.append(produces)
        lora = getattr(self.runner, "lora", None)
        if lora is not None:                               # requests of one step may use different adapters
            segs, r0 = [], 0
            for slot, toks in zip(seats, token_lists):
                segs.append((r0, r0 + len(toks), self.seqs[slot].req.lora_name or None))
                r0 += len(toks)
            lora.set_segments(segs)
        graph_tokens = None
        if self._graph_step_ok(seqs, seats, token_lists):
            # every row is a plain greedy decode row: the step replays the captured graph of this batch size, and while the
            # same sequences keep decoding the step state never leaves the device (ModelRunner.decode_step_graph)
            if self.mirror is not None:
                self.mirror.send(("decode_graph", seats, [t[0] for t in token_lists]))
            graph_tokens = self.runner.decode_step_graph(seats, [t[0] for t in token_lists])
            self.graph_steps += 1
            logits = None
        elif any(s.kind == rt.WorkKind.Context and self.seqs[s.slot].mm is not None for s in seqs):
            logits = self._step_with_embeds(seqs, seats, token_lists)          # mirrors itself (rows travel with the plan)
        else:
            if self.mirror is not None:
                self.mirror.send(("step", seats, token_lists))
            logits = self.runner.step(seats, token_lists)      # one row per sequence (its last token)
        rows = [i for i, p in enumerate(producers) if p]
        out = rt.StepResult()
        deltas = []
        if rows:
            row_seqs = [self.seqs[seats[i]] for i in rows]
            states = [q.row_state for q in row_seqs]
            special = any(st is not None for st in states)
            if graph_tokens is not None:
                new = graph_tokens
            else:
                sel = logits[rows] if len(rows) != logits.shape[0] else logits
                if special:
                    sel = lp.process(sel, states)
                new = self._sample(sel, row_seqs)
            if special:
                reports = lp.logprobs(sel, new, states)
                constraint_done = lp.advance(states, new)
            for j, (i, tok) in enumerate(zip(rows, new)):
                q = self.seqs[seats[i]]
                q.generated += 1
                q.last_token = tok
                q.tokens.append(tok)
                d = rt.TokenDelta()
                d.slot, d.tokens = seats[i], [tok]
                if special and reports[j] is not None:
                    rep = rt.TokenLogprobs()
                    rep.chosen, rep.top_ids, rep.top_values = reports[j].chosen, reports[j].top_ids[0], reports[j].top_values[0]
                    d.logprobs = rep
                if special and constraint_done[j]:
                    d.tokens = []                        # the end-of-sequence token that closes a constraint is not output
                    d.finished, d.reason = True, rt.FinishReason.EndId
                elif not q.req.ignore_eos and (tok in self.eos or tok in q.req.stop_token_ids):
                    d.finished = True
                    d.reason = rt.FinishReason.EndId if tok in self.eos else rt.FinishReason.StopWords
                elif (special and states[j] is not None and getattr(states[j].guided, "jump_forward", False)
                      and states[j].num_logprobs < 0):       # a log-probability report has one row per sampled token
                    # jump-forward (cpp/runtime/decoding/jumpForward.cpp): tokens the grammar forces next are emitted with
                    # the sampled one and fed together in the sequence's next decode row (one row of several tokens)
                    extra = states[j].guided.forced_tokens(self.guided_vocab.tokenizer, q.req.max_tokens - q.generated)
                    if extra:
                        d.tokens = [tok] + extra
                        q.feed = [tok] + extra
                        q.tokens += extra
                        q.generated += len(extra)
                        q.last_token = extra[-1]
                        self.jump_forward_tokens += len(extra)
                deltas.append(d)
        for slot, upto in getattr(self, "_snap_after", []):
            self._take_snapshot(slot, self.seqs[slot], upto)
        self._snap_after = []
        # a finished prefill publishes its full prompt pages for reuse
        if self.prefix is not None:
            for s in seqs:
                if s.kind == rt.WorkKind.Context and s.last_chunk:
                    q = self.seqs[s.slot]
                    if q.req.cache_commit >= 1 and q.mm is None:      # placeholder ids of media prompts must not be shared
                        seed = self._prefix_seed(q.req)
                        if self.mirror is not None:
                            self.mirror.send(("prefix_insert", s.slot, list(q.req.prompt_ids), len(q.req.prompt_ids), seed))
                        self.prefix.insert(list(q.req.prompt_ids), len(q.req.prompt_ids), self.kv.pages_of(s.slot), seed)
        out.deltas = deltas
        return out

    def _graph_step_ok(self, seqs, seats, token_lists) -> bool:
        """A step may replay the decode graph when all of its rows are ordinary greedy decode rows: no prompt chunk, no
        multi-token row (jump-forward), no logits processing (bias, constraint, log-probabilities), no adapter routing, no
        multimodal position offset, sampling off.  Everything else runs the eager ragged step."""
        if not self.runner.can_graph_step(seats) or getattr(self.runner, "lora", None) is not None:
            return False
        for s, toks in zip(seqs, token_lists):
            q = self.seqs[s.slot]
            if (s.kind == rt.WorkKind.Context or len(toks) != 1 or q.row_state is not None or q.mm is not None
                    or q.req.temperature >= 1e-3):
                return False
        return True

    def _step_with_embeds(self, seqs, seats, token_lists) -> torch.Tensor:
        """A step that holds a prompt chunk of a multimodal request: every row is fed as an embedding row — media rows from
        the request's prepared prompt, all other rows (text prompts, decode rows) through the token table."""
        embeds, pos3, deep = [], [], {}
        row0 = 0
        for s, toks in zip(seqs, token_lists):
            q = self.seqs[s.slot]
            if q.mm is not None and s.kind == rt.WorkKind.Context:
                lo, hi = s.start, s.start + s.length
                embeds.append(q.mm["emb"][lo:hi])
                pos3.append(None if q.mm["pos3"] is None else q.mm["pos3"][:, lo:hi])
                for k, (rows, feats) in q.mm["deepstack"].items():
                    sel = (rows >= lo) & (rows < hi)
                    if bool(sel.any()):
                        acc = deep.setdefault(k, ([], []))
                        acc[0].append(rows[sel] - lo + row0)
                        acc[1].append(feats[sel.to(feats.device)])
            else:
                embeds.append(self.runner.embed_tokens(toks))
                pos3.append(None)
            row0 += len(toks)
        deepstack = {k: (torch.cat(r), torch.cat(f)) for k, (r, f) in deep.items()} or None
        deltas = [(s.slot, self.seqs[s.slot].mm["delta"]) for s in seqs
                  if self.seqs[s.slot].mm is not None and s.kind == rt.WorkKind.Context and s.last_chunk]
        if self.mirror is not None:                  # follower ranks replay the step with the same rows
            host = lambda t: None if t is None else t.detach().to("cpu")
            self.mirror.send(("step_embeds", seats, [host(e) for e in embeds], [host(p) for p in pos3],
                              None if deepstack is None else {k: (host(r), host(f)) for k, (r, f) in deepstack.items()}, deltas))
        logits = self.runner.step_embeds(seats, embeds, pos3, deepstack)
        for slot, d in deltas:
            self.runner.rope_delta[slot] = d         # decode rows continue after the largest media position
        return logits

    def release(self, slot):
        if slot in self.seqs:
            q = self.seqs[slot]
            if self.prefix is not None and q.req.cache_commit >= 2 and not self.hybrid and q.mm is None:
                # "including generated tokens": the full pages of prompt + output become reusable (a follow-up turn that
                # quotes the answer starts from them); hybrid models publish prompts only, their snapshots end there
                filled = min(self.kv.lengths[slot], len(q.tokens))
                if filled > len(q.req.prompt_ids):
                    seed = self._prefix_seed(q.req)
                    if self.mirror is not None:
                        self.mirror.send(("prefix_insert", slot, list(q.tokens[:filled]), filled, seed))
                    self.prefix.insert(list(q.tokens[:filled]), filled, self.kv.pages_of(slot), seed)
            del self.seqs[slot]
            if self.spec is not None:
                self.spec.release([slot])
            if self.mirror is not None:
                self.mirror.send(("release", slot))
            self.kv.free(slot)
            self.slots.release(slot)

    # ---- sampling --------------------------------------------------------------------------------
    def _sample(self, logits: torch.Tensor, seqs: List[_Seq]) -> List[int]:
        if all(q.req.temperature < 1e-3 for q in seqs):
            return [int(t) for t in self.runner.pick(logits).tolist()]
        n = logits.shape[0]
        dev = logits.device
        temp = torch.tensor([q.req.temperature for q in seqs], device=dev)
        topk = torch.tensor([q.req.top_k for q in seqs], device=dev, dtype=torch.int32)
        topp = torch.tensor([q.req.top_p for q in seqs], device=dev)
        # the uniform depends on (seed, request, step) only, so batching never changes a request's draws
        u = torch.tensor([rt.request_stable_uniform(q.req.seed, q.request_id, q.generated) for q in seqs], device=dev)
        return [int(t) for t in self.runner.to_full_vocab(ops.sample(logits, temp, topk, topp, u)).tolist()]
