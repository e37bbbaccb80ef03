"""DFlash speculative decoding: a block draft proposes ``block - 1`` tokens per round, the target verifies them as a chain.

Round for one sequence whose target cache holds ``n`` tokens and whose last accepted token ``y0`` is not in it yet::

    draft   : block [y0, mask × (B-1)] at positions n .. n+B-1 over the draft cache (context rows 0 .. n-1) → d1 .. d(B-1)
    target  : causal pass over [y0, d1 .. d(B-1)] with tapped hidden states → its own next token after every row
    accept  : the longest prefix of d that equals the target's choices, plus the target's token after it (a+1 tokens)
    commit  : target cache advances by a+1 rows (y0, d1 .. da); their tapped hidden states become a+1 new context rows
              of the draft cache; the next round's y0 is the bonus token

Greedy requests get exactly the target's greedy continuation; sampled requests are verified by rejection sampling along
the chain (static batches), so every token is distributed as the target's own sample.  Parity: ``cpp/runtime/decoding/dflashDecoder.cpp`` (round
structure, delta lengths, block layout) with the draft of ``models/dflash.py``.  Hybrid targets are
not supported (a partly accepted chain would need the recurrent state rolled back)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from .. import profiling as prof
from ..ops.meta import build_step_meta
from .block_diffusion import full_mask
from .kv_cache import KVCacheManager
from .speculative import default_tap_layers


@dataclass
class DFlashStats:
    rounds: int = 0
    emitted: int = 0
    draft_forwards: int = 0

    @property
    def mean_accept_length(self) -> float:
        return self.emitted / max(self.rounds, 1)


@dataclass
class _Headroom:
    verify_tokens: int


class DFlashDecoder:
    name = "dflash"
    is_speculative = True

    def __init__(self, runner, draft, draft_kv: KVCacheManager, block_size: Optional[int] = None, mask_token_id: Optional[int] = None,
                 tree_top_k: int = 1, verify_tokens: int = 0):
        """``tree_top_k > 1`` switches greedy requests from one chain per round to a verification tree: the ``tree_top_k``
        most likely tokens of every block position are candidates, and the ``verify_tokens`` best prefixes (root included)
        are verified in one target pass (``cpp/runtime/decoding/dsparkDecoder.cpp`` / ``dflashDecoder`` tree mode over
        ``ddtreeBuild``)."""
        self.r, self.model, self.draft, self.dkv = runner, runner.model, draft, draft_kv
        if getattr(self.model.cfg, "is_hybrid", False):
            raise ValueError("DFlash decoding is not available for hybrid (recurrent-state) targets")
        self.device = runner.device
        self.block = int(block_size or draft.cfg.dflash_block_size)
        self.mask_id = int(draft.cfg.dflash_mask_token_id if mask_token_id is None else mask_token_id)
        if not 2 <= self.block <= 64:
            raise ValueError("DFlash block size must be between 2 and 64")
        n = self.model.cfg.num_hidden_layers
        self.taps = list(draft.cfg.dflash_target_layer_ids) or default_tap_layers(n)
        if draft.embed_tokens is None:
            draft.share_with(self.model)
        self.stats = DFlashStats()
        self.spec = _Headroom(self.block)          # what the request engine's session reads for KV head room
        self.sampling: Optional[dict] = None       # {"temperature", "top_k", "top_p", "seed"}: rejection-sampled verification
        self._sample_gen: Optional[torch.Generator] = None
        self.root: Dict[int, int] = {}
        self._mask_cache: Dict[int, torch.Tensor] = {}
        self.tree_top_k = int(tree_top_k)
        if not 1 <= self.tree_top_k <= 8:
            raise ValueError("tree_top_k must be in 1..8")
        if self.tree_top_k > 1 and hasattr(draft, "propose_tokens"):
            raise ValueError("tree verification needs a draft that returns per-position logits (this one proposes tokens itself)")
        # every depth offers tree_top_k children per node, so the candidate tree holds k + k² + … nodes: never ask for more
        possible = sum(min(self.tree_top_k ** d, 4096) for d in range(1, self.block))
        self.verify_tokens = min(int(verify_tokens or 2 * self.block), 1 + possible, 64) if self.tree_top_k > 1 else 0
        if self.tree_top_k > 1:
            self.spec = _Headroom(max(self.block, self.verify_tokens))

    def kv_headroom(self) -> int:
        return max(self.block, self.verify_tokens)

    # ---- steps --------------------------------------------------------------------------------
    def _target_step(self, seats, rows: torch.Tensor, q_lens, tree_mask=None, positions=None):
        meta = self.r._meta(seats, q_lens, logits_all=True, tree_mask=tree_mask, positions=positions)
        uniq = sorted(set(self.taps))
        x, taps = self.model.hidden_states(rows, meta, self.r.cache, capture_layers=uniq)
        by_layer = dict(zip(uniq, taps))
        return self.model.logits_from_hidden(x, meta), torch.cat([by_layer[t] for t in self.taps], dim=-1)

    def _write_context(self, seats, feats: torch.Tensor, q_lens) -> None:
        past = [self.dkv.lengths[s] for s in seats]
        for s, q, p in zip(seats, q_lens, past):
            self.dkv.reserve(s, p + q + self.block)
        meta = build_step_meta(q_lens, past, self.dkv.table_rows(seats), self.dkv.page_size, slot_ids=seats, device=self.device)
        self.draft.write_context(feats, meta, self.dkv.pool)
        for s, q in zip(seats, q_lens):
            self.dkv.commit(s, q)

    def _propose(self, seats, want_logits: bool = False) -> torch.Tensor:
        """Draft tokens ``[N, block - 1]`` after each sequence's current root (``want_logits``: the block's logits
        ``[N, block, V]`` instead, on the device)."""
        n, b = len(seats), self.block
        ids = torch.full((n, b), self.mask_id, dtype=torch.int32)
        ids[:, 0] = torch.tensor([self.root[s] for s in seats], dtype=torch.int32)
        embeds = ops.embedding(ids.reshape(-1).to(self.device), self.draft.embed_tokens.weight)
        scale = getattr(self.model.model, "embed_scale", 1.0)
        if scale != 1.0:
            embeds = (embeds * torch.tensor(scale, dtype=embeds.dtype)).to(embeds.dtype)
        past = [self.dkv.lengths[s] for s in seats]
        causal = bool(self.draft.cfg.dflash_query_causal)          # JetSpec drafts: each block row sees the rows before it only
        if not causal and n not in self._mask_cache:
            self._mask_cache[n] = full_mask(n * b, b, self.device)
        meta = build_step_meta([b] * n, past, self.dkv.table_rows(seats), self.dkv.page_size, slot_ids=seats, logits_all=True,
                               device=self.device, tree_mask=None if causal else self._mask_cache[n])
        self.stats.draft_forwards += 1
        if hasattr(self.draft, "propose_tokens"):                        # Domino: proposals corrected by what precedes them
            return self.draft.propose_tokens(embeds, meta, self.dkv.pool, ids[:, 0].to(self.device), b).to("cpu")
        logits = self.draft.propose(embeds, meta, self.dkv.pool)        # block rows are written past the context, never committed
        if want_logits:
            return logits.view(n, b, -1)
        return ops.argmax(logits).view(n, b)[:, 1:].to("cpu")

    # ---- prefill / round -----------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, seats: Sequence[int], prompts: Sequence[Sequence[int]]) -> List[int]:
        q_lens = [len(p) for p in prompts]
        flat = torch.tensor([t for p in prompts for t in p], dtype=torch.int32, device=self.device)
        with prof.time_stage(prof.PREFILL, batch=len(seats), tokens=int(flat.numel())):
            logits, feats = self._target_step(seats, flat, q_lens)
            for s, q in zip(seats, q_lens):
                self.r.kv.commit(s, q)
                self.dkv.free(s)
            ends = torch.tensor(q_lens).cumsum(0) - 1
            last = logits.index_select(0, ends.to(self.device))
            if self.sampling is None:
                first = ops.argmax(last).tolist()
            else:                                   # sampled request: the first token is a draw from the target distribution too
                pr = ops.ref.sampling_probs(last, self.sampling["temperature"], self.sampling["top_k"], self.sampling["top_p"])
                u = self._uniforms(len(seats), 1, 1)[:, 0, 0].to(pr.device)
                first = torch.searchsorted(pr.double().cumsum(-1), u.double()[:, None]).clamp(max=pr.shape[-1] - 1)[:, 0].tolist()
            self._write_context(seats, feats, q_lens)
        for s, t in zip(seats, first):
            self.root[s] = int(t)
        return [int(t) for t in first]

    @torch.no_grad()
    def round(self, seats: Sequence[int], forced_accept: Optional[Sequence[int]] = None) -> List[List[int]]:
        """One draft → verify round; returns the new tokens of every sequence (accepted drafts + the target's next token).
        ``forced_accept`` prescribes the accepted draft count per sequence (benchmarks with random weights)."""
        n, b = len(seats), self.block
        if self.tree_top_k > 1 and self.sampling is None and forced_accept is None:
            return self._round_tree(seats)
        drafts = self._propose(seats)                                     # [N, B-1] host
        chain = torch.cat([torch.tensor([[self.root[s]] for s in seats], dtype=torch.int64), drafts.long()], dim=1)
        # a draft with a confidence head (DSpark) may shorten a sequence's proposal: the verification step is ragged then
        plens = getattr(self.draft, "last_proposal_lengths", None) if (self.sampling is None and forced_accept is None) else None
        q_lens = [b] * n if plens is None else [1 + max(1, min(b - 1, int(v))) for v in plens]
        starts = [0]
        for q in q_lens:
            starts.append(starts[-1] + q)
        rows = (chain.reshape(-1) if plens is None else torch.cat([chain[i, :q] for i, q in enumerate(q_lens)])).to(torch.int32).to(self.device)
        logits, feats = self._target_step(seats, rows, q_lens)            # rows written past the committed length, not committed yet
        sampled = None
        if self.sampling is not None and forced_accept is None:
            # the chain is a tree with one child per node: draft d is kept with the target's probability of d, a rejected
            # position is redrawn from the target distribution without d, which keeps every token distributed as the target's
            pr = ops.ref.sampling_probs(logits, self.sampling["temperature"], self.sampling["top_k"], self.sampling["top_p"]).view(n, b, -1)
            parents = torch.arange(-1, b - 1).repeat(n, 1)
            path, plen, bonus = ops.ref.spec_accept_sampling(pr.to("cpu"), chain, parents, b, self._uniforms(n, b, 2))
            sampled = ((plen - 1).tolist(), bonus.tolist())
            choice = None
        else:
            choice = ops.argmax(logits).to("cpu")                         # target's token after each chain row (flat over the ragged rows)
        out: List[List[int]] = []
        keep_rows, keep_lens = [], []
        for i, s in enumerate(seats):
            a = 0
            if sampled is not None:
                a = int(sampled[0][i])
                toks = [int(t) for t in drafts[i, :a]] + [int(sampled[1][i])]
            else:
                limit = q_lens[i] - 1 if forced_accept is None else min(int(forced_accept[i]), b - 1)
                while a < limit and (forced_accept is not None or int(drafts[i, a]) == int(choice[starts[i] + a])):
                    a += 1
                toks = [int(t) for t in drafts[i, :a]] + [int(choice[starts[i] + a])]
            out.append(toks)
            self.r.kv.commit(s, a + 1)                                    # y0 and the accepted drafts are real history now
            keep_rows.append(torch.arange(starts[i], starts[i] + a + 1))
            keep_lens.append(a + 1)
            self.root[s] = toks[-1]
        self._write_context(seats, feats.index_select(0, torch.cat(keep_rows).to(self.device)), keep_lens)
        self.stats.rounds += 1
        self.stats.emitted += sum(len(t) for t in out)
        return out

    @torch.no_grad()
    def _round_tree(self, seats: Sequence[int]) -> List[List[int]]:
        """One draft → tree → verify round for greedy requests.  The block's positions are predicted independently, so the
        candidates of a node depend on its depth only; the best ``verify_tokens - 1`` prefixes form the tree.  The target
        scores every node in one pass under the tree's ancestor mask; the accepted path is the longest one on which each
        node is the target's own choice after its parent, so the output equals plain greedy decoding."""
        n, b, nodes = len(seats), self.block, self.verify_tokens
        dev = self.device
        logits = self._propose(seats, want_logits=True)                    # [N, B, V]; row j + 1 predicts the token at depth j + 1
        ids, lp = ops.ddtree_candidates(logits[:, 1:], self.tree_top_k)
        root = torch.tensor([self.root[s] for s in seats], dtype=torch.int32, device=dev)
        tok, par, _, _, valid = ops.ddtree_assemble(ids, lp, root, nodes)
        if int(valid.min()) < nodes:
            raise RuntimeError("the candidate tree holds fewer nodes than verify_tokens")      # excluded by the constructor's cap
        past = torch.tensor([self.r.kv.lengths[s] for s in seats], dtype=torch.int32, device=dev)
        tmask, _, pos = ops.eagle_tree_meta(par, past, 0, 0)
        tlogits, feats = self._target_step(seats, tok.reshape(-1).to(torch.int32), [nodes] * n, tree_mask=tmask, positions=pos)
        choice = ops.argmax(tlogits).view(n, nodes).to(torch.int32)
        path, plen, bonus = ops.spec_accept_greedy(choice, tok.to(torch.int32), par.to(torch.int32), b, 0)
        # the accepted nodes' KV rows move to consecutive positions behind the committed history
        ops.kv_commit_path(self.r.kv.pool, self.r.kv.table_rows(seats).to(dev), past, path, plen)
        path_h, plen_h, bonus_h, tok_h = path.tolist(), plen.tolist(), bonus.tolist(), tok.tolist()
        out: List[List[int]] = []
        keep_rows, keep_lens = [], []
        for i, s in enumerate(seats):
            m = plen_h[i]
            kept = path_h[i][:m]
            out.append([tok_h[i][j] for j in kept[1:]] + [bonus_h[i]])
            self.r.kv.commit(s, m)
            keep_rows.extend(i * nodes + j for j in kept)
            keep_lens.append(m)
            self.root[s] = bonus_h[i]
        self._write_context(seats, feats.index_select(0, torch.tensor(keep_rows, device=dev)), keep_lens)
        self.stats.rounds += 1
        self.stats.emitted += sum(len(t) for t in out)
        return out

    @torch.no_grad()
    def generate(self, seats: Sequence[int], prompts: Sequence[Sequence[int]], max_new_tokens: int, eos_id: Optional[int] = None,
                 sampling=None) -> List[List[int]]:
        self.sampling, self._sample_gen = sampling, None
        for s in seats:
            self.r.kv.free(s)
        first = self.prefill(seats, prompts)
        out = [[t] for t in first]
        live = [i for i in range(len(seats)) if not (eos_id is not None and first[i] == eos_id) and max_new_tokens > 1]
        while live:
            cur = [seats[i] for i in live]
            room = min(self.r.kv.max_pages_per_seq * self.r.kv.page_size - self.r.kv.lengths[s] for s in cur)
            if room < self.block:
                break
            new = self.round(cur)
            nxt = []
            for i, toks in zip(live, new):
                for t in toks:
                    if len(out[i]) >= max_new_tokens:
                        break
                    out[i].append(t)
                    if eos_id is not None and t == eos_id:
                        break
                done = len(out[i]) >= max_new_tokens or (eos_id is not None and out[i][-1] == eos_id)
                if not done:
                    nxt.append(i)
            live = nxt
        return out

    def _uniforms(self, b: int, depth: int, width: int) -> torch.Tensor:
        if self._sample_gen is None:
            self._sample_gen = torch.Generator().manual_seed(int((self.sampling or {}).get("seed", 0)))
        return torch.rand(b, depth, width, generator=self._sample_gen)

    def release(self, seats: Sequence[int]) -> None:
        for s in seats:
            self.r.kv.free(s)
            self.dkv.free(s)
            self.root.pop(s, None)
            if hasattr(self.draft, "forget"):            # per-seat draft state (LiLiCorr's anchor row)
                self.draft.forget(s)
