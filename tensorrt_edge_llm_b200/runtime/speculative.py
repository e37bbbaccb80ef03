"""EAGLE-3 tree speculative decoding over the paged ragged step ABI.

One round per call of :meth:`EagleDecoder.round`:

1. grow a draft tree: the draft's distribution after the last accepted token gives the ``top_k``
   depth-1 candidates; ``draft_steps - 1`` draft forwards (tree-masked, one per depth) expand the
   ``top_k`` best frontier nodes into ``top_k²`` candidates scored by cumulative log-probability;
2. keep the ``verify_tokens - 1`` best candidates (closed under ancestors because scores fall
   along a path) plus the root and verify them with ONE tree-masked target forward;
3. accept greedily along the tree (kernel), compact the accepted path in the target's paged KV
   cache in place (kernel), and emit the accepted tokens plus the target's bonus token;
4. feed the accepted tokens with the target's tapped hidden states to the draft (its KV is
   rewound to the committed length first), which yields the next round's depth-1 candidates.

Greedy acceptance is lossless: the emitted stream equals plain greedy decoding of the target.

Parity: ``cpp/runtime/decoding/eagleDecoder.cpp`` — ``decodeStep`` (:287-320),
``constructDraftProposal`` (:502-729), ``runBaseModelVerification`` (:731-871),
``runDraftModelAcceptToken`` (:873-959), KV headroom (:223-238); tree size cap
``cpp/common/specDecodeLimits.h:30``; forced acceptance length for benchmarks
``cpp/runtime/config/runtimeBenchmarkOptions.h``.
"""
from __future__ import annotations

import weakref
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from .. import ops
from .. import profiling as prof
from ..ops.meta import build_step_meta
from .kv_cache import KVCacheManager
from .runner import ModelRunner


@dataclass
class SpecConfig:
    draft_steps: int = 4          # tree depth
    top_k: int = 8                # children kept per node and frontier width
    verify_tokens: int = 32       # tree nodes verified per round, root included (<= 128)
    force_accept_len: int = 0     # benchmark mode: nodes accepted per round (root included), tokens ignored
    force_accept_mean: float = 0.0  # benchmark mode: per-round lengths drawn from a seeded distribution with this mean
    force_seed: int = 0
    block_tree_top_k: int = 1     # block drafts (DFlash): > 1 verifies a tree of that many candidates per position instead of one chain

    def __post_init__(self):
        if not 1 <= self.block_tree_top_k <= 8:
            raise ValueError("block_tree_top_k must be in 1..8")
        if not 1 <= self.verify_tokens <= 128:
            raise ValueError("verify_tokens must be in 1..128")
        if self.draft_steps < 1 or self.top_k < 1:
            raise ValueError("draft_steps and top_k must be positive")
        pool = self.top_k + (self.draft_steps - 1) * self.top_k * self.top_k
        self.verify_tokens = min(self.verify_tokens, pool + 1)


@dataclass
class SpecStats:
    rounds: int = 0
    emitted: int = 0
    draft_forwards: int = 0
    replays: int = 0                 # hybrid targets: sequences whose recurrent state was restored and replayed
    recurrent_replays: int = 0       # ... of which from recorded kernel inputs (recurrent kernels only, no second model pass)

    @property
    def mean_accept_length(self) -> float:
        return self.emitted / max(self.rounds, 1)


def default_tap_layers(num_layers: int) -> List[int]:
    """Low / middle / high target layers whose hidden states feed the draft (EAGLE-3 convention)."""
    ids = sorted({min(max(i, 0), num_layers - 1) for i in (2, num_layers // 2, num_layers - 3)})
    while len(ids) < 3:                      # very shallow test models: reuse the last layer
        ids.append(ids[-1])
    return ids


def _dense_pick(draft, lp, k):
    """Proposals of a draft without a ``pick`` of its own: top-k of a dense log-probability row, mapped through ``d2t``."""
    sc, idx = lp.topk(min(k, lp.shape[-1]), dim=-1)
    return sc, draft.d2t.long()[idx]


class _VerifyGraph:
    """One captured tree-verification pass of the target for a fixed (batch, tree size): token ids, positions, ancestor
    mask, cache lengths and page-table rows live in static device buffers that are refilled before every replay (the first
    three by device-to-device copies from the tree kernels' outputs, so the tree never visits the host)."""

    def __init__(self, dec: "EagleDecoder", b: int, nn: int):
        from ..ops.meta import StepMeta
        r = dec.r
        dev, kv = r.device, r.kv
        i32 = dict(dtype=torch.int32, device=dev)
        t = b * nn
        self._dec = weakref.ref(dec)              # the decoder owns this object: no reference cycle through it
        self.b, self.nn = b, nn
        self.ids = torch.zeros(t, **i32)
        self.meta = StepMeta(
            q_start=torch.arange(0, t + 1, nn, **i32), q_len=torch.full((b,), nn, **i32), past_len=torch.zeros(b, **i32),
            positions=torch.zeros(t, **i32), seq_ids=torch.arange(b, **i32).repeat_interleave(nn),
            page_table=torch.full((b, kv.max_pages_per_seq), -1, **i32), slot_ids=torch.zeros(b, **i32),
            logits_idx=torch.arange(t, **i32), page_size=kv.page_size, num_seqs=b, num_tokens=t, max_q_len=nn,
            max_seq_len=kv.max_pages_per_seq * kv.page_size, tree_mask=torch.zeros(t, (nn + 31) // 32, **i32))
        self._pin = torch.empty(b * (kv.max_pages_per_seq + 2), dtype=torch.int32, pin_memory=True)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.tgt = self.taps = None
        self.launches = 0

    @property
    def dec(self) -> "EagleDecoder":
        d = self._dec()
        if d is None:
            raise RuntimeError("the decoder of this verification graph is gone")
        return d

    def _body(self):
        dec = self.dec
        uniq = sorted(set(dec.taps))
        x, taps = dec.model.hidden_states(self.ids, self.meta, dec.r.cache, capture_layers=uniq)
        by_layer = dict(zip(uniq, taps))
        return dec.model.greedy_from_hidden(x, self.meta), torch.cat([by_layer[t] for t in dec.taps], dim=-1)

    def _load(self, seats, tree_tok, positions, mask):
        kv, b = self.dec.r.kv, self.b
        host = self._pin
        host[:b] = torch.tensor([kv.lengths[s] for s in seats], dtype=torch.int32)
        host[b:2 * b] = torch.tensor(list(seats), dtype=torch.int32)
        host[2 * b:] = kv.table_rows(seats).reshape(-1)
        devbuf = host.to(self.dec.device, non_blocking=True)
        m = self.meta
        m.past_len.copy_(devbuf[:b])
        m.slot_ids.copy_(devbuf[b:2 * b])
        m.page_table.copy_(devbuf[2 * b:].view(b, -1))
        self.ids.copy_(tree_tok.reshape(-1))
        m.positions.copy_(positions.reshape(-1))
        m.tree_mask.copy_(mask)

    def run(self, seats, tree_tok, positions, mask):
        from ..ops import cuda as cu
        kv = self.dec.r.kv
        for s in seats:
            kv.reserve(s, kv.lengths[s] + self.nn)
        self._load(seats, tree_tok, positions, mask)
        if self.graph is None:
            side = torch.cuda.Stream(device=self.dec.device)           # one eager pass first: lazy set-up, allocator warm-up
            side.wait_stream(torch.cuda.current_stream(self.dec.device))
            with torch.cuda.stream(side):
                self._body()
            torch.cuda.current_stream(self.dec.device).wait_stream(side)
            before = cu.LAUNCHES
            g = torch.cuda.CUDAGraph()
            from .runner import capture_guard
            with capture_guard(), torch.cuda.graph(g, capture_error_mode="thread_local"):
                self.tgt, self.taps = self._body()
            self.graph = g
            self.launches = cu.LAUNCHES - before
            cu.LAUNCHES = before
        self.graph.replay()
        cu.LAUNCHES += self.launches
        return self.tgt, self.taps


class EagleDecoder:
    def __init__(self, runner: ModelRunner, draft, draft_kv: KVCacheManager, spec: Optional[SpecConfig] = None,
                 tap_layers: Optional[Sequence[int]] = None):
        spec = spec or SpecConfig()
        # Recurrent layers cannot evaluate a branching tree in one pass: hybrid targets verify a chain (top-k 1) with
        # the causal mask, and a partly accepted chain is undone by restoring the state rows saved before the
        # verification and replaying only the accepted tokens.
        self.hybrid = bool(runner.model.cfg.is_hybrid)
        if self.hybrid and spec.top_k != 1:
            raise ValueError("a hybrid (Mamba / DeltaNet) target verifies a draft chain: set top_k = 1")
        self.r = runner
        self.model = runner.model
        self.draft = draft
        self.dkv = draft_kv
        self.spec = spec or SpecConfig()
        if tap_layers is None and getattr(draft.cfg, "draft_type", None) == "mtp":
            tap_layers = [runner.model.cfg.num_hidden_layers - 1]       # an MTP head reads the target's last hidden state
        self.taps = list(tap_layers or runner.model.cfg.eagle3_target_layer_ids or default_tap_layers(runner.model.cfg.num_hidden_layers))
        self.device = runner.device
        self.stats = SpecStats()
        self._force_gen = None
        self.sampling: Optional[dict] = None       # {"temperature", "top_k", "top_p", "seed"} for sampled requests, None = greedy
        self._sample_gen = None
        # per seat: pending root token, draft log-probs and hidden after the last accepted token
        self._verify_graphs: Dict[tuple, _VerifyGraph] = {}
        self.root: Dict[int, int] = {}
        self.lp: Dict[int, torch.Tensor] = {}
        self.hid: Dict[int, torch.Tensor] = {}

    # ---- helpers ------------------------------------------------------------------------------
    def _embed(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(ids.to(torch.int32), self.model.model.embed_tokens.weight)

    def _target_step(self, seats, rows: torch.Tensor, q_lens, tree_mask=None, positions=None, greedy=False):
        """Target pass over ``rows`` with the tapped layers; returns ``(logits, taps)``, or ``(arg-max ids, taps)`` when
        ``greedy`` (a vocabulary-sharded head then exchanges one candidate per row and rank instead of the logits)."""
        meta = self.r._meta(seats, q_lens, logits_all=True, tree_mask=tree_mask, positions=positions)
        uniq = sorted(set(self.taps))
        x, taps = self.model.hidden_states(rows, meta, self.r.cache, capture_layers=uniq)
        if greedy and hasattr(self.model, "greedy_from_hidden"):
            logits = self.model.greedy_from_hidden(x, meta)
        else:
            logits = self.model.logits_from_hidden(x, meta)
            if greedy:
                logits = ops.argmax(logits)
        by_layer = dict(zip(uniq, taps))
        return logits, torch.cat([by_layer[t] for t in self.taps], dim=-1)

    def _draft_step(self, seats, embeds, feature, q_lens, logits_rows, tree_mask=None, positions=None, commit=False):
        past = [self.dkv.lengths[s] for s in seats]
        for s, q, p in zip(seats, q_lens, past):
            self.dkv.reserve(s, p + q)
        meta = build_step_meta(q_lens, past, self.dkv.table_rows(seats), self.dkv.page_size, slot_ids=seats, logits_all=True,
                               device=self.device, tree_mask=tree_mask, positions=positions)
        meta.logits_idx = torch.as_tensor(logits_rows, dtype=torch.int32, device=self.device)
        lp, h = self.draft(embeds, feature, meta, self.dkv.pool)
        if commit:
            for s, q in zip(seats, q_lens):
                self.dkv.commit(s, q)
        self.stats.draft_forwards += 1
        return lp, h

    # ---- prefill ------------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, seats: Sequence[int], prompts: Sequence[Sequence[int]]) -> List[int]:
        """Target prefill with tapped hidden states, then draft prefill.  Returns the first generated
        token of every sequence (the root of its first tree)."""
        q_lens = [len(p) for p in prompts]
        flat = torch.tensor([t for p in prompts for t in p], dtype=torch.int32, device=self.device)
        logits, taps = self._target_step(seats, flat, q_lens)
        for s, q in zip(seats, q_lens):
            self.r.kv.commit(s, q)
        ends = torch.tensor(q_lens).cumsum(0) - 1
        last = logits.index_select(0, ends.to(self.device))
        if self.sampling is None:
            first = ops.argmax(last).tolist()
        else:                                   # sampled request: the first token is a draw from the target distribution too
            pr = ops.ref.sampling_probs(last, self.sampling["temperature"], self.sampling["top_k"], self.sampling["top_p"])
            u = self._uniforms(len(seats), 1, 1)[:, 0, 0].to(pr.device)
            first = torch.searchsorted(pr.double().cumsum(-1), u.double()[:, None]).clamp(max=pr.shape[-1] - 1)[:, 0].tolist()
        # draft row i pairs the target feature of position i with the token of position i + 1
        nxt = flat.clone()
        nxt[:-1] = flat[1:]
        nxt[ends.to(self.device)] = torch.tensor(first, dtype=torch.int32, device=self.device)
        lp, h = self._draft_step(seats, self._embed(nxt), taps, q_lens, ends.tolist(), commit=True)
        for i, s in enumerate(seats):
            self.root[s] = int(first[i])
            self.lp[s] = lp[i]
            self.hid[s] = h[int(ends[i])]
        return [int(t) for t in first]

    def _graph_verify_ok(self, greedy: bool) -> bool:
        """Tree verification replays from a CUDA graph on the GPU for greedy requests of attention-only targets (recurrent
        layers need the state snapshot / replay around the pass); ``EDGELLM_DISABLE_CUDA_GRAPH=1`` or ``use_verify_graph =
        False`` keep the eager pass."""
        import os
        return (greedy and not self.hybrid and self.device.type == "cuda" and getattr(self, "use_verify_graph", True)
                and hasattr(self.model, "greedy_from_hidden") and os.environ.get("EDGELLM_DISABLE_CUDA_GRAPH", "0") != "1"
                and self.r.rope_delta_empty())

    # ---- one speculative round ----------------------------------------------------------------
    @torch.no_grad()
    def round(self, seats: Sequence[int]) -> List[List[int]]:
        """Returns the tokens emitted for every seat in one draft-verify pass (accepted draft tokens + bonus)."""
        sp, dev = self.spec, self.device
        b, k, steps, n = len(seats), self.spec.top_k, self.spec.draft_steps, self.spec.verify_tokens
        timer = prof.timer()
        stage = timer.begin(prof.SPEC_DRAFT, batch=b)
        pick = getattr(self.draft, "pick", None) or (lambda lp_, k_: _dense_pick(self.draft, lp_, k_))
        lp0 = torch.stack([self.lp[s] for s in seats])                       # [B, Vd] (candidate heads: [B, 2, Kc])
        h0 = torch.stack([self.hid[s] for s in seats])                       # [B, H]
        sc, tok0 = pick(lp0, k)
        k1 = sc.shape[-1]
        # candidate pool (depth-ordered): token, parent pool index (-1 = root), depth, cumulative score
        p_tok, p_par, p_dep, p_sc = [tok0], [torch.full((b, k1), -1, device=dev)], [torch.ones(b, k1, dtype=torch.long, device=dev)], [sc]
        # draft rows fed so far: token, feature, parent row (-1 = none), depth, pool index
        r_tok, r_feat, r_par, r_dep = tok0, h0[:, None, :].expand(b, k1, h0.shape[-1]), torch.full((b, k1), -1, device=dev), torch.ones(b, k1, dtype=torch.long, device=dev)
        r_pool, r_sc = torch.arange(k1, device=dev).expand(b, k1), sc
        front0, kf = 0, k1                                                    # first row / width of the current frontier
        pool_base = k1
        ld = torch.tensor([self.dkv.lengths[s] for s in seats], dtype=torch.int32).to(dev, non_blocking=True)
        for depth in range(2, steps + 1):
            rows = r_tok.shape[1]
            # ancestor mask and RoPE positions of the draft rows, built on the device from the parent table
            mask, _, pos = ops.eagle_tree_meta(r_par, ld, 1, -1)
            want = [i * rows + front0 + j for i in range(b) for j in range(kf)]
            lp, h = self._draft_step(seats, self._embed(r_tok.reshape(-1)), r_feat.reshape(b * rows, -1).contiguous(), [rows] * b, want,
                                     tree_mask=mask, positions=pos)
            csc, ctok = pick(lp.reshape(b, kf, *lp.shape[1:]), k)             # [B, kf, kc]
            kc = csc.shape[-1]
            cum = r_sc[:, front0:front0 + kf, None] + csc
            cpar = r_pool[:, front0:front0 + kf, None].expand(b, kf, kc)
            p_tok.append(ctok.reshape(b, -1)); p_par.append(cpar.reshape(b, -1)); p_sc.append(cum.reshape(b, -1))
            p_dep.append(torch.full((b, kf * kc), depth, dtype=torch.long, device=dev))
            if depth == steps:
                break
            # next frontier: the best `k` of the new candidates
            kn = min(k, kf * kc)
            fsc, fsel = cum.reshape(b, -1).topk(kn, dim=-1)
            fpar_row = front0 + fsel // kc                                    # parent's draft row
            hrows = h.view(b, rows, -1)
            r_tok = torch.cat([r_tok, ctok.reshape(b, -1).gather(1, fsel)], dim=1)
            r_feat = torch.cat([r_feat, hrows.gather(1, fpar_row[..., None].expand(b, kn, hrows.shape[-1]))], dim=1)
            r_par = torch.cat([r_par, fpar_row], dim=1)
            r_dep = torch.cat([r_dep, torch.full((b, kn), depth, dtype=torch.long, device=dev)], dim=1)
            r_pool = torch.cat([r_pool, pool_base + fsel], dim=1)
            n_new = kf * kc
            r_sc = torch.cat([r_sc, fsc], dim=1)
            front0, kf = rows, kn
            pool_base += n_new
        p_tok, p_par, p_dep, p_sc = (torch.cat(x, dim=1) for x in (p_tok, p_par, p_dep, p_sc))
        timer.end(stage)
        stage = timer.begin(prof.SPEC_VERIFY, batch=b, tokens=b * n)
        # ---- choose the verification tree ----
        npool = p_tok.shape[1]
        keep = min(n - 1, npool)
        nn_ = keep + 1
        root = torch.tensor([self.root[s] for s in seats], dtype=torch.int32).to(dev, non_blocking=True)
        lt = [self.r.kv.lengths[s] for s in seats]
        lt_dev = torch.tensor(lt, dtype=torch.int32).to(dev, non_blocking=True)
        # best `keep` candidates in pool order behind the root, then the tree's mask and positions: two kernels, no host read
        tree_tok, tree_par, tree_dep = ops.eagle_select_verify(p_sc, p_tok, p_par, p_dep, root, keep)
        tmask, _, pos = ops.eagle_tree_meta(tree_par, lt_dev, 0, 0)
        state_before = self.r.kv.recurrent.snapshot(seats) if self.hybrid else None
        can_record = self.hybrid and hasattr(self.model, "replay_recurrent") and getattr(self, "use_recurrent_replay", True)
        if can_record:
            self.r.kv.recurrent.begin_record()          # the mixers keep their recurrent-kernel inputs of the verification pass
        greedy = self.sampling is None
        if self._graph_verify_ok(greedy):
            # fixed (batch, tree size) and a tree that already lives on the device: the whole target pass replays from a graph
            vg = self._verify_graphs.get((b, nn_))
            if vg is None:
                vg = self._verify_graphs[(b, nn_)] = _VerifyGraph(self, b, nn_)
            logits, taps = vg.run(seats, tree_tok, pos, tmask)
        else:
            logits, taps = self._target_step(seats, tree_tok.reshape(-1).to(torch.int32), [nn_] * b, tree_mask=None if self.hybrid else tmask,
                                             positions=None if self.hybrid else pos, greedy=greedy)
        tgt = logits.view(b, nn_) if greedy else None
        timer.end(stage)
        stage = timer.begin(prof.SPEC_ACCEPT, batch=b)
        # ---- accept, commit KV ----
        max_path = steps + 1
        if self.sampling is None:
            path, plen, bonus = ops.spec_accept_greedy(tgt, tree_tok.to(torch.int32), tree_par.to(torch.int32), max_path, self._forced(b))
        else:
            # lossless for sampled requests: sibling-by-sibling rejection against the target distribution of each node,
            # bonus token from the residual (see ops.reference.spec_accept_sampling)
            sm = self.sampling
            probs = ops.ref.sampling_probs(logits, sm["temperature"], sm["top_k"], sm["top_p"]).view(b, nn_, -1)
            path, plen, bonus = ops.spec_accept_sampling(probs, tree_tok.to(torch.int32), tree_par.to(torch.int32), max_path,
                                                          self._uniforms(b, max_path, k + 1))
            path, plen, bonus = path.to(dev), plen.to(dev), bonus.to(dev)
        past_t = lt_dev
        ops.kv_commit_path(self.r.kv.pool, self.r.kv.table_rows(seats).to(dev), past_t, path, plen)
        path_h, plen_h, bonus_h = path.tolist(), plen.tolist(), bonus.tolist()   # the round's one device→host read
        tok_h = tree_tok.tolist()
        if self.hybrid:
            # commit policy: the recurrent state now holds all nn_ chain tokens; seats that accepted fewer get their saved rows
            # back and the state is advanced over the accepted prefix again — from the recorded kernel inputs of the verification
            # pass (recurrent kernels only), or, without a record, by running the prefix through the model once more (KV rows
            # are rewritten with the same values)
            record = self.r.kv.recurrent.end_record() if can_record else None
            short = [i for i in range(b) if plen_h[i] < nn_]
            if short:
                self.r.kv.recurrent.restore(seats, state_before, short)
                sub = [seats[i] for i in short]
                meta = self.r._meta(sub, [plen_h[i] for i in short], logits_all=False)
                if record:
                    idx = torch.tensor([i * nn_ + j for i in short for j in range(plen_h[i])], dtype=torch.long, device=dev)
                    self.model.replay_recurrent(record, idx, meta, self.r.cache)
                    self.stats.recurrent_replays += len(short)
                else:
                    rows = torch.tensor([t for i in short for t in tok_h[i][:plen_h[i]]], dtype=torch.int32, device=dev)
                    self.model.hidden_states(rows, meta, self.r.cache)
                self.stats.replays += len(short)
        out: List[List[int]] = []
        acc_rows, acc_tok, q_lens = [], [], []
        for i, s in enumerate(seats):
            m = plen_h[i]
            self.r.kv.commit(s, m)
            nodes = path_h[i][:m]
            emitted = [tok_h[i][j] for j in nodes[1:]] + [bonus_h[i]]
            out.append(emitted)
            acc_rows.extend(i * nn_ + j for j in nodes)
            acc_tok.extend(emitted)
            q_lens.append(m)
            self.root[s] = bonus_h[i]
        # ---- draft catches up on the accepted tokens ----
        feat = taps.index_select(0, torch.tensor(acc_rows, device=dev))
        emb = self._embed(torch.tensor(acc_tok, dtype=torch.int32, device=dev))
        ends = (torch.tensor(q_lens).cumsum(0) - 1).tolist()
        lp, h = self._draft_step(seats, emb, feat, q_lens, ends, commit=True)
        for i, s in enumerate(seats):
            self.lp[s] = lp[i]
            self.hid[s] = h[ends[i]]
        timer.end(stage)
        self.stats.rounds += b
        self.stats.emitted += sum(len(e) for e in out)
        return out

    def _uniforms(self, b: int, depth: int, width: int) -> torch.Tensor:
        """Seeded uniforms of the sampled-acceptance path (one generator per decoder, advanced every call)."""
        if self._sample_gen is None:
            self._sample_gen = torch.Generator().manual_seed(int((self.sampling or {}).get("seed", 0)))
        return torch.rand(b, depth, width, generator=self._sample_gen)

    def _forced(self, b: int):
        """Forced accept lengths of the current draft-verify pass: a constant, or draws in ``1..draft_steps+1`` from a seeded
        distribution whose mean is ``force_accept_mean`` (random weights accept almost nothing, so
        benchmarks of the verify / rewind path prescribe the lengths)."""
        sp = self.spec
        if sp.force_accept_mean <= 0:
            return sp.force_accept_len
        if self._force_gen is None:
            self._force_gen = torch.Generator().manual_seed(sp.force_seed)
        hi = sp.draft_steps + 1
        # binomial on (hi - 1) trials shifted by one has mean 1 + (hi - 1) p
        p = min(max((sp.force_accept_mean - 1.0) / max(hi - 1, 1), 0.0), 1.0)
        draws = (torch.rand(b, hi - 1, generator=self._force_gen) < p).sum(-1) + 1
        return draws.to(torch.int32)

    @staticmethod
    def _ancestors(parents: torch.Tensor) -> torch.Tensor:
        """``[B, R, R]`` bool: row r may attend row c iff c is r or one of its ancestors."""
        return ops.ref.eagle_ancestors(parents)

    @staticmethod
    def _pack_mask(anc: torch.Tensor) -> torch.Tensor:
        """Pack ``[B, R, R]`` bool into int32 words ``[B·R, ceil(R/32)]`` (bit c of row r)."""
        return ops.ref.eagle_pack_mask(anc)

    # ---- whole-request driver -----------------------------------------------------------------
    @torch.no_grad()
    def generate(self, seats: Sequence[int], prompts: Sequence[Sequence[int]], max_new_tokens: int,
                 eos_token_id: Optional[int] = None, sampling: Optional[dict] = None) -> List[List[int]]:
        """``sampling`` = ``{"temperature", "top_k", "top_p", "seed"}`` switches the verification from greedy matching to
        rejection sampling; the emitted tokens are then distributed as plain sampling from the target would be."""
        self.sampling = dict(sampling) if sampling is not None and sampling.get("temperature", 0.0) >= 1e-3 else None
        self._sample_gen = None
        first = self.prefill(seats, prompts)
        outs = [[t] for t in first]
        active = [i for i in range(len(seats)) if not (eos_token_id is not None and first[i] == eos_token_id) and max_new_tokens > 1]
        while active:
            emitted = self.round([seats[i] for i in active])
            still = []
            for i, e in zip(active, emitted):
                for t in e:
                    if len(outs[i]) >= max_new_tokens:
                        break
                    outs[i].append(t)
                    if eos_token_id is not None and t == eos_token_id:
                        break
                done = len(outs[i]) >= max_new_tokens or (eos_token_id is not None and outs[i][-1] == eos_token_id)
                if not done:
                    still.append(i)
            active = still
        return outs

    def release(self, seats: Sequence[int]) -> None:
        for s in seats:
            self.r.kv.free(s)
            self.dkv.free(s)
            self.root.pop(s, None); self.lp.pop(s, None); self.hid.pop(s, None)
