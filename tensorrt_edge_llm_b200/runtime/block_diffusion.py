"""Block-diffusion decoding: generate ``canvas_length`` tokens at a time by denoising a canvas.

One block::

    canvas ← uniform random ids                       (init_canvas)
    for step in 0 .. steps-1:
        T       = t_min + (t_max - t_min) · (steps - step) / steps
        inputs  = self_condition(E[canvas], soft)     (soft = 0 on the first pass)
        logits  = backbone(inputs)                    every canvas row sees the history and the whole canvas; KV not committed
        soft    = softmax(logits / T) @ E             (expected embedding, next pass's conditioning)
        sampled, argmax, entropy = sample(logits / T) (Gumbel-max draw, arg-max and entropy of every row)
        update_canvas: keep the sampled ids of the lowest-entropy rows within the entropy budget, re-noise the others,
                       track per-row arg-max stability; a row set has converged when all arg-maxes were stable for more
                       than `stability_window` passes and the mean entropy is below `entropy_threshold`;
                       the last pass accepts the arg-max of every row
    commit: the arg-max canvas (cut at an end token and at the request's budget) runs through the backbone once more with the
            ordinary causal mask, which writes the KV entries later blocks attend to

The passes use the engine's own kernels: the canvas pass is a ragged step whose tree mask has every bit set (the
speculative-verify attention path with a full mask is bidirectional attention over the new rows), the commit pass is an
ordinary prefill chunk.  Sampling, the entropy budget and the canvas bookkeeping are torch ops over ``[rows, vocab]`` and
``[batch, canvas]`` tensors.

Parity: ``cpp/runtime/decoding/blockDiffusionDecoder.cpp`` (``decodeStep`` :538, ``denoiseTemperature`` :349,
``sampleCanvasEntropyBound`` :383) and ``cpp/sampler/diffusionGemma/diffusionGemmaSampling.cu`` (sample + entropy :247,
``initializeDiffusionCanvasKernel`` :325, ``diffusionSampleAndUpdateCanvasKernel`` :344).  A block whose rows have all
converged ends its passes early here: converged rows are no longer updated, so the remaining passes cannot change the
committed tokens."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch

from .. import profiling as prof
from ..config import DiffusionConfig

DEFAULT_SEED = 42
DEFAULT_RUNTIME_STEPS = 48


# ---- sampler ----------------------------------------------------------------------------------

def sample_rows(logits: torch.Tensor, temperature: float, generator: Optional[torch.Generator]
                ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per row of ``logits [R, V]``: a draw from ``softmax(logits / T)`` (Gumbel-max), the arg-max and the entropy (nats)."""
    z = logits.float() / max(float(temperature), 1e-6)
    logp = torch.log_softmax(z, dim=-1)
    entropy = -(logp.exp() * logp).nan_to_num(0.0).sum(-1)
    argmax = z.argmax(-1)
    on_device = generator is None or generator.device.type == z.device.type
    u = torch.rand(z.shape, generator=generator, device=z.device if on_device else "cpu").to(z.device).clamp_(1e-20, 1.0 - 1e-7)
    sampled = (z - torch.log(-torch.log(u))).argmax(-1)
    return sampled, argmax, entropy


def entropy_budget(entropy: torch.Tensor, valid_len: torch.Tensor, bound: float) -> torch.Tensor:
    """Rows of ``entropy [B, C]`` kept by the entropy-bound policy, as a bool mask.

    Positions are visited from the most to the least certain; position k is kept while the entropy of everything kept so
    far, not counting the largest (the candidate itself), stays within ``bound``.  The most certain position is always kept;
    a negative bound keeps nothing."""
    b, c = entropy.shape
    cols = torch.arange(c, device=entropy.device)[None, :]
    valid = cols < valid_len[:, None]
    if bound < 0:
        return torch.zeros_like(valid)
    key = torch.where(valid & torch.isfinite(entropy), entropy, torch.full_like(entropy, float("inf")))
    order = torch.argsort(key, dim=1, stable=True)
    sorted_e = torch.gather(key, 1, order).clamp_min(0.0)
    finite = torch.isfinite(sorted_e)
    e = torch.where(finite, sorted_e, torch.zeros_like(sorted_e))
    before = torch.cumsum(e, 1) - e                                   # entropy of the positions kept earlier
    keep_sorted = finite & (before <= bound)
    keep_sorted = torch.cumprod(keep_sorted.to(torch.int32), 1).bool()   # stop at the first position over budget
    keep = torch.zeros_like(valid)
    keep.scatter_(1, order, keep_sorted)
    return keep & valid


@dataclass
class CanvasState:
    canvas: torch.Tensor          # int64 [B, C]  ids the next pass reads
    argmax: torch.Tensor          # int64 [B, C]  arg-max ids of the latest pass (what a commit takes)
    previous: torch.Tensor        # int64 [B, C]  arg-max ids of the pass before
    stable: torch.Tensor          # int32 [B, C]  consecutive passes with the same arg-max, this one included
    accepted: torch.Tensor        # bool  [B, C]  rows inside the entropy budget in the latest pass
    prefix: torch.Tensor          # int32 [B]     converged length (0 or the row's valid length); sticky


def init_canvas(batch: int, canvas_len: int, vocab: int, generator: Optional[torch.Generator], device) -> CanvasState:
    ids = torch.randint(0, vocab, (batch, canvas_len), generator=generator).to(device)
    z = lambda dt: torch.zeros(batch, canvas_len, dtype=dt, device=device)
    return CanvasState(ids, z(torch.int64), torch.full((batch, canvas_len), -1, dtype=torch.int64, device=device), z(torch.int32),
                       z(torch.bool), torch.zeros(batch, dtype=torch.int32, device=device))


def update_canvas(st: CanvasState, sampled: torch.Tensor, argmax: torch.Tensor, entropy: torch.Tensor, valid_len: torch.Tensor,
                  cfg: DiffusionConfig, vocab: int, force_accept: bool, generator: Optional[torch.Generator]) -> None:
    """Entropy-bound acceptance, re-noising and convergence tracking for one pass (in place)."""
    b, c = st.canvas.shape
    sampled, argmax, entropy = sampled.view(b, c), argmax.view(b, c), entropy.view(b, c)
    cols = torch.arange(c, device=st.canvas.device)[None, :]
    valid_len = valid_len.clamp(1, c)
    valid = cols < valid_len[:, None]
    live = (st.prefix < valid_len)[:, None]                          # converged rows are left alone
    upd = valid & live
    if force_accept:
        st.previous = torch.where(upd, argmax, st.previous)
        st.stable = torch.where(upd, torch.full_like(st.stable, cfg.stability_window + 1), st.stable)
        st.argmax = torch.where(upd, argmax, st.argmax)
        st.canvas = torch.where(upd, argmax, st.canvas)
        st.accepted = torch.where(live, valid, st.accepted)
        st.prefix = torch.where(live[:, 0], valid_len.to(torch.int32), st.prefix)
        return
    keep = entropy_budget(entropy, valid_len, cfg.entropy_bound)
    same = argmax == st.previous
    stable = torch.where(same, st.stable + 1, torch.ones_like(st.stable))
    token_stable = (stable > cfg.stability_window) if cfg.stability_window > 0 else torch.ones_like(same)
    noise = torch.randint(0, vocab, (b, c), generator=generator).to(st.canvas.device)
    st.previous = torch.where(upd, argmax, st.previous)
    st.stable = torch.where(upd, stable, st.stable)
    st.argmax = torch.where(upd, argmax, st.argmax)
    st.accepted = torch.where(live, keep, st.accepted)
    nxt = torch.where(keep, sampled, noise)
    e = torch.where(torch.isfinite(entropy), entropy.clamp_min(0.0), torch.full_like(entropy, 3.0e35))
    mean_e = (e * valid).sum(1) / valid_len
    converged = (token_stable | ~valid).all(1) & (mean_e < cfg.entropy_threshold) & live[:, 0]
    nxt = torch.where(converged[:, None], argmax, nxt)
    st.canvas = torch.where(upd, nxt, st.canvas)
    st.prefix = torch.where(converged, valid_len.to(torch.int32), st.prefix)


def denoise_temperature(cfg: DiffusionConfig, step: int, steps: int) -> float:
    if steps <= 0:
        return cfg.t_min
    step = min(max(step, 0), steps - 1)
    return cfg.t_min + (cfg.t_max - cfg.t_min) * (steps - step) / steps


def full_mask(rows: int, canvas_len: int, device) -> torch.Tensor:
    """Tree mask ``[rows, ceil(C / 32)]`` with the low ``C`` bits of every row set: each canvas row attends to all of them."""
    words = (canvas_len + 31) // 32
    m = torch.full((rows, words), -1, dtype=torch.int32)
    tail = canvas_len % 32
    if tail:
        last = (1 << tail) - 1
        m[:, -1] = last - (1 << 32) if last >= (1 << 31) else last
    return m.to(device)


# ---- decoder ----------------------------------------------------------------------------------

@dataclass
class DiffusionStats:
    blocks: int = 0
    denoise_passes: int = 0
    commit_passes: int = 0
    emitted: int = 0
    passes_per_block: List[int] = field(default_factory=list)


class BlockDiffusionDecoder:
    """Drives a :class:`~tensorrt_edge_llm_b200.models.diffusion_gemma.DiffusionGemmaLM` through prefill, denoise and
    commit passes.  Every generated token is in the KV cache when ``generate`` returns (there is no pending last token)."""

    name = "block_diffusion"
    is_speculative = False

    def __init__(self, runner, cfg: Optional[DiffusionConfig] = None, seed: int = DEFAULT_SEED):
        self.runner = runner
        self.model = runner.model
        self.cfg = cfg or self.model.cfg.diffusion or DiffusionConfig()
        if self.cfg.sampler_type != "entropy_bound":
            raise ValueError(f"block-diffusion sampler {self.cfg.sampler_type!r} is not supported (entropy_bound is)")
        if runner.vocab_map is not None:
            raise ValueError("block diffusion needs the full LM head: self-conditioning mixes embeddings of every token")
        self.vocab = self.model.cfg.vocab_size
        self.seed = seed
        self.stats = DiffusionStats()

    def kv_headroom(self) -> int:
        """Extra KV slots a sequence needs beyond its committed tokens: every pass writes a whole canvas."""
        return self.cfg.canvas_length

    def effective_steps(self, requested: int = 0) -> int:
        if requested <= 0:
            return min(self.cfg.max_denoising_steps, DEFAULT_RUNTIME_STEPS)
        return min(max(requested, 1), self.cfg.max_denoising_steps)

    # ---- one block ----------------------------------------------------------------------------
    @torch.no_grad()
    def denoise_block(self, seats: Sequence[int], canvas_len: int, steps: int, generator, row_generator=None
                      ) -> Tuple[torch.Tensor, int]:
        """Denoise one canvas for ``seats``; returns the arg-max canvas ``[B, C]`` (host) and the passes run.
        ``generator`` (host) draws the canvas noise, ``row_generator`` (on the logits' device) the per-row Gumbel noise."""
        r, dev, b = self.runner, self.runner.device, len(seats)
        row_generator = row_generator or generator
        st = init_canvas(b, canvas_len, self.vocab, generator, dev)
        valid = torch.full((b,), canvas_len, dtype=torch.int64, device=dev)
        mask = full_mask(b * canvas_len, canvas_len, dev)
        soft = None
        passes = 0
        for step in range(steps):
            temp = denoise_temperature(self.cfg, step, steps)
            with prof.time_stage("block_diffusion_denoise", batch=b, tokens=b * canvas_len):
                x = self.model.canvas_inputs(st.canvas.reshape(-1), soft)
                meta = r._meta(seats, [canvas_len] * b, logits_all=True, tree_mask=mask)
                logits = self.model(None, meta, r.cache, inputs_embeds=x.to(self.model.cfg.compute_dtype))
            passes += 1
            force = step + 1 >= steps
            if force:
                argmax = logits.float().argmax(-1)
                update_canvas(st, argmax, argmax, torch.zeros(argmax.shape, device=dev), valid, self.cfg, self.vocab, True, generator)
                break
            if self.model.self_conditioning is not None:
                soft = self.model.soft_embeddings(logits, temp)
            sampled, argmax, entropy = sample_rows(logits, temp, row_generator)
            update_canvas(st, sampled, argmax, entropy, valid, self.cfg, self.vocab, False, generator)
            if bool((st.prefix >= valid).all()):
                break
        return st.argmax.to("cpu"), passes

    # ---- whole requests -----------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, seats: Sequence[int], prompts: Sequence[Sequence[int]], max_tokens: int, eos_ids: Sequence[int] = (),
                 max_denoising_steps: int = 0, seed: Optional[int] = None, should_stop=None) -> List[List[int]]:
        """Generate up to ``max_tokens`` per prompt.  ``should_stop(i, tokens_so_far)`` (optional) ends request ``i`` after
        the token just appended (stop strings); ``eos_ids`` end it after an end token, which stays in the output."""
        r, kv = self.runner, self.runner.kv
        n = len(seats)
        seed = self.seed if seed is None else int(seed)
        gen = torch.Generator(device="cpu").manual_seed(seed)
        row_gen = torch.Generator(device=r.device).manual_seed(seed + 1) if r.device.type == "cuda" else gen
        eos = set(int(e) for e in eos_ids)
        steps = self.effective_steps(max_denoising_steps)
        for s in seats:
            kv.free(s)
        r.prefill(list(seats), [list(map(int, p)) for p in prompts])       # history is fully committed; its logits are not used
        out: List[List[int]] = [[] for _ in range(n)]
        live = list(range(n))
        while live:
            live = [i for i in live if len(out[i]) < max_tokens]
            if not live:
                break
            cur = [seats[i] for i in live]
            room = min(kv.max_pages_per_seq * kv.page_size - kv.lengths[s] for s in cur)
            if room <= 0:
                break
            canvas_len = max(1, min(self.cfg.canvas_length, room))
            # the canvas keeps its full length even when fewer tokens are wanted: a shorter canvas changes the
            # bidirectional distribution (the reference notes a bias towards an early end token)
            canvas, passes = self.denoise_block(cur, canvas_len, steps, gen, row_gen)
            self.stats.blocks += 1
            self.stats.denoise_passes += passes
            self.stats.passes_per_block.append(passes)
            commit: List[List[int]] = []
            done: List[int] = []
            for row, i in enumerate(live):
                take = min(canvas_len, max_tokens - len(out[i]))
                toks: List[int] = []
                for t in canvas[row, :take].tolist():
                    toks.append(int(t))
                    if int(t) in eos or (should_stop is not None and should_stop(i, out[i] + toks)):
                        done.append(i)
                        break
                commit.append(toks)
                out[i].extend(toks)
                self.stats.emitted += len(toks)
            with prof.time_stage("block_diffusion_commit", batch=len(cur), tokens=sum(len(c) for c in commit)):
                r.step(cur, commit)                                          # causal pass: writes the committed KV
            self.stats.commit_passes += 1
            live = [i for i in live if i not in done]
        return out
