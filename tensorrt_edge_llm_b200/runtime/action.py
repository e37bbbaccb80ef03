"""Action generation for vision-language-action deployments: flow-matching rollout of the action expert over the
language model's KV cache, plus the trajectory-history tokeniser of the prompt side.

``ActionRunner.sample(seats)`` — for sequences whose prompt (camera frames, trajectory history, reasoning) is already in
the language model's cache — starts from Gaussian noise ``[B, T, 2]`` and takes ``num_steps`` Euler steps of the expert's
flow from t = 0 to t = 1.  Every step is one ragged engine step: the ``T`` waypoint rows of a sequence are written behind
its committed context (never committed, so the next step and any later decode overwrite them) and attend to the whole
context and to one another.

Parity: ``cpp/action/alpamayo1ActionRunner.cpp`` (ten denoise steps, t0 = i / N, t1 = (i + 1) / N, :558-561),
``cpp/action/actionUtils.cpp:27`` (``trajectoryToTokenIds``), ``cpp/action/actionKvBatch.*`` (the expert reads the
language model's per-layer KV; here it reads the same page pool through the same page table)."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from .. import profiling as prof
from .block_diffusion import full_mask

DEFAULT_DENOISE_STEPS = 10
EGO_MIN = (-4.0, -4.0, -10.0)
EGO_MAX = (4.0, 4.0, 10.0)


def trajectory_to_token_ids(history: Sequence[Tuple[float, float, float]], num_traj_tokens: int, traj_token_start: int) -> List[int]:
    """Past ego positions → prompt tokens: the first point as it is, every later one as the step from its predecessor, each
    coordinate clamped to the ego range, quantised to ``num_traj_tokens`` levels and offset by ``traj_token_start``."""
    out: List[int] = []
    prev = None
    for pt in history:
        cur = tuple(float(v) for v in pt)
        rel = cur if prev is None else tuple(c - p for c, p in zip(cur, prev))
        prev = cur
        for v, lo, hi in zip(rel, EGO_MIN, EGO_MAX):
            level = int(round((v - lo) / (hi - lo) * (num_traj_tokens - 1)))
            out.append(min(max(level, 0), num_traj_tokens - 1) + traj_token_start)
    return out


class ActionRunner:
    def __init__(self, runner, expert, num_steps: int = DEFAULT_DENOISE_STEPS):
        self.r, self.expert = runner, expert
        tc, ec = runner.model.cfg, expert.cfg
        if (ec.num_hidden_layers, ec.num_key_value_heads, ec.head_dim) != (tc.num_hidden_layers, tc.num_key_value_heads // max(tc.tp_size, 1)
                                                                           * max(tc.tp_size, 1), tc.head_dim):
            raise ValueError("the action expert must match the language model's layer count, KV heads and head dimension "
                             f"(expert {ec.num_hidden_layers}/{ec.num_key_value_heads}/{ec.head_dim}, "
                             f"model {tc.num_hidden_layers}/{tc.num_key_value_heads}/{tc.head_dim})")
        if getattr(tc, "is_hybrid", False):
            raise ValueError("the action expert reads attention KV of every layer: hybrid language models are not supported")
        self.num_steps = int(num_steps)
        self.tokens = expert.action_cfg.n_diffusion_tokens
        self._masks = {}

    def kv_headroom(self) -> int:
        return self.tokens

    @torch.no_grad()
    def sample(self, seats: Sequence[int], seed: int = 0, noise: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Trajectories ``[B, T, 2]`` (fp32: acceleration, curvature per waypoint) for the sequences on ``seats``."""
        r, b, t = self.r, len(seats), self.tokens
        dev = r.device
        if noise is None:
            noise = torch.randn(b, t, 2, generator=torch.Generator().manual_seed(int(seed)))
        x = noise.to(dev, torch.float32)
        if b not in self._masks:
            self._masks[b] = full_mask(b * t, t, dev)
        # waypoint rows take the positions right after the context (text-like positions: all rotary components move together)
        positions = [r.kv.lengths[s] + r.rope_delta.get(s, 0) + j for s in seats for j in range(t)]
        with prof.time_stage("action_denoise", batch=b, tokens=b * t * self.num_steps):
            for i in range(self.num_steps):
                t0, t1 = i / self.num_steps, (i + 1) / self.num_steps
                meta = r._meta(seats, [t] * b, tree_mask=self._masks[b], positions=positions)     # reserves, never commits
                v = self.expert.velocity(x, torch.full((b,), t0, device=dev), meta, r.cache)
                x = x + (t1 - t0) * v.float()
        return x.to("cpu")
