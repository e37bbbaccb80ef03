"""Ragged, token-major step metadata shared by every op and by the runtime.

One step executes ``N`` sequences whose new tokens are packed back to back in ``T`` rows.  A
prefill chunk contributes ``q_len > 1`` rows, a decode row contributes one, and a
speculative-verify step contributes a small tree of rows per sequence.  Persistent state
(paged KV, recurrent state rows) is addressed through ``page_table`` / ``slot_ids`` and never
moves.

Parity: the ragged plugin ABI of the reference (``docs/source/developer_guide/customization/
tensorrt-plugins.md:41-74``; ``cpp/runtime/exec/raggedBatchBuilder.h``).  Here it is a plain
dataclass of tensors instead of engine bindings.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch


@dataclass
class StepMeta:
    q_start: torch.Tensor        # int32 [N+1] first row of each sequence
    q_len: torch.Tensor          # int32 [N]   rows this step
    past_len: torch.Tensor       # int32 [N]   tokens already in the KV cache
    positions: torch.Tensor      # int32 [T]   RoPE position of each row
    seq_ids: torch.Tensor        # int32 [T]   owning sequence of each row
    page_table: torch.Tensor     # int32 [N, max_pages] physical page of each logical page, -1 unused
    slot_ids: torch.Tensor       # int32 [N]   row in the resident state pools
    logits_idx: torch.Tensor     # int32 [L]   rows whose logits are wanted
    page_size: int
    num_seqs: int
    num_tokens: int
    max_q_len: int
    max_seq_len: int
    # Speculative verification: row r of a sequence may attend to new row c of the same sequence
    # iff bit c of tree_mask[r] is set (int32 words, [T, ceil(max_q_len/32)]).  None = causal.
    tree_mask: Optional[torch.Tensor] = None
    # KV slot of each row relative to past_len (None = row index within the sequence).
    kv_offsets: Optional[torch.Tensor] = None
    # Multimodal RoPE: temporal / height / width position of each row, int32 [3, T].  The model turns them into
    # per-row cos / sin rows (`rope_rows` [T, D], looked up with `rope_pos` = 0..T-1) before its layers run.
    # Deepstack (Qwen3-VL): {layer index: (row indices int64 [M], features [M, H])} — vision features of intermediate
    # encoder levels that are added to the hidden state of the image rows after the given decoder layers.
    deepstack: Optional[dict] = None
    positions3: Optional[torch.Tensor] = None
    rope_rows: Optional[torch.Tensor] = None
    rope_pos: Optional[torch.Tensor] = None
    # Skip-softmax: fp32 [N] log2(lambda) per sequence (lambda = S / sequence length from the deployed scale table; -inf where
    # the sequence is shorter than the first calibrated length), or None when the deployment runs dense.
    skip_thr: Optional[torch.Tensor] = None

    @property
    def is_decode(self) -> bool:
        return self.max_q_len == 1

    def to(self, device) -> "StepMeta":
        kw = {}
        for k, v in self.__dict__.items():
            if isinstance(v, dict):
                v = {kk: tuple(t.to(device, non_blocking=True) for t in vv) for kk, vv in v.items()}
            kw[k] = v.to(device, non_blocking=True) if isinstance(v, torch.Tensor) else v
        return StepMeta(**kw)


def build_step_meta(q_lens: Sequence[int], past_lens: Sequence[int], page_table: torch.Tensor,
                    page_size: int, slot_ids: Optional[Sequence[int]] = None,
                    logits_all: bool = False, device="cpu",
                    positions: Optional[Sequence[int]] = None,
                    tree_mask: Optional[torch.Tensor] = None) -> StepMeta:
    """Host-side construction of a :class:`StepMeta` (the Python twin of the native builder)."""
    n = len(q_lens)
    q_start = [0]
    for q in q_lens:
        q_start.append(q_start[-1] + int(q))
    t = q_start[-1]
    pos: List[int] = []
    sid: List[int] = []
    for i, (q, p) in enumerate(zip(q_lens, past_lens)):
        pos.extend(range(int(p), int(p) + int(q)))
        sid.extend([i] * int(q))
    pos_t = None
    if isinstance(positions, torch.Tensor):          # already on the device (tree steps): no host copy of the values
        pos_t = positions.to(device=device, dtype=torch.int32).reshape(-1)
    elif positions is not None:
        pos = [int(x) for x in positions]
    if logits_all:
        lidx = list(range(t))
    else:
        lidx = [q_start[i + 1] - 1 for i in range(n)]
    i32 = dict(dtype=torch.int32, device=device)
    return StepMeta(
        q_start=torch.tensor(q_start, **i32), q_len=torch.tensor(list(q_lens), **i32),
        past_len=torch.tensor(list(past_lens), **i32), positions=pos_t if pos_t is not None else torch.tensor(pos, **i32),
        seq_ids=torch.tensor(sid, **i32), page_table=page_table.to(device=device, dtype=torch.int32),
        slot_ids=torch.tensor(list(slot_ids) if slot_ids is not None else list(range(n)), **i32),
        logits_idx=torch.tensor(lidx, **i32), page_size=page_size, num_seqs=n, num_tokens=t,
        max_q_len=max(q_lens) if n else 0,
        max_seq_len=max((int(q) + int(p) for q, p in zip(q_lens, past_lens)), default=0),
        tree_mask=tree_mask.to(device) if tree_mask is not None else None)
