"""Per-request logits processing shared by the static-batch path and the in-flight-batching session:
additive logit bias, guided-decoding token masks and log-probability reporting.

Order of operations follows the reference's decode step (``cpp/runtime/decoding/vanillaDecoder.cpp:304-404``:
logit bias → guided mask → sample → log-probabilities) with the limits of its sampler
(``cpp/sampler/sampling.h``: at most 50 alternatives per token)."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import ops

MAX_LOGPROBS = 50


@dataclass
class RowState:
    """What one request carries from step to step."""
    guided: Optional[object] = None                 # GuidedDecoder
    bias_ids: Optional[torch.Tensor] = None         # int64 [n]
    bias_values: Optional[torch.Tensor] = None      # fp32 [n]
    num_logprobs: int = -1                          # -1 off, 0 chosen token only, k alternatives as well

    @property
    def active(self) -> bool:
        return self.guided is not None or self.bias_ids is not None or self.num_logprobs >= 0


@dataclass
class StepLogprobs:
    chosen: List[float] = field(default_factory=list)
    top_ids: List[List[int]] = field(default_factory=list)
    top_values: List[List[float]] = field(default_factory=list)


class GuidedVocabulary:
    """Token texts of a tokenizer, built once (the per-token decode is the slow part of mask construction)."""

    def __init__(self, tokenizer, vocab_size: int, eos_ids: Sequence[int]):
        self.tokenizer, self.vocab_size, self.eos_ids = tokenizer, vocab_size, [int(e) for e in eos_ids if e is not None]
        self._texts = None

    @property
    def texts(self):
        if self._texts is None:
            from .guided import GuidedDecoder
            if self.tokenizer is None:
                raise ValueError("guided decoding needs a tokenizer (token texts)")
            self._texts = GuidedDecoder.vocabulary(self.tokenizer, self.vocab_size)
        return self._texts

    def decoder(self, params):
        from .guided import GuidedDecoder
        return GuidedDecoder(params, self.texts, self.eos_ids)


def make_row_state(vocab: Optional[GuidedVocabulary], *, guided=None, logit_bias: Optional[Dict[int, float]] = None,
                   num_logprobs: Optional[int] = None, vocab_size: int = 0) -> RowState:
    st = RowState()
    if guided is not None:
        if vocab is None:
            raise ValueError("guided decoding needs a tokenizer (token texts)")
        st.guided = vocab.decoder(guided)
    if logit_bias:
        ids = [int(k) for k in logit_bias]
        if vocab_size and any(i < 0 or i >= vocab_size for i in ids):
            raise ValueError("logit_bias names a token id outside the vocabulary")
        st.bias_ids = torch.tensor(ids, dtype=torch.int64)
        st.bias_values = torch.tensor([float(logit_bias[k]) for k in logit_bias], dtype=torch.float32).clamp(-100.0, 100.0)
    if num_logprobs is not None and num_logprobs >= 0:
        if num_logprobs > MAX_LOGPROBS:
            raise ValueError(f"at most {MAX_LOGPROBS} log-probabilities per token")
        st.num_logprobs = int(num_logprobs)
    return st


def guided_from_wire(kind: str, spec: str):
    """Rebuild constraint parameters from the two strings a native request carries."""
    from .guided import GuidedDecodingParams
    if not kind:
        return None
    d = json.loads(spec) if spec else {}
    return GuidedDecodingParams(kind, **d)


def guided_to_wire(params) -> Tuple[str, str]:
    if params is None:
        return "", ""
    return params.type, json.dumps({"choices": list(params.choices), "pattern": params.pattern, "json_schema": params.json_schema,
                                    "max_depth": params.max_depth, "grammar": params.grammar, "structural_tag": params.structural_tag, "jump_forward": params.jump_forward})


def process(logits: torch.Tensor, states: Sequence[Optional[RowState]]) -> torch.Tensor:
    """Bias and mask ``logits [n, V]`` row by row; rows without state pass through.  Returns fp32 when anything changed."""
    if not any(s is not None and (s.guided is not None or s.bias_ids is not None) for s in states):
        return logits
    out = logits.float().clone()
    dev = out.device
    for i, s in enumerate(states):
        if s is not None and s.bias_ids is not None:
            out[i].index_add_(0, s.bias_ids.to(dev), s.bias_values.to(dev))
    if any(s is not None and s.guided is not None for s in states):
        words = (out.shape[1] + 31) // 32
        mask = torch.full((len(states), words), -1, dtype=torch.int32)
        for i, s in enumerate(states):
            if s is not None and s.guided is not None:
                m = s.guided.bitmask()
                mask[i, :min(words, m.numel())] = m[:words]
        out = ops.apply_token_bitmask(out, mask.to(dev))
    return out


def logprobs(processed: torch.Tensor, tokens: Sequence[int], states: Sequence[Optional[RowState]]) -> List[Optional[StepLogprobs]]:
    """Log-probabilities of the sampled tokens (and the k most likely) under the processed distribution."""
    want = [i for i, s in enumerate(states) if s is not None and s.num_logprobs >= 0]
    res: List[Optional[StepLogprobs]] = [None] * len(states)
    if not want:
        return res
    tok = torch.tensor([int(tokens[i]) for i in want], dtype=torch.int64).to(processed.device)
    kmax = max(states[i].num_logprobs for i in want)
    rows = processed if len(want) == processed.shape[0] else processed[want]
    if kmax <= 32:                      # one kernel per step on the GPU: log-sum-exp, the chosen token, k ordered arg-max passes
        chosen_t, top_i_t, top_v_t = ops.token_logprobs(rows, tok, kmax)
    else:
        lp = torch.log_softmax(rows.float(), dim=-1)
        chosen_t = lp.gather(1, tok[:, None])[:, 0]
        top_v_t, top_i_t = lp.topk(kmax, dim=-1)
    chosen = chosen_t.tolist()
    top_v = top_v_t.tolist() if kmax > 0 else None
    top_i = top_i_t.tolist() if kmax > 0 else None
    for j, i in enumerate(want):
        k = states[i].num_logprobs
        res[i] = StepLogprobs([chosen[j]], [top_i[j][:k]] if k > 0 else [[]], [top_v[j][:k]] if k > 0 else [[]])
    return res


def advance(states: Sequence[Optional[RowState]], tokens: Sequence[int]) -> List[bool]:
    """Move the matchers on; ``True`` for a row whose constraint just completed (its request is done)."""
    done = []
    for s, t in zip(states, tokens):
        if s is None or s.guided is None:
            done.append(False)
            continue
        s.guided.advance(int(t))
        done.append(bool(s.guided.finished))
    return done
