"""Skip-softmax attention (the BLASST tile vote): which per-length scale table a deployment uses and the per-sequence
thresholds the attention kernel consumes.

A KV tile is skipped when its largest score lies below the running row maximum by more than ``ln(lambda)`` for every query
row, with ``lambda = S / L``: ``S`` comes from a calibrated ``[[seqlen_bin, S], ...]`` table (looked up by the largest bin not
above the sequence length ``L``), so the share of skipped tiles stays roughly constant as sequences grow.  Below the first bin
— or wherever ``S >= L`` would make ``lambda`` meaningless — the sequence runs dense.

Checkpoint / flag resolution follows the reference (``tensorrt_edgellm/skip_softmax.py``): keys are read per phase under
``skip_softmax_prefill_*`` and ``skip_softmax_decode_*`` (text config first, then the checkpoint root); for each phase the first
of these wins: an explicit table flag (``[]`` = dense), a target-sparsity flag with a matching tier in ``*_scale_tables``, the
checkpoint's own tier / ``*_scale_table``, a target through the checkpoint's ``*_calibration`` fit ``round(a * exp(b * R))``,
dense.  The prefill tile kernel (``csrc/kernels/attention_tc5_extra.cu``) implements the vote; decode steps run dense here.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Any, Dict, List, Mapping, Optional, Sequence

import torch

MAX_TABLE_ROWS = 128
PHASES = ("prefill", "decode")


class SkipSoftmaxConfigError(ValueError):
    pass


@dataclasses.dataclass(frozen=True)
class SkipSoftmaxDeployment:
    prefill_table: Optional[List[List[int]]] = None      # None = dense
    decode_table: Optional[List[List[int]]] = None
    prefill_calibration: Optional[Dict[str, float]] = None
    prefill_target_sparsity: Optional[float] = None

    @property
    def enabled(self) -> bool:
        return self.prefill_table is not None or self.decode_table is not None


def tier_key(target: float) -> str:
    return f"{round(float(target) * 100):d}%"


def validate_table(rows: Any, name: str = "skip_softmax_prefill_scale_table") -> List[List[int]]:
    """``rows`` as a table sorted by bin; raises on anything but unique non-negative integer ``[seqlen_bin, S]`` pairs."""
    ok = isinstance(rows, list) and len(rows) > 0
    if ok:
        for r in rows:
            if not isinstance(r, (list, tuple)) or len(r) != 2:
                ok = False
                break
            for v in r:
                if isinstance(v, bool) or not isinstance(v, (int, float)) or v < 0 or int(v) != v:
                    ok = False
    if not ok:
        raise SkipSoftmaxConfigError(f"{name} must be a non-empty list of non-negative integer [seqlen_bin, S] rows")
    if len(rows) > MAX_TABLE_ROWS:
        raise SkipSoftmaxConfigError(f"{name} has more than {MAX_TABLE_ROWS} rows")
    table = sorted([int(b), int(s)] for b, s in rows)
    bins = [b for b, _ in table]
    if len(set(bins)) != len(bins):
        raise SkipSoftmaxConfigError(f"{name} repeats a seqlen_bin")
    return table


def _sparsity(value: Any, name: str) -> float:
    try:
        v = float(value)
    except (TypeError, ValueError):
        raise SkipSoftmaxConfigError(f"{name} must be a number in (0, 1), got {value!r}") from None
    if not 0.0 < v < 1.0:
        raise SkipSoftmaxConfigError(f"{name} must be in (0, 1), got {v!r}")
    return v


def _fit(value: Any, name: str) -> Dict[str, float]:
    if not isinstance(value, Mapping):
        raise SkipSoftmaxConfigError(f"{name} must be an object with numeric keys a and b")
    out = {}
    for k in ("a", "b"):
        try:
            out[k] = float(value[k])
        except (KeyError, TypeError, ValueError):
            raise SkipSoftmaxConfigError(f"{name} must carry numeric keys a and b") from None
        if not math.isfinite(out[k]):
            raise SkipSoftmaxConfigError(f"{name}[{k!r}] is not finite")
    return out


def _resolve_phase(phase: str, lookup, table_flag: Any, target_flag: Optional[float]):
    pre = f"skip_softmax_{phase}_"
    if target_flag is not None:
        target_flag = _sparsity(target_flag, f"--{phase}-target-sparsity")
    tiers = lookup(pre + "scale_tables")
    tiers = tiers if isinstance(tiers, Mapping) else {}
    fit = lookup(pre + "calibration")
    fit = _fit(fit, pre + "calibration") if fit is not None else None
    table, target = None, None
    if table_flag is not None:
        if not (isinstance(table_flag, list) and not table_flag):              # [] spells "dense"
            table = validate_table(table_flag, f"--skip-softmax-{phase}-scale-table")
    elif target_flag is not None:
        target = target_flag
        if tier_key(target) in tiers:
            table = validate_table(tiers[tier_key(target)], f"{pre}scale_tables[{tier_key(target)!r}]")
    else:
        ck_target = lookup(pre + "target_sparsity")
        if ck_target is not None:
            ck_target = _sparsity(ck_target, pre + "target_sparsity")
        ck_table = lookup(pre + "scale_table")
        if ck_target is not None and tier_key(ck_target) in tiers:
            target, table = ck_target, validate_table(tiers[tier_key(ck_target)], f"{pre}scale_tables[{tier_key(ck_target)!r}]")
        elif ck_table is not None:
            table = validate_table(ck_table, pre + "scale_table")
        elif ck_target is not None:
            target = ck_target
    if table is None and target is not None:
        if fit is None:
            raise SkipSoftmaxConfigError(f"{phase} target sparsity {target}: no {tier_key(target)!r} table under {pre}scale_tables "
                                         f"and no {pre}calibration to derive S from")
        table = [[0, int(round(fit["a"] * math.exp(fit["b"] * target)))]]
    return table, target, fit


def resolve(config_root: Mapping[str, Any], config_llm: Optional[Mapping[str, Any]] = None, *, prefill_target_sparsity=None,
            prefill_table=None, decode_target_sparsity=None, decode_table=None) -> SkipSoftmaxDeployment:
    """The deployment of one model: checkpoint keys (text config first, then the root) overridden by the four flags."""
    cfgs = [c for c in (config_llm, config_root) if c is not None]

    def lookup(key):
        for c in cfgs:
            if c.get(key) is not None:
                return c.get(key)
        return None

    pt, ptarget, pfit = _resolve_phase("prefill", lookup, prefill_table, prefill_target_sparsity)
    dt, _, _ = _resolve_phase("decode", lookup, decode_table, decode_target_sparsity)
    return SkipSoftmaxDeployment(prefill_table=pt, decode_table=dt, prefill_calibration=pfit if pt is not None else None,
                                 prefill_target_sparsity=ptarget if pt is not None else None)


def scale_for_length(table: Sequence[Sequence[int]], length: int) -> Optional[int]:
    """S of the largest bin not above ``length``; None below the first bin (dense)."""
    s = None
    for b, v in table:
        if b <= length:
            s = v
        else:
            break
    return s


def thresholds_log2(table: Optional[Sequence[Sequence[int]]], seq_lens: Sequence[int], device="cpu") -> Optional[torch.Tensor]:
    """Per-sequence ``log2(S / L)`` for the kernel (``-inf`` = dense); None when no sequence of the step skips anything."""
    if not table:
        return None
    out, any_on = [], False
    for length in seq_lens:
        s = scale_for_length(table, int(length))
        if s is None or s <= 0 or s >= length:
            out.append(float("-inf"))
        else:
            out.append(math.log2(s / float(length)))
            any_on = True
    return torch.tensor(out, dtype=torch.float32, device=device) if any_on else None
