"""LoRA adapters at run time: named adapters attached to a model's linear layers, switched in O(1).

``y = W x + B (A x)`` with ``A [r, in]`` and ``B [out, r]`` (``alpha / r`` folded into B by
``process_lora_weights``).  The low-rank pair runs as two small GEMMs; the second one adds the base
projection's output in its epilogue (``residual``), so an adapted layer costs no extra elementwise pass.
Fused layers (q/k/v, gate/up) take one adapter per source projection: A matrices are stacked, and each B
writes its own column block.

Parity: ``cpp/runtime/state/loraManager.{h,cpp}`` (named adapters, O(1) switch by rebinding ``lora_A_*`` /
``lora_B_*`` tensors; ``docs/source/user_guide/features/lora.md:15-52``)."""
from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
from torch import nn

from .. import ops
from ..checkpoint.safetensors_io import SafetensorsFile
from ..models.linear import LinearBase, TPMode


class _Adapted:
    """Low-rank weights of one linear layer for one adapter: per source, (A [r, in], B [out_src, r], column offset)."""

    def __init__(self):
        self.parts: List[Tuple[torch.Tensor, torch.Tensor, int]] = []


class LoraLinear(nn.Module):
    """Wraps a linear layer; adds the active adapter's low-rank update to its output."""

    grouped_calls = 0                   # how often the stacked form ran (diagnostics / tests)

    def __init__(self, base: LinearBase):
        super().__init__()
        self.base = base
        self.adapters: Dict[str, _Adapted] = {}
        self.active: Optional[_Adapted] = None
        # per-step routing for batches that mix adapters: [(first row, end row, adapter name or None)], rows of the step
        self.segments: Optional[List[Tuple[int, int, Optional[str]]]] = None
        self.segment_rows = 0
        self.row_gid: Optional[torch.Tensor] = None
        self.adapter_ids: Dict[str, int] = {}
        self.grouped = True             # steps that mix adapters use the stacked two-GEMM form (False: one GEMM pair per segment)

    def __getattr__(self, name):            # the model reads attributes such as fused_input_scale, tp_mode, weight
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("base"), name)

    def _stacked(self, names: Tuple[str, ...]):
        """Low-rank factors of several adapters side by side, per adapted column block of this layer:
        ``[(col, n_out, A_cat [m · r, in], B_cat [n_out, m · r], r, {adapter: block index})]`` (ranks padded to the largest)."""
        cache = self.__dict__.setdefault("_stack_cache", {})
        plan = cache.get(names)
        if plan is not None:
            return plan
        blocks: Dict[Tuple[int, int], List[Tuple[str, torch.Tensor, torch.Tensor]]] = {}
        for name in names:
            for a, b, col in self.adapters[name].parts:
                blocks.setdefault((col, b.shape[0]), []).append((name, a, b))
        plan = []
        for (col, n_out), members in blocks.items():
            r = max(a.shape[0] for _, a, _ in members)
            a_cat = torch.zeros(len(members) * r, members[0][1].shape[1], dtype=members[0][1].dtype, device=members[0][1].device)
            b_cat = torch.zeros(n_out, len(members) * r, dtype=members[0][2].dtype, device=members[0][2].device)
            index = {}
            for j, (name, a, b) in enumerate(members):
                a_cat[j * r:j * r + a.shape[0]] = a
                b_cat[:, j * r:j * r + b.shape[1]] = b
                index[name] = j
            plan.append((col, n_out, a_cat, b_cat, r, index))
        if len(cache) > 8:
            cache.clear()
        cache[names] = plan
        return plan

    def _add_grouped(self, y, x, segments) -> None:
        """Batches that mix adapters, in two GEMMs per column block whatever the number of segments (the reference's grouped LoRA
        GEMM, ``cpp/kernels/lora/groupedLoraGemm``): every row is projected through all the step's adapters' ``A`` factors at
        once, the blocks of the adapters a row does not use are zeroed, and one GEMM with the concatenated ``B`` factors adds
        the updates.  The extra ``A`` work is ``m · r`` columns, tiny next to the layer itself."""
        names = tuple(sorted({n for _, _, n in segments if n and n in self.adapters}))
        if not names:
            return
        LoraLinear.grouped_calls += 1
        rows = y.shape[0]
        gid = self.row_gid                       # per row: the adapter's position in the manager's list (-1 = none), built once per step
        if gid is None or gid.shape[0] != rows:
            gid = torch.full((rows,), -1, dtype=torch.long)
            for r0, r1, name in segments:
                if name in self.adapter_ids and r1 > r0:
                    gid[r0:r1] = self.adapter_ids[name]
        gid = gid.to(y.device)
        for col, n_out, a_cat, b_cat, r, index in self._stacked(names):
            lut = torch.full((max(self.adapter_ids.values(), default=0) + 2,), -1, dtype=torch.long)
            for name, j in index.items():
                lut[self.adapter_ids[name] + 1] = j
            owner = lut.to(y.device)[gid + 1]
            t = ops.linear(x, a_cat)                                             # [T, m · r]
            block = torch.arange(a_cat.shape[0], device=y.device) // r
            t = t * (block[None, :] == owner[:, None]).to(t.dtype)
            y[..., col:col + n_out] += ops.linear(t, b_cat)

    def _add(self, y, x16, ad: _Adapted):
        for a, b, col in ad.parts:
            t = ops.linear(x16, a)
            n = b.shape[0]
            y[..., col:col + n] += ops.linear(t, b)

    def forward(self, x):
        y = self.base(x)
        if self.segments is not None and isinstance(y, torch.Tensor) and y.shape[0] == self.segment_rows:
            # segment-routed (``cpp/kernels/lora/groupedLoraGemm`` in the reference): every request's rows get the update
            # of that request's adapter; rows without an adapter pass through
            if not isinstance(x, torch.Tensor):
                raise RuntimeError("LoRA needs 16-bit activations: disable fused activation quantisation for adapted layers")
            live = {n for _, _, n in self.segments if n and n in self.adapters}
            if len(live) > 1 and self.grouped:
                self._add_grouped(y, x, self.segments)
                return y
            for r0, r1, name in self.segments:
                ad = self.adapters.get(name) if name else None
                if ad is not None and r1 > r0:
                    self._add(y[r0:r1], x[r0:r1], ad)
            return y
        ad = self.active
        if ad is None or not isinstance(y, torch.Tensor):
            return y
        x16 = x if isinstance(x, torch.Tensor) else None
        if x16 is None:
            raise RuntimeError("LoRA needs 16-bit activations: disable fused activation quantisation for adapted layers")
        for a, b, col in ad.parts:
            t = ops.linear(x16, a)                                        # [T, r]
            n = b.shape[0]
            if col == 0 and n == y.shape[-1]:
                y = y + ops.linear(t, b) if not y.is_cuda else ops.cuda_ops().gemm(t, b, residual=y)
            else:
                y[..., col:col + n] += ops.linear(t, b)
        return y


class LoraManager:
    """Loads processed adapters (``lora_weights.safetensors`` + ``lora_config.json``) and binds them to a model."""

    def __init__(self, model: nn.Module):
        self.model = model
        self.names: List[str] = []
        self.active: Optional[str] = None
        self._wrapped: Dict[str, LoraLinear] = {}
        self._generation: Dict[str, int] = {}       # name → number of times an adapter was loaded under it

    def generation(self, name: str) -> int:
        """Load counter of ``name``: part of the prefix-cache identity, so K/V cached under an adapter that was later
        replaced under the same name is not reused."""
        return self._generation.get(name, 0)

    def _wrap(self, module_name: str) -> LoraLinear:
        if module_name in self._wrapped:
            return self._wrapped[module_name]
        parent_name, _, leaf = module_name.rpartition(".")
        parent = self.model.get_submodule(parent_name) if parent_name else self.model
        base = getattr(parent, leaf)
        if not isinstance(base, LinearBase):
            raise TypeError(f"{module_name} is not a linear layer")
        if getattr(base, "gate_up_interleaved", False):
            raise RuntimeError(f"{module_name} already stores interleaved gate / up rows for the fused SwiGLU epilogue; attach adapters "
                               "before the model's first GPU step or set TELB_DISABLE_SWIGLU_FUSION=1")
        if hasattr(base, "want_interleave"):
            base.want_interleave = False             # the low-rank update is added to plain [gate | up] columns
        w = LoraLinear(base)
        setattr(parent, leaf, w)
        self._wrapped[module_name] = w
        return w

    def reserve_slots(self, slots_file: str) -> int:
        """Wrap the layers a ``lora_slots.json`` (``trtedge insert-lora --model_dir``) declares adaptable, before any adapter is
        loaded and before the model's first step; records the declared maximum rank.  Returns the number of layers wrapped."""
        with open(slots_file, "r", encoding="utf-8") as f:
            decl = json.load(f)
        self.max_rank = int(decl.get("max_lora_rank", 0) or 0)
        n = 0
        for ckpt_mod in decl.get("slots", {}):
            mod_name, _, _ = self._locate(ckpt_mod)
            if mod_name not in self._wrapped:
                self._wrap(mod_name)
                n += 1
        return n

    def _locate(self, ckpt_module: str) -> Tuple[str, int, LinearBase]:
        """Runtime module, source index of a checkpoint module name (``…self_attn.q_proj`` → ``…self_attn.qkv_proj``, 0)."""
        name = ckpt_module
        for pre in ("base_model.model.",):
            if name.startswith(pre):
                name = name[len(pre):]
        parent, _, leaf = name.rpartition(".")
        for mod_name, mod in self.model.named_modules():
            base = mod.base if isinstance(mod, LoraLinear) else mod
            if not isinstance(base, LinearBase):
                continue
            p2, _, l2 = mod_name.rpartition(".")
            if p2 != parent and not parent.endswith(p2) and not p2.endswith(parent):
                continue
            srcs = base.sources or [l2]
            if leaf in srcs and (p2 == parent or p2.endswith(parent) or parent.endswith(p2)):
                return mod_name, srcs.index(leaf), base
        raise KeyError(f"adapter module {ckpt_module} has no counterpart in the model")

    def load_adapter(self, name: str, adapter_dir: str) -> None:
        f = SafetensorsFile(os.path.join(adapter_dir, "lora_weights.safetensors"))
        with open(os.path.join(adapter_dir, "lora_config.json"), "r", encoding="utf-8") as fh:
            meta = json.load(fh)
        if getattr(self, "max_rank", 0) and int(meta.get("rank", 0)) > self.max_rank:
            raise ValueError(f"adapter {name!r} has rank {meta.get('rank')}, the model declares at most {self.max_rank}")
        if name in self.names:                      # reloading under a known name replaces the old weights
            for w in self._wrapped.values():
                old = w.adapters.pop(name, None)
                if old is not None and w.active is old:
                    w.active = None
        self._generation[name] = self._generation.get(name, 0) + 1
        for w in self._wrapped.values():
            w.__dict__.pop("_stack_cache", None)          # stacked factors are rebuilt with the new adapter set
        for ckpt_mod in meta["modules"]:
            mod_name, src, base = self._locate(ckpt_mod)
            a, b = f.get(f"lora_A_{ckpt_mod}").clone(), f.get(f"lora_B_{ckpt_mod}").clone()
            dev, dt = base.weight.device, getattr(base, "act_dtype", None) or (base.weight.dtype if base.weight.dtype.is_floating_point else torch.bfloat16)
            if base.tp_mode == TPMode.COL and base.tp_size > 1:
                b = b.chunk(base.tp_size, 0)[base.tp_rank]
            elif base.tp_mode == TPMode.ROW and base.tp_size > 1:
                a = a.chunk(base.tp_size, 1)[base.tp_rank]
            col = sum(base.out_sizes[:src])
            w = self._wrap(mod_name)
            w.adapters.setdefault(name, _Adapted()).parts.append((a.to(dev, dt).contiguous(), b.to(dev, dt).contiguous(), col))
        if name not in self.names:
            self.names.append(name)

    def set_segments(self, segments: Optional[Sequence[Tuple[int, int, Optional[str]]]]) -> None:
        """Route the rows of the next step(s): ``[(first row, end row, adapter name or None), ...]``; ``None`` returns to
        the single active adapter.  Unknown names raise before anything runs."""
        rows = 0
        if segments is not None:
            for r0, r1, name in segments:
                if name and name not in self.names:
                    raise KeyError(f"unknown adapter {name!r}; loaded: {self.names}")
                rows = max(rows, r1)
            if not any(name for _, _, name in segments):
                segments = None                      # nobody uses an adapter this step: skip the routing entirely
        gid = None
        ids = {n: i for i, n in enumerate(self.names)}
        if segments is not None:
            gid = torch.full((rows,), -1, dtype=torch.long)
            for r0, r1, name in segments:
                if name and r1 > r0:
                    gid[r0:r1] = ids[name]
            dev = next((w.base.weight.device for w in self._wrapped.values()), None)
            if dev is not None:
                gid = gid.to(dev)                     # one upload per step, shared by every adapted layer
        for w in self._wrapped.values():
            w.segments = list(segments) if segments is not None else None
            w.segment_rows = rows
            w.row_gid, w.adapter_ids = gid, ids

    def set_active(self, name: Optional[str]) -> None:
        if name is not None and name not in self.names:
            raise KeyError(f"unknown adapter {name!r}; loaded: {self.names}")
        for w in self._wrapped.values():
            w.active = w.adapters.get(name) if name is not None else None
        self.active = name
