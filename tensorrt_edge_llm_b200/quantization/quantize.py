from __future__ import annotations

import json
import os
import shutil
from typing import Dict, Iterable, List, Optional, Sequence

import torch

from ..checkpoint.safetensors_io import CheckpointReader, save_file
from ..ops import reference as ref

_LINEAR_SUFFIXES = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj", "in_proj", "out_proj",
                    "in_proj_qkv", "in_proj_z", "fc1", "fc2")
_ALGOS = {"nvfp4": "NVFP4", "int4_awq": "W4A16_AWQ", "int4_gptq": "W4A16_GPTQ", "fp8": "FP8", "int8_sq": "W8A8_SQ_PER_CHANNEL",
          "mxfp8": "MXFP8", "q8_0": "Q8_0", "fp16": None, "bf16": None}


def build_quant_config(quantization: str, exclude: Sequence[str] = ("lm_head",), kv_cache_quantization: Optional[str] = None,
                       group_size: Optional[int] = None) -> dict:
    """The ``hf_quant_config.json`` body for one of the supported weight formats."""
    if quantization not in _ALGOS or _ALGOS[quantization] is None:
        raise ValueError(f"unsupported quantization {quantization!r}; choose one of {sorted(k for k, v in _ALGOS.items() if v)}")
    if kv_cache_quantization not in (None, "fp8"):
        raise ValueError("kv_cache_quantization must be fp8 or unset")
    return {"producer": {"name": "tensorrt_edge_llm_b200"},
            "quantization": {"quant_algo": _ALGOS[quantization], "group_size": group_size or (16 if quantization == "nvfp4" else 128),
                             "kv_cache_quant_algo": "FP8" if kv_cache_quantization == "fp8" else None,
                             "exclude_modules": list(exclude)}}


def _is_target(name: str, shape, exclude: Sequence[str]) -> bool:
    if not name.endswith(".weight") or len(shape) != 2:
        return False
    mod = name[:-len(".weight")]
    if any(mod == e or mod.endswith("." + e) or e.strip("*") in mod for e in exclude):
        return False
    return mod.rsplit(".", 1)[-1] in _LINEAR_SUFFIXES


def _int4_group_qdq(w: torch.Tensor, g: int) -> torch.Tensor:
    """Symmetric 4-bit group quantise-dequantise of ``w [out, in]`` along the input dimension."""
    wg = w.reshape(w.shape[0], w.shape[1] // g, g)
    scale = (wg.abs().amax(-1, keepdim=True) / 7.0).clamp(min=1e-8)
    return (torch.round(wg / scale).clamp(-8, 7) * scale).reshape(w.shape)


@torch.no_grad()
def gptq_quantize(w: torch.Tensor, x: torch.Tensor, group: int = 128, block: int = 128, damp: float = 0.01):
    """GPTQ for one linear layer: quantise ``w [out, in]`` to asymmetric 4-bit groups column by column, after each column
    spreading its rounding error over the columns not yet quantised, weighted by the inverse Hessian of the layer's
    least-squares objective ``|x (w - q)ᵀ|²`` (``H = 2 xᵀx / n`` from calibration rows ``x [n, in]``, damped by ``damp`` of
    its mean diagonal).  A group's scale and zero point are taken from the group's columns as they stand when the walk
    reaches them.  Returns ``(codes [out, in] in 0..15, scales [out, in / group], zeros [out, in / group])`` with
    ``w ≈ (codes - zero) · scale``."""
    w = w.float().clone()
    n_out, n_in = w.shape
    if n_in % group or block % group:
        raise ValueError("GPTQ: the input size must be a multiple of the group, the block a multiple of the group")
    h = (x.float().t() @ x.float()) * (2.0 / max(x.shape[0], 1))
    dead = h.diagonal() == 0
    h[dead, dead] = 1.0
    w[:, dead] = 0.0
    h += torch.eye(n_in) * damp * float(h.diagonal().mean())
    u = torch.linalg.cholesky(torch.cholesky_inverse(torch.linalg.cholesky(h)), upper=True)
    codes = torch.zeros_like(w)
    scales = torch.zeros(n_out, n_in // group)
    zeros = torch.zeros(n_out, n_in // group)
    for i1 in range(0, n_in, block):
        i2 = min(i1 + block, n_in)
        w1, err1, u1 = w[:, i1:i2].clone(), torch.zeros(n_out, i2 - i1), u[i1:i2, i1:i2]
        for i in range(i2 - i1):
            col = i1 + i
            if col % group == 0:
                seg = w1[:, i:i + group]
                lo, hi = seg.amin(1).clamp(max=0), seg.amax(1).clamp(min=0)
                sc = ((hi - lo) / 15.0).clamp(min=1e-8)
                scales[:, col // group], zeros[:, col // group] = sc, torch.round(-lo / sc).clamp(0, 15)
            sc, zp = scales[:, col // group], zeros[:, col // group]
            q = torch.round(w1[:, i] / sc + zp).clamp(0, 15)
            codes[:, col] = q
            e = (w1[:, i] - (q - zp) * sc) / u1[i, i]
            w1[:, i:] -= e[:, None] * u1[i, i:][None, :]
            err1[:, i] = e
        w[:, i2:] -= err1 @ u[i1:i2, i2:]
    return codes, scales, zeros


def _collect_linear_inputs(model_dir: str, calib_ids, num_samples: int, seq_len: int, device: str, max_rows: int):
    """Run the 16-bit model over calibration ids and keep up to ``max_rows`` input rows of every linear layer.
    Returns ``(model, {runtime module name: rows [n, in] fp32 on the CPU})``."""
    from ..model import AutoModel
    from ..models.linear import LinearBase
    from ..runtime.kv_cache import KVCacheManager
    from ..runtime.runner import ModelRunner
    model = AutoModel.from_pretrained(model_dir, device=device)
    cfg = model.cfg
    if calib_ids is None:
        calib_ids = torch.randint(0, cfg.vocab_size, (num_samples, seq_len), generator=torch.Generator().manual_seed(0))
    acts: Dict[str, List[torch.Tensor]] = {}
    hooks = []
    for name, mod in model.named_modules():
        if isinstance(mod, LinearBase) and name.rsplit(".", 1)[-1] != "lm_head":
            def pre(m, args, name=name):
                x = args[0]
                if isinstance(x, torch.Tensor):
                    keep = acts.setdefault(name, [])
                    if sum(t.shape[0] for t in keep) < max_rows:
                        keep.append(x.detach().reshape(-1, x.shape[-1]).float()[:max_rows].cpu())
            hooks.append(mod.register_forward_pre_hook(pre))
    page = 64
    pages_per_seq = (calib_ids.shape[1] + page - 1) // page + 1
    kv = KVCacheManager(cfg, num_pages=pages_per_seq * 2, page_size=page, max_seats=2, max_pages_per_seq=pages_per_seq, device=device)
    runner = ModelRunner(model, kv)
    runner.use_cuda_graphs = False
    for row in calib_ids.tolist():
        runner.prefill([0], [row])
        kv.free(0)
    for hk in hooks:
        hk.remove()
    return model, {k: torch.cat(v, 0)[:max_rows] for k, v in acts.items()}


@torch.no_grad()
def gptq_calibration_rows(model_dir: str, calib_ids: Optional[torch.Tensor] = None, num_samples: int = 8, seq_len: int = 128,
                          device: str = "cpu", max_rows: int = 512) -> Dict[str, torch.Tensor]:
    """Calibration input rows per *checkpoint* linear module (fused projections share theirs), for :func:`gptq_quantize`."""
    from ..models.linear import LinearBase
    model, acts = _collect_linear_inputs(model_dir, calib_ids, num_samples, seq_len, device, max_rows)
    out: Dict[str, torch.Tensor] = {}
    for name, mod in model.named_modules():
        if isinstance(mod, LinearBase) and name in acts:
            parent = name.rsplit(".", 1)[0] if "." in name else ""
            for src in (mod.sources or [name.rsplit(".", 1)[-1]]):
                out[(parent + "." if parent else "") + src] = acts[name]
    return out


@torch.no_grad()
def awq_search(model_dir: str, calib_ids: Optional[torch.Tensor] = None, num_samples: int = 8, seq_len: int = 128, device: str = "cpu",
               group_size: int = 128, grid: int = 20, max_rows: int = 512) -> Dict[str, torch.Tensor]:
    """Activation-aware weight scaling (AWQ) for INT4 group quantisation.

    Weights that multiply large activations matter more; scaling input channel ``c`` of ``W`` up by ``s_c`` before rounding
    (and the activation down by the same factor at run time: the checkpoint's ``pre_quant_scale = 1 / s``) spends the 4-bit
    grid where it counts.  Per linear layer — fused projections share their input, hence one scale vector — the search
    takes ``s = mean|x|^alpha`` (normalised to geometric mean 1 between its extremes), tries ``alpha`` on a grid from 0
    (plain rounding) to 1 and keeps the one with the smallest output error on calibration activations.
    Returns ``{checkpoint module name: pre_quant_scale [in]}`` (fp32) for the layers where a scale other than 1 won.
    (The search of ModelOpt's ``awq_lite``, which produces the ``pre_quant_scale`` tensors of INT4-AWQ checkpoints.)"""
    from ..models.linear import LinearBase
    model, acts = _collect_linear_inputs(model_dir, calib_ids, num_samples, seq_len, device, max_rows)
    out: Dict[str, torch.Tensor] = {}
    for name, mod in model.named_modules():
        if not isinstance(mod, LinearBase) or name not in acts or not hasattr(mod, "weight") or not mod.weight.dtype.is_floating_point:
            continue
        w = mod.weight.detach().float().cpu()
        if w.dim() != 2 or w.shape[1] % group_size:
            continue
        x = acts[name]
        want = x @ w.t()
        s_x = x.abs().mean(0).clamp(min=1e-4)
        best_err, best_s = float((x @ _int4_group_qdq(w, group_size).t() - want).pow(2).mean()), None
        for step in range(1, grid + 1):
            sc = s_x.pow(step / grid)
            sc = (sc / (sc.max() * sc.min()).sqrt()).clamp(min=1e-4)
            err = float(((x / sc) @ _int4_group_qdq(w * sc, group_size).t() - want).pow(2).mean())
            if err < best_err:
                best_err, best_s = err, sc
        if best_s is not None:
            parent = name.rsplit(".", 1)[0] if "." in name else ""
            for src in (mod.sources or [name.rsplit(".", 1)[-1]]):
                out[(parent + "." if parent else "") + src] = (1.0 / best_s).float()
    return out


@torch.no_grad()
def calibrate_input_scales(model_dir: str, calib_ids: Optional[torch.Tensor] = None, num_samples: int = 8, seq_len: int = 128,
                           device: str = "cpu") -> Dict[str, float]:
    """Max-calibrate the input of every linear layer: run the 16-bit model over calibration token ids
    and record ``amax / (6 · 448)`` per checkpoint module (fused layers share their input, so every
    source module gets the same scale).  Without calibration ids, seeded uniform ids are used."""
    from ..model import AutoModel
    from ..models.linear import LinearBase
    from ..runtime.kv_cache import KVCacheManager
    from ..runtime.runner import ModelRunner
    model = AutoModel.from_pretrained(model_dir, device=device)
    cfg = model.cfg
    if calib_ids is None:
        g = torch.Generator().manual_seed(0)
        calib_ids = torch.randint(0, cfg.vocab_size, (num_samples, seq_len), generator=g)
    amax: Dict[str, float] = {}
    hooks = []
    for name, mod in model.named_modules():
        if isinstance(mod, LinearBase):
            def pre(m, args, name=name):
                x = args[0]
                if isinstance(x, torch.Tensor):
                    amax[name] = max(amax.get(name, 0.0), float(x.detach().abs().max()))
            hooks.append(mod.register_forward_pre_hook(pre))
    page = 64
    pages_per_seq = (calib_ids.shape[1] + page - 1) // page + 1
    kv = KVCacheManager(cfg, num_pages=pages_per_seq * 2, page_size=page, max_seats=2, max_pages_per_seq=pages_per_seq, device=device)
    runner = ModelRunner(model, kv)
    runner.use_cuda_graphs = False
    for row in calib_ids.tolist():
        runner.prefill([0], [row])
        kv.free(0)
    for h in hooks:
        h.remove()
    scales: Dict[str, float] = {}
    for name, mod in model.named_modules():
        if isinstance(mod, LinearBase) and name in amax:
            parent = name.rsplit(".", 1)[0] if "." in name else ""
            for s in (mod.sources or [name.rsplit(".", 1)[-1]]):
                scales[(parent + "." if parent else "") + s] = max(amax[name], 1e-6) / (ref.FP4_MAX * ref.E4M3_MAX)
    return scales


@torch.no_grad()
def quantize_and_export(model_dir: str, out_dir: str, quantization: str = "nvfp4", exclude: Sequence[str] = ("lm_head",),
                        kv_cache_quantization: Optional[str] = None, calib_ids: Optional[torch.Tensor] = None,
                        calibrate: bool = True, device: str = "cpu", group_size: int = 128) -> dict:
    """Quantise the linear layers of a 16-bit checkpoint and write a unified quantised checkpoint."""
    qcfg = build_quant_config(quantization, exclude, kv_cache_quantization, None if quantization == "nvfp4" else group_size)
    os.makedirs(out_dir, exist_ok=True)
    scales = calibrate_input_scales(model_dir, calib_ids, device=device) if (calibrate and quantization == "nvfp4") else {}
    pre_quant = awq_search(model_dir, calib_ids, device=device, group_size=group_size) if (calibrate and quantization == "int4_awq") else {}
    gptq_rows = gptq_calibration_rows(model_dir, calib_ids, device=device) if (calibrate and quantization == "int4_gptq") else {}
    reader = CheckpointReader(model_dir)
    out: Dict[str, torch.Tensor] = {}
    n_q = 0
    for key in reader.keys():
        t = reader.get(key)
        canon = key
        for pre in ("model.language_model.", "language_model.model."):
            if canon.startswith(pre):
                canon = "model." + canon[len(pre):]
        if not _is_target(canon, t.shape, exclude):
            out[key] = t.clone()
            continue
        base = key[:-len(".weight")]
        w = t.to(device).float()
        if quantization == "nvfp4":
            if w.shape[1] % 16:
                out[key] = t.clone()
                continue
            packed, sf, gs = ref.nvfp4_quantize(w)
            out[key] = packed.cpu()
            out[base + ".weight_scale"] = sf.cpu()
            out[base + ".weight_scale_2"] = gs.reshape(()).cpu()
            mod = canon[:-len(".weight")]
            out[base + ".input_scale"] = torch.tensor(scales.get(mod, 1.0 / 448.0), dtype=torch.float32)
        elif quantization in ("int4_gptq", "fp8", "int8_sq", "mxfp8", "q8_0"):
            from ..checkpoint import repacking as rp
            g = group_size
            if (quantization == "int4_gptq" and (w.shape[1] % g or w.shape[0] % 8)) or w.shape[1] % 32:
                out[key] = t.clone()
                continue
            rows = gptq_rows.get(canon[:-len(".weight")]) if quantization == "int4_gptq" else None
            if rows is not None and rows.shape[1] == w.shape[1]:
                # error-compensated rounding against the layer's calibration inputs, then the GPTQ tensor layout
                codes, sc, zp = gptq_quantize(w.cpu(), rows, g, block=max(g, 128) if 128 % g == 0 or g % 128 == 0 else g)
                enc = {"qweight": rp._pack_int32_nibbles(codes.t().contiguous(), 0), "qzeros": rp._pack_int32_nibbles((zp.t().contiguous() - 1) % 16, 1),
                       "scales": sc.t().contiguous().to(torch.float16), "g_idx": (torch.arange(w.shape[1]) // g).to(torch.int32)}
            else:
                enc = {"int4_gptq": lambda x: rp.encode_gptq(x, g), "fp8": rp.encode_fp8, "int8_sq": rp.encode_int8_sq,
                       "mxfp8": rp.encode_mxfp8, "q8_0": rp.encode_q8_0}[quantization](w.cpu())
            for name, v in enc.items():
                out[base + "." + name] = v.reshape(-1) if v.dim() == 0 else v
        else:
            g = group_size
            if w.shape[1] % g or w.shape[0] % 2:
                out[key] = t.clone()
                continue
            pqs = pre_quant.get(canon[:-len(".weight")])
            if pqs is not None:                       # activation-aware scaling: W · diag(s) is rounded, the run time applies 1 / s
                w = w / pqs.to(w.device)[None, :]
                out[base + ".pre_quant_scale"] = pqs.to(t.dtype).cpu()
            wg = w.reshape(w.shape[0], w.shape[1] // g, g)
            scale = (wg.abs().amax(-1) / 7.0).clamp(min=1e-8)
            q = (torch.round(wg / scale[..., None]).clamp(-8, 7) + 8).to(torch.uint8).reshape(w.shape)
            out[key] = (q[0::2] | (q[1::2] << 4)).cpu()
            out[base + ".weight_scale"] = scale.to(t.dtype).cpu()
        n_q += 1
    save_file(out, os.path.join(out_dir, "model.safetensors"))
    for fname in os.listdir(model_dir):
        if fname.endswith((".json", ".jinja", ".txt", ".model")) and not fname.startswith("model.safetensors") and fname != "hf_quant_config.json":
            shutil.copy(os.path.join(model_dir, fname), os.path.join(out_dir, fname))
    with open(os.path.join(out_dir, "hf_quant_config.json"), "w", encoding="utf-8") as f:
        json.dump(qcfg, f, indent=1)
    return {"quantized_linears": n_q, "tensors": len(out), "config": qcfg}
