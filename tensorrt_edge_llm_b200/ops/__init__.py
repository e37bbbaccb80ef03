"""Operator front end.

Each function executes the hand-written sm_100a kernel when its tensors live on a CUDA
device and the plain-PyTorch statement (``ops.reference``) on CPU.  There is no silent
fallback on a GPU: if the native library is missing, the CUDA path raises.

Parity: the custom-op surface of ``tensorrt_edgellm/models/ops.py`` (attention_plugin :145,
nvfp4 ops :917-951, causal_conv1d :1541, update_ssm_state :1631, gated_delta_net :1908,
MoE plugins :2017-2209, all_reduce :2754) expressed as directly executable functions.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import reference as ref
from .meta import StepMeta, build_step_meta

__all__ = ["StepMeta", "build_step_meta", "ref", "cuda_ops"]


def cuda_ops():
    """The ctypes binding module (imported lazily so CPU-only use never touches it)."""
    from . import cuda as _cuda
    return _cuda


def rmsnorm(x, weight, eps):
    if x.is_cuda:
        return cuda_ops().rmsnorm(x, weight, eps)
    return ref.rmsnorm(x, weight, eps)


def add_rmsnorm(x, residual, weight, eps, quant_scale=None):
    """``quant_scale`` (CUDA only): emit the normalised output directly as NVFP4 for the next GEMM."""
    if x.is_cuda:
        if quant_scale is not None:
            return cuda_ops().rmsnorm_quant(x, residual, weight, eps, quant_scale)
        return cuda_ops().add_rmsnorm(x, residual, weight, eps)
    return ref.add_rmsnorm(x, residual, weight, eps)


def rmsnorm_maybe_quant(x, weight, eps, quant_scale=None):
    if x.is_cuda and quant_scale is not None:
        return cuda_ops().rmsnorm_quant(x, None, weight, eps, quant_scale)[0]
    return rmsnorm(x, weight, eps)


def layernorm(x, weight, bias, eps):
    if x.is_cuda:
        return cuda_ops().layernorm(x, weight, bias, eps)
    return ref.layernorm(x, weight, bias, eps)


def gated_group_rmsnorm(x, z, weight, n_groups, eps):
    if x.is_cuda:
        return cuda_ops().gated_group_rmsnorm(x, z, weight, n_groups, eps)
    return ref.gated_group_rmsnorm(x, z, weight, n_groups, eps)


def swiglu(gate_up, quant_scale=None, interleaved=False):
    """``interleaved``: the columns hold blocks of 64 gate features followed by their 64 up features (the layout the fused
    gate/up GEMM epilogue uses) instead of ``[gate | up]``; only the quantising CUDA form takes it."""
    if gate_up.is_cuda:
        if quant_scale is not None:
            return cuda_ops().swiglu_quant(gate_up, quant_scale, interleaved)
        assert not interleaved
        return cuda_ops().swiglu(gate_up)
    assert not interleaved
    return ref.swiglu(gate_up)


def geglu(gate_up, tanh_approx=True):
    """``gelu(gate) * up`` over the fused ``[T, 2·I]`` projection output (GeGLU MLPs)."""
    if gate_up.is_cuda:
        return cuda_ops().geglu(gate_up, tanh_approx)
    inter = gate_up.shape[-1] // 2
    g = torch.nn.functional.gelu(gate_up[..., :inter].float(), approximate="tanh" if tanh_approx else "none")
    return (g * gate_up[..., inter:].float()).to(gate_up.dtype)


def relu2(x):
    if x.is_cuda:
        return cuda_ops().relu2(x)
    return ref.relu2(x)


def gelu(x, tanh_approx=False):
    if x.is_cuda:
        return cuda_ops().gelu(x, tanh_approx)
    return torch.nn.functional.gelu(x.float(), approximate="tanh" if tanh_approx else "none").to(x.dtype)


def embedding(ids, table):
    if hasattr(table, "lookup"):              # FP8 / NVFP4 table (models/embedding.py): gather stored rows, then expand
        return table.lookup(ids)
    if table.is_cuda:
        return cuda_ops().embedding(ids, table)
    return ref.embedding(ids, table)


def linear(x, weight, bias=None):
    if x.is_cuda:
        return cuda_ops().gemm(x, weight, bias)
    return ref.linear(x, weight, bias)


def rope_kv_write(qkv, kv_layer, meta, cos_sin, num_q_heads, num_kv_heads, head_dim,
                  q_norm_w=None, k_norm_w=None, eps=1e-6):
    if qkv.is_cuda:
        return cuda_ops().rope_kv_write(qkv, kv_layer, meta, cos_sin, num_q_heads, num_kv_heads, head_dim,
                                        q_norm_w, k_norm_w, eps)
    return ref.rope_kv_write(qkv, kv_layer, meta, cos_sin, num_q_heads, num_kv_heads, head_dim,
                             q_norm_w, k_norm_w, eps)


def rope_cos_sin(max_pos, rotary_dim, theta, scaling=None, device="cpu"):
    """RoPE ``[max_pos, rotary_dim]`` cos | sin table (fp32, angles in fp64) with the frequency scaling of the checkpoint; built by
    a kernel when the table lives on a GPU."""
    dev = torch.device(device)
    if dev.type == "cuda":
        inv, att = ref.rope_frequencies(max_pos, rotary_dim, theta, scaling)
        return cuda_ops().rope_table(inv, att, max_pos, dev)
    return ref.rope_cos_sin(max_pos, rotary_dim, theta, scaling, device=device)


def mrope_rows(cos_sin, positions3, sections):
    """Multimodal RoPE: per-row cos | sin tables gathered by each row's (temporal, height, width) positions."""
    if cos_sin.is_cuda:
        return cuda_ops().mrope_rows(cos_sin, positions3, sections)
    return ref.mrope_rows(cos_sin, positions3, sections)


def rope_q(q, kv_layer, meta, cos_sin, num_q_heads, head_dim, q_norm_w=None, eps=1e-6):
    """Per-head RMSNorm and RoPE of the queries of a layer that writes no keys / values (``kv_layer`` is only read later; the
    GPU form runs the RoPE + KV-write kernel with zero KV heads, so nothing is stored)."""
    if q.is_cuda:
        return cuda_ops().rope_kv_write(q, kv_layer, meta, cos_sin, num_q_heads, 0, head_dim, q_norm_w, None, eps)
    return ref.rope_q(q, meta, cos_sin, num_q_heads, head_dim, q_norm_w, eps)


def paged_attention(q, kv_layer, meta, scale, sliding_window=None, sinks=None, causal=True):
    if q.is_cuda:
        return cuda_ops().paged_attention(q, kv_layer, meta, scale, sliding_window, sinks, causal=causal)
    return ref.paged_attention(q, kv_layer, meta, scale, sliding_window, sinks, causal=causal)


def kv_fp8_prepare(kv_layer, meta, scales, dtype, window=0):
    """FP8 KV layer → the 16-bit staging layer holding the step's cached pages (new rows are written into it next)."""
    if kv_layer.is_cuda:
        cu = cuda_ops()
        stage = cu.kv_fp8_stage(kv_layer, dtype)
        cu.kv_fp8_load(kv_layer, stage, meta, scales, window)
        return stage
    stage = torch.zeros(kv_layer.shape, dtype=dtype)
    ref.kv_fp8_load(kv_layer, stage, meta, scales, window)
    return stage


def kv_fp8_commit(kv_layer, stage, meta, scales):
    """Quantise the step's new rows from the staging layer into the FP8 layer (and round the staged rows the same way)."""
    if kv_layer.is_cuda:
        return cuda_ops().kv_fp8_store(kv_layer, stage, meta, scales)
    return ref.kv_fp8_store(kv_layer, stage, meta, scales)


def argmax(logits):
    if logits.is_cuda:
        return cuda_ops().argmax(logits)
    return ref.argmax(logits)


def sample(logits, temperature, top_k, top_p, uniforms):
    if logits.is_cuda:
        return cuda_ops().sample(logits, temperature, top_k, top_p, uniforms)
    return ref.sample(logits, temperature, top_k, top_p, uniforms)


def moe_route(logits, top_k, renormalize=True):
    if logits.is_cuda:
        return cuda_ops().moe_route_softmax_topk(logits, top_k, renormalize)
    return ref.moe_route_softmax_topk(logits, top_k, renormalize)


def causal_conv1d(x, weight, bias, conv_state, meta, activation=True):
    if x.is_cuda:
        return cuda_ops().causal_conv1d(x, weight, bias, conv_state, meta, activation)
    return ref.causal_conv1d(x, weight, bias, conv_state, meta, activation)


def ssm_scan(x, dt, A, B, C, D, dt_bias, ssm_state, meta, z=None, dt_softplus=True, dt_limit=0.0):
    if x.is_cuda:
        return cuda_ops().ssm_scan(x, dt, A, B, C, D, dt_bias, ssm_state, meta, z, dt_softplus, dt_limit)
    return ref.ssm_scan(x, dt, A, B, C, D, dt_bias, ssm_state, meta, z, dt_softplus, dt_limit)


def gated_delta_rule(q, k, v, a, b, A_log, dt_bias, state, meta):
    if q.is_cuda:
        return cuda_ops().gated_delta_rule(q, k, v, a, b, A_log, dt_bias, state, meta)
    return ref.gated_delta_rule(q, k, v, a, b, A_log, dt_bias, state, meta)


def spec_accept_greedy(target_tokens, tree_tokens, parents, max_path, force_len=0):
    if tree_tokens.is_cuda:
        return cuda_ops().spec_accept_greedy(target_tokens, tree_tokens, parents, max_path, force_len)
    return ref.spec_accept_greedy(target_tokens, tree_tokens, parents, max_path, force_len)


def token_logprobs(logits, tokens, k):
    """Log-probability of each row's token and its ``k`` most likely tokens: ``(chosen, top_ids, top_values)``."""
    if logits.is_cuda and logits.stride(-1) == 1 and k <= 32 and logits.dtype in (torch.float16, torch.bfloat16, torch.float32):
        return cuda_ops().token_logprobs(logits, tokens, k)
    return ref.token_logprobs(logits, tokens, k)


def spec_accept_sampling(target_probs, tree_tokens, parents, max_path, uniforms):
    """Lossless acceptance along a draft tree for sampled requests (sibling-by-sibling rejection against each node's target
    distribution, bonus token from the residual): ``(path, path_len, bonus)``."""
    if target_probs.is_cuda:
        return cuda_ops().spec_accept_sampling(target_probs, tree_tokens, parents, max_path, uniforms)
    return ref.spec_accept_sampling(target_probs, tree_tokens, parents, max_path, uniforms)


def eagle_tree_meta(parents, base_pos, depth_base, pos_offset):
    """``(mask [B*R, W], depth [B, R], positions [B*R])`` of a batch of trees given as parent tables."""
    if parents.is_cuda:
        return cuda_ops().eagle_tree_meta(parents, base_pos, depth_base, pos_offset)
    return ref.eagle_tree_meta(parents, base_pos, depth_base, pos_offset)


def eagle_select_verify(p_sc, p_tok, p_par, p_dep, root, keep):
    """Verification tree ``(tokens, parents, depths)``: the ``keep`` best pool candidates in pool order behind the root."""
    if p_sc.is_cuda:
        return cuda_ops().eagle_select_verify(p_sc, p_tok, p_par, p_dep, root, keep)
    return ref.eagle_select_verify(p_sc, p_tok, p_par, p_dep, root, keep)


def dflash2_grouped_dynamic_conv(hidden, delta, base, residual, block, group_size):
    """``out[t, c] = Σ_k (base[k, c] + delta[t, k, c // group_size]) · hidden[t - k, c]`` over the taps that stay inside row ``t``'s
    proposal block, plus ``residual`` when given."""
    if hidden.is_cuda and hidden.dtype in (torch.float16, torch.bfloat16) and group_size % 2 == 0 and base.shape[0] <= 4:
        return cuda_ops().dflash2_grouped_dynamic_conv(hidden, delta, base, residual, block, group_size)
    return ref.dflash2_grouped_dynamic_conv(hidden, delta, base, residual, block, group_size)


def dflash2_selector_walk(cand_ids, unary, projected, anchor, pred_codebook, succ_codebook, temperatures=None, uniforms=None):
    """Chain selector of DFlash 2: per slot, the candidate with the best ``unary + <P[prev] ⊙ z, Q[candidate]>`` (or a draw from
    the softmax of those scores) becomes the slot's token and the next slot's predecessor."""
    if (cand_ids.is_cuda and projected.dtype in (torch.float16, torch.bfloat16) and pred_codebook.dtype == projected.dtype
            and succ_codebook.dtype == projected.dtype and cand_ids.shape[-1] <= 32 and projected.shape[-1] <= 1024):
        return cuda_ops().dflash2_selector_walk(cand_ids, unary, projected, anchor, pred_codebook, succ_codebook, temperatures, uniforms)
    return ref.dflash2_selector_walk(cand_ids, unary, projected, anchor, pred_codebook, succ_codebook, temperatures, uniforms)


def markov_chain_propose(logits, w1, w2, first_prev, temperatures=None, uniforms=None):
    """DSpark's Markov head: step ``i`` picks from ``logits[:, i] + W2 · W1[previous token]``.  All-greedy batches run as one
    fused correction + arg-max kernel per step on the GPU; batches with sampled rows use library ops."""
    if (logits.is_cuda and temperatures is None and w1.dtype in (torch.float16, torch.bfloat16) and w2.dtype == w1.dtype
            and w1.shape[1] <= 512 and logits.shape[0] * w1.shape[1] <= 48 * 1024 and w2.shape[0] == logits.shape[-1]):
        return cuda_ops().markov_greedy_chain(logits, w1, w2, first_prev)
    return ref.markov_chain_propose(logits, w1, w2, first_prev, temperatures, uniforms)


def lattice_chain_walk(cand_ids, transition, temperatures=None, uniforms=None):
    """LiLiCorr's walk: per slot, the candidate with the best ``transition[slot, previous index, ·]`` (or a draw from its softmax)."""
    if cand_ids.is_cuda and cand_ids.shape[-1] <= 32:
        return cuda_ops().lattice_chain_walk(cand_ids, transition, temperatures, uniforms)
    return ref.lattice_chain_walk(cand_ids, transition, temperatures, uniforms)


def low_rank_candidate_head(hidden, down_proj, up_proj, lm_head, num_candidates):
    """EAGLE-4 candidate head: ``(ids [R, Kc] int32, log-probabilities [R, Kc] fp32)`` of the ``Kc`` tokens the low-rank
    scores pick, ordered by their exact logits.  On the GPU the two low-rank products and the top-k are library ops and the
    exact rescoring, ordering and log-softmax are one kernel."""
    if hidden.is_cuda and hidden.dtype in (torch.float16, torch.bfloat16) and lm_head.dtype == hidden.dtype:
        proj = (hidden @ down_proj.to(hidden.dtype).t())                  # fp32 accumulation, rounded to the 16-bit type
        scores = (proj @ up_proj.to(hidden.dtype).t()).float()
        scores = torch.nan_to_num(scores, nan=float("-inf"))
        cand = scores.topk(num_candidates, dim=-1).indices
        return cuda_ops().candidate_rescore(hidden, lm_head, cand)
    return ref.low_rank_candidate_head(hidden, down_proj, up_proj, lm_head, num_candidates)


def kv_commit_path(pool, page_table, past_len, path, path_len):
    if pool.is_cuda:
        return cuda_ops().kv_commit_path(pool, page_table, past_len, path, path_len)
    return ref.kv_commit_path(pool, page_table, past_len, path, path_len)


def apply_token_bitmask(logits, bitmask):
    """Entries whose bit is 0 in ``bitmask [rows, ceil(V/32)]`` become very negative (guided decoding)."""
    if logits.is_cuda:
        return cuda_ops().apply_token_bitmask(logits, bitmask)
    return ref.apply_token_bitmask(logits, bitmask)


def ddtree_candidates(logits, k):
    """Per-depth top-``k`` candidates of a block draft with whole-vocabulary log-probabilities (torch ops on the logits' device)."""
    return ref.ddtree_candidates(logits, k)


def ddtree_assemble(cand_ids, cand_lp, root_tokens, num_nodes, depth_confidence=None, survival_threshold=0.0):
    """Best-first verification tree from per-depth candidates.  A few dozen nodes per sequence: assembled on the host from the
    candidate lists (one small device→host copy), results returned on the candidates' device."""
    return ref.ddtree_assemble(cand_ids, cand_lp, root_tokens, num_nodes, depth_confidence, survival_threshold)
