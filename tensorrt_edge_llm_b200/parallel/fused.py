"""Communicator whose hot entries run fused peer-memory kernels.

``add_rmsnorm`` — the all-reduce after every row-parallel projection — is a single kernel at
decode size: each rank publishes its partial rows in symmetric memory and reads its peers'
rows over NVLink inside the kernel that also adds the residual, normalises and (for NVFP4
layers) quantises the next GEMM's input (``csrc/kernels/comm_fused.cu``).  Larger messages
(prefill) and the remaining collectives go through NCCL.

The symmetric buffers come from ``torch.distributed._symmetric_memory`` (allocation + handle
exchange only); all data movement on them is done by this package's own kernels.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch

from .. import ops
from .comm import TorchComm

MAX_ROWS = 256


class RsPartial:
    """Marker for a row-parallel projection whose partial rows were stored into their owners'
    symmetric buffers by the GEMM epilogue; only ``add_rmsnorm`` can consume it."""

    __slots__ = ("rows", "hidden", "dtype", "rows_per_rank", "sum_slots", "slot_base")
    is_cuda = True

    def __init__(self, rows, hidden, dtype, rows_per_rank, sum_slots=0, slot_base=0):
        self.rows, self.hidden, self.dtype, self.rows_per_rank = rows, hidden, dtype, rows_per_rank
        # 0 = every rank's slot holds a partial sum; (1, rank) = this rank's slot already holds complete rows
        self.sum_slots, self.slot_base = sum_slots, slot_base

    @property
    def shape(self):
        return (self.rows, self.hidden)


class _RsState:
    """Symmetric buffers of the reduce-scatter / all-gather path for one hidden size."""

    def __init__(self, device, hidden: int, dtype: torch.dtype, group, max_tokens: int, cu):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        gname = group.group_name if group is not None else dist.group.WORLD.group_name
        world = dist.get_world_size(group)
        self.cap = max_tokens + world
        L = cu.lib()
        L.telb_nvfp4_sf_bytes.restype = ctypes.c_longlong
        sf_bytes = int(L.telb_nvfp4_sf_bytes(ctypes.c_longlong(self.cap), ctypes.c_int(hidden)))
        self.partial = symm_mem.empty(self.cap * hidden, dtype=dtype, device=device)
        self.gather_y = symm_mem.empty(self.cap * hidden, dtype=dtype, device=device)
        self.gather_xq = symm_mem.empty(self.cap * hidden // 2, dtype=torch.uint8, device=device)
        self.gather_sf = symm_mem.empty(sf_bytes, dtype=torch.uint8, device=device)
        self.flags = symm_mem.empty(16, dtype=torch.int32, device=device)       # [0:8] GEMM finished, [8:16] shard gathered
        self.flags.zero_()
        self.gather_sf.zero_()
        hs = {n: symm_mem.rendezvous(getattr(self, n), gname) for n in ("partial", "gather_y", "gather_xq", "gather_sf", "flags")}
        self._handles = hs

        def table(name, offset_bytes=0):
            return (ctypes.c_void_p * world)(*[int(p) + offset_bytes for p in hs[name].buffer_ptrs])

        self.c_partial, self.c_gather_y = table("partial"), table("gather_y")
        self.c_gather_xq, self.c_gather_sf = table("gather_xq"), table("gather_sf")
        self.c_gemm_flags, self.c_ag_flags = table("flags"), table("flags", 32)
        self.partial_ptrs = [int(p) for p in hs["partial"].buffer_ptrs]
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)


class _EpState:
    """Symmetric buffers of the expert-parallel all-to-all for one (hidden, dtype, top_k)."""

    def __init__(self, device, hidden: int, dtype: torch.dtype, group, tokens_local_cap: int, top_k: int):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        gname = group.group_name if group is not None else dist.group.WORLD.group_name
        world = dist.get_world_size(group)
        self.slots_cap = tokens_local_cap * top_k
        self.recv_rows = symm_mem.empty(world * self.slots_cap * hidden, dtype=dtype, device=device)
        self.recv_ids = symm_mem.empty(world * self.slots_cap, dtype=torch.int32, device=device)
        self.comb_rows = symm_mem.empty(self.slots_cap * hidden, dtype=dtype, device=device)
        self.flags = symm_mem.empty(16, dtype=torch.int32, device=device)
        self.recv_ids.fill_(-1)
        self.flags.zero_()
        hs = {n: symm_mem.rendezvous(getattr(self, n), gname) for n in ("recv_rows", "recv_ids", "comb_rows", "flags")}
        self._handles = hs
        self.c = {n: (ctypes.c_void_p * world)(*[int(p) for p in hs[n].buffer_ptrs]) for n in hs}
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)        # dispatch, return
        self.ticket = torch.zeros(2, dtype=torch.int32, device=device)
        self.arange = torch.arange(self.slots_cap, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)


class _Rows:
    """Minimal stand-in for a routing workspace: slot s reads row s."""

    def __init__(self, dst_row):
        self.dst_row = dst_row


class _SymState:
    def __init__(self, device, hidden: int, dtype: torch.dtype, group):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        self.hidden, self.dtype = hidden, dtype
        self.partial = symm_mem.empty(2 * MAX_ROWS * hidden, dtype=dtype, device=device)
        self.flags = symm_mem.empty(2 * 8 * MAX_ROWS, dtype=torch.int32, device=device)
        self.flags.zero_()
        self.partial.zero_()
        gname = group.group_name if group is not None else dist.group.WORLD.group_name
        self.h_partial = symm_mem.rendezvous(self.partial, gname)
        self.h_flags = symm_mem.rendezvous(self.flags, gname)
        self.row_epoch = torch.zeros(MAX_ROWS, dtype=torch.int32, device=device)
        world = self.h_partial.world_size
        self.c_partial = (ctypes.c_void_p * world)(*[int(p) for p in self.h_partial.buffer_ptrs])
        self.c_flags = (ctypes.c_void_p * world)(*[int(p) for p in self.h_flags.buffer_ptrs])
        torch.cuda.synchronize(device)
        dist.barrier(group)


class _ArgmaxState:
    """Symmetric candidate tables of the vocabulary-sharded greedy pick: ``[2][8][MAX_ARGMAX_ROWS]`` 64-bit keys and
    ``[2][8]`` epoch flags per rank."""

    def __init__(self, device, group):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem
        gname = group.group_name if group is not None else dist.group.WORLD.group_name
        world = dist.get_world_size(group)
        self.keys = symm_mem.empty(2 * 8 * MAX_ARGMAX_ROWS, dtype=torch.int64, device=device)
        self.flags = symm_mem.empty(16, dtype=torch.int32, device=device)
        self.keys.zero_()
        self.flags.zero_()
        hk, hf = symm_mem.rendezvous(self.keys, gname), symm_mem.rendezvous(self.flags, gname)
        self._handles = (hk, hf)
        self.c_keys = (ctypes.c_void_p * world)(*[int(p) for p in hk.buffer_ptrs])
        self.c_flags = (ctypes.c_void_p * world)(*[int(p) for p in hf.buffer_ptrs])
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)


MAX_ARGMAX_ROWS = 1024


def _default_rs_min_rows(world: int) -> int:
    """Smallest step (rows) of a dense layer that takes the reduce-scatter → norm → all-gather path instead of the one-shot
    all-reduce.  The one-shot form is a single hop but moves ``(world - 1) x rows x hidden`` 16-bit values into every GPU; the
    sharded form moves 1/world of that plus the quantised rows over two hops.  Measured on the Qwen3-8B shape at 64 rows per
    step: one-shot 3.99 / 3.61 / 3.98 ms per decode step on 2 / 4 / 8 GPUs against 4.49 / 4.02 / 3.70 ms sharded, so up to
    four ranks decode-size steps (at most 128 rows) stay one-shot and eight ranks shard from 16 rows up.
    ``TELB_RS_MIN_ROWS`` overrides."""
    import os
    env = int(os.environ.get("TELB_RS_MIN_ROWS", "0"))
    if env > 0:
        return env
    return 129 if world <= 4 else max(16, 2 * world)


class FusedComm(TorchComm):
    def __init__(self, device=None, group=None, rs_max_tokens: int = 8192, rs_min_rows: Optional[int] = None):
        super().__init__(group)
        if rs_min_rows is None:
            rs_min_rows = _default_rs_min_rows(self.world_size)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._sym: Dict[Tuple[int, torch.dtype], _SymState] = {}
        self._rs: Dict[Tuple[int, torch.dtype], _RsState] = {}
        self._ep: Dict[Tuple[int, torch.dtype, int], _EpState] = {}
        self.rs_max_tokens = rs_max_tokens
        self.rs_min_rows = rs_min_rows          # below this the one-shot all-reduce is faster
        # expert parallelism: steps of at least this many rows ship token rows all-to-all; smaller ones run the local experts on
        # every row and reduce the partial sums (its own threshold: the dense layers' one does not describe the all-to-all)
        self.ep_min_rows = max(16, 2 * self.world_size)
        self.rs_enabled = True
        self.rs_single_rank = False             # tests: run the fused path on one rank too
        self.force_nccl = False                 # benchmarks: every entry falls back to the NCCL composition
        self._argmax: Optional[_ArgmaxState] = None

    # ---- prefill path: GEMM → reduce-scatter epilogue, norm, all-gather → GEMM prologue -----------
    def use_rs(self, rows: int) -> bool:
        return (self.rs_enabled and not self.force_nccl and (self.world_size > 1 or self.rs_single_rank)
                and self.rs_min_rows <= rows <= self.rs_max_tokens)

    def use_ep_all_to_all(self, rows: int) -> bool:
        return (self.rs_enabled and not self.force_nccl and (self.world_size > 1 or self.rs_single_rank)
                and self.ep_min_rows <= rows <= self.rs_max_tokens)

    def _rs_state(self, hidden: int, dtype: torch.dtype) -> _RsState:
        key = (hidden, dtype)
        st = self._rs.get(key)
        if st is None:
            st = self._rs[key] = _RsState(self.device, hidden, dtype, self.group, self.rs_max_tokens, ops.cuda_ops())
        return st

    def prepare_rs(self, hidden: int, dtype: torch.dtype) -> None:
        """Allocate and exchange the reduce-scatter / all-gather buffers up front (collective)."""
        self._rs_state(hidden, dtype)

    def gemm_reduce_scatter(self, linear, x) -> RsPartial:
        """Row-parallel projection whose epilogue stores each output row into its owner's partial
        buffer over peer memory (``x`` 16-bit or NVFP4 ``QuantActs``)."""
        cu = ops.cuda_ops()
        rows = x.shape[0]
        dtype = x.dtype
        st = self._rs_state(linear.out_features, dtype)
        rpr = (rows + self.world_size - 1) // self.world_size
        f = cu.GemmFusion()
        for r in range(self.world_size):
            f.rs_out[r] = st.partial_ptrs[r]
        f.rs_world = max(self.world_size, 2) if self.world_size == 1 else self.world_size
        f.rs_rank, f.rs_rows_per_rank = self.rank, rpr
        if self.world_size == 1:                 # single-rank test mode: "scatter" into the local buffer
            f.rs_out[1] = st.partial_ptrs[0]
            f.rs_rows_per_rank = rpr = rows
        ag = getattr(x, "ag_wait", None)
        if ag is not None:
            f.ag_flags, f.ag_epoch, f.ag_world, f.ag_rows_per_rank = ag.ag_flags, ag.ag_epoch, ag.ag_world, ag.ag_rows_per_rank
        if hasattr(linear, "_gpu_weight_sf"):    # NVFP4: quantise 16-bit activations first
            if not isinstance(x, cu.QuantActs):
                x2 = x.reshape(-1, x.shape[-1])
                xq, sf = cu.nvfp4_quantize(x2, linear.input_scale)
                x = cu.QuantActs(xq, sf, x2.shape, dtype)
            cu.gemm_fused(x, linear.weight, f, w_sf=linear._gpu_weight_sf, alpha=linear.alpha, bias=linear.bias)
        else:
            cu.gemm_fused(x.reshape(-1, x.shape[-1]).contiguous(), linear.weight, f, bias=linear.bias)
        return RsPartial(rows, linear.out_features, dtype, rpr)

    # ---- expert parallelism: all-to-all dispatch → grouped expert GEMMs → all-to-all return → weighted combine ----
    def _ep_state(self, hidden: int, dtype: torch.dtype, top_k: int) -> _EpState:
        key = (hidden, dtype, top_k)
        st = self._ep.get(key)
        if st is None:
            cap = (self.rs_max_tokens + self.world_size - 1) // self.world_size
            st = self._ep[key] = _EpState(self.device, hidden, dtype, self.group, cap, top_k)
        return st

    def moe_all_to_all(self, block, x: torch.Tensor) -> RsPartial:
        """Expert-parallel MoE over token shards.  ``x`` holds all rows (gathered); this rank routes its own
        shard, ships every (token, k) row to the rank that owns the expert (peer stores), runs its local experts on
        what it received, ships the results back and reduces its tokens' top-k rows with the router weights.
        The result is this rank's complete rows, handed to ``add_rmsnorm`` as an already-reduced shard."""
        cu = ops.cuda_ops()
        rows, hidden = x.shape
        world, rank = self.world_size, self.rank
        rpr = (rows + world - 1) // world
        lo, hi = min(rows, rank * rpr), min(rows, (rank + 1) * rpr)
        t_local = hi - lo
        st = self._ep_state(hidden, x.dtype, block.top_k)
        rs = self._rs_state(hidden, x.dtype)
        ws0 = cu.Workspace.get(self.device)
        xs = x[lo:hi].contiguous()
        logits = block.gate(xs)
        w, idx = cu.moe_route_softmax_topk(logits, block.top_k, block.cfg.norm_topk_prob)
        epr = block.num_experts // world
        c = st.c
        # the slot stride follows the step (every rank derives it from the global row count), so a decode step touches a few
        # hundred slots instead of the buffers' prefill-size capacity
        stride = max(1, rpr * block.top_k)
        if stride > st.slots_cap:
            raise ValueError(f"{rows} rows exceed the expert all-to-all capacity of {st.slots_cap // block.top_k * world} rows")
        cu._check(cu.lib().telb_ep_dispatch(cu._p(xs), cu._p(idx), c["recv_rows"], c["recv_ids"], c["comb_rows"], c["flags"], ctypes.c_int(rank),
                                            ctypes.c_int(world), ctypes.c_int(t_local), ctypes.c_int(block.top_k), ctypes.c_int(hidden),
                                            ctypes.c_int(epr), ctypes.c_int(stride),
                                            ctypes.c_void_p(st.epoch.data_ptr()), ctypes.c_void_p(st.ticket.data_ptr()), cu._stream()),
                  "ep_dispatch")
        cu._check(cu.lib().telb_ep_wait(cu._p(st.flags), ctypes.c_int(0), ctypes.c_int(world), ctypes.c_void_p(st.epoch.data_ptr()),
                                        cu._p(ws0.status), cu._stream()), "ep_wait")
        n_recv = world * stride
        ws = cu.moe_align(st.recv_ids.view(-1)[:n_recv].view(n_recv, 1), block.e_local, 0, block.e_local)
        recv = st.recv_rows.view(-1)[:n_recv * hidden].view(n_recv, hidden)
        if block.nvfp4:
            if block._w13_sf is None:
                block.finalize()
            a = cu.moe_gather(recv, ws, 1, block.input_scale)
            y = cu.gemm_grouped(block.expert_fc1(a, ws), block.w2, ws, block.e_local, alpha=block.w2_alpha, w_sf=block._w2_sf)
        else:
            a = cu.moe_gather(recv, ws, 1, None)
            y = cu.gemm_grouped(cu.swiglu(cu.gemm_grouped(a, block.w13, ws, block.e_local)), block.w2, ws, block.e_local)
        cu._check(cu.lib().telb_ep_return(cu._p(y), cu._p(ws.dst_row), c["recv_rows"], c["recv_ids"], c["comb_rows"], c["flags"],
                                          ctypes.c_int(rank), ctypes.c_int(world), ctypes.c_int(stride), ctypes.c_int(hidden),
                                          ctypes.c_void_p(st.epoch.data_ptr() + 4), ctypes.c_void_p(st.ticket.data_ptr() + 4), cu._stream()),
                  "ep_return")
        cu._check(cu.lib().telb_ep_wait(cu._p(st.flags), ctypes.c_int(1), ctypes.c_int(world), ctypes.c_void_p(st.epoch.data_ptr() + 4),
                                        cu._p(ws0.status), cu._stream()), "ep_wait")
        out = rs.partial[rank * rpr * hidden:(rank * rpr + t_local) * hidden].view(t_local, hidden)
        if t_local > 0:
            cu.moe_combine(st.comb_rows.view(-1)[:stride * hidden].view(stride, hidden), _Rows(st.arange), w, out=out)
        return RsPartial(rows, hidden, x.dtype, rpr, sum_slots=1, slot_base=rank)

    def _rs_add_rmsnorm(self, part: RsPartial, residual, weight, eps, quant_scale, defer_gather):
        cu = ops.cuda_ops()
        st = self._rs_state(part.hidden, part.dtype)
        rows, hidden, rpr = part.rows, part.hidden, part.rows_per_rank
        rows_local = max(0, min(rpr, rows - self.rank * rpr))
        res_out = torch.empty(rows_local, hidden, dtype=part.dtype, device=self.device)
        full = 1 if (residual is not None and residual.shape[0] == rows and (rows_local != rows or self.world_size == 1)) else 0
        ws = cu.Workspace.get(self.device)
        quant = quant_scale is not None
        cu._check(cu.lib().telb_rs_add_rmsnorm_ag(
            cu._p(st.partial), st.c_gemm_flags, st.c_ag_flags, cu._p(st.epoch), cu._p(st.ticket), cu._p(residual), ctypes.c_int(full),
            cu._p(weight), cu._p(res_out), None if quant else st.c_gather_y, st.c_gather_xq if quant else None,
            st.c_gather_sf if quant else None, cu._p(quant_scale), ctypes.c_int(self.rank), ctypes.c_int(self.world_size),
            ctypes.c_int(rows), ctypes.c_int(rpr), ctypes.c_int(hidden), ctypes.c_float(eps), ctypes.c_int(0 if defer_gather else 1),
            ctypes.c_int(cu._is_bf16(res_out)), cu._p(ws.status), ctypes.c_int(part.sum_slots), ctypes.c_int(part.slot_base),
            cu._stream()), "rs_add_rmsnorm_ag")
        wait = None
        if defer_gather and self.world_size > 1:
            wait = cu.GemmFusion()
            wait.ag_flags = st.flags.data_ptr() + 32
            wait.ag_epoch = st.epoch.data_ptr()
            wait.ag_world, wait.ag_rows_per_rank = self.world_size, rpr
        if quant:
            y = cu.QuantActs(st.gather_xq[:rows * hidden // 2].view(rows, hidden // 2), st.gather_sf, (rows, hidden), part.dtype)
            y.ag_wait = wait
        else:
            y = st.gather_y[:rows * hidden].view(rows, hidden)
            if wait is not None:
                y.ag_wait = wait
        return y, res_out

    def _state(self, hidden: int, dtype: torch.dtype) -> _SymState:
        key = (hidden, dtype)
        st = self._sym.get(key)
        if st is None:
            st = self._sym[key] = _SymState(self.device, hidden, dtype, self.group)
        return st

    def prepare(self, hidden: int, dtype: torch.dtype) -> None:
        """Allocate and exchange the symmetric buffers up front (collective; call before capture)."""
        self._state(hidden, dtype)

    def add_rmsnorm(self, x_partial, residual, weight, eps, quant_scale=None, defer_gather=False):
        if isinstance(x_partial, RsPartial):
            return self._rs_add_rmsnorm(x_partial, residual, weight, eps, quant_scale, defer_gather)
        rows, hidden = x_partial.shape
        if not x_partial.is_cuda or rows > MAX_ROWS or hidden % 16 or self.force_nccl:
            return super().add_rmsnorm(x_partial, residual, weight, eps, quant_scale)
        cu = ops.cuda_ops()
        st = self._state(hidden, x_partial.dtype)
        x_partial = x_partial.contiguous()
        res_out = torch.empty_like(x_partial)
        y = xq = sf = None
        if quant_scale is not None:
            L = cu.lib()
            L.telb_nvfp4_sf_bytes.restype = ctypes.c_longlong
            nbytes = L.telb_nvfp4_sf_bytes(ctypes.c_longlong(rows), ctypes.c_int(hidden))
            xq = torch.empty(rows, hidden // 2, dtype=torch.uint8, device=x_partial.device)
            sf = cu._sf_buffer(nbytes, hidden, x_partial.device)
        else:
            y = torch.empty_like(x_partial)
        ws = cu.Workspace.get(x_partial.device)
        cu._check(cu.lib().telb_ar_add_rmsnorm(
            cu._p(x_partial), st.c_partial, st.c_flags, cu._p(st.row_epoch), cu._p(residual), cu._p(weight), cu._p(res_out),
            cu._p(y), cu._p(xq), cu._p(sf), cu._p(quant_scale), ctypes.c_int(self.rank), ctypes.c_int(self.world_size),
            ctypes.c_int(rows), ctypes.c_int(hidden), ctypes.c_int(MAX_ROWS), ctypes.c_float(eps),
            ctypes.c_int(cu._is_bf16(x_partial)), cu._p(ws.status), cu._stream()), "ar_add_rmsnorm")
        if quant_scale is not None:
            return cu.QuantActs(xq, sf, (rows, hidden), x_partial.dtype), res_out
        return y, res_out

    def prepare_argmax(self) -> None:
        """Allocate and exchange the candidate tables up front (collective; call before capture)."""
        if self._argmax is None:
            self._argmax = _ArgmaxState(self.device, self.group)

    def argmax_sharded(self, logits_local: torch.Tensor) -> torch.Tensor:
        rows, vloc = logits_local.shape
        if not logits_local.is_cuda or rows > MAX_ARGMAX_ROWS or self.force_nccl or logits_local.stride(1) != 1:
            return super().argmax_sharded(logits_local)
        cu = ops.cuda_ops()
        self.prepare_argmax()
        st = self._argmax
        local = cu.argmax(logits_local)
        out = torch.empty(rows, dtype=torch.int32, device=logits_local.device)
        ws = cu.Workspace.get(logits_local.device)
        dt = 2 if logits_local.dtype == torch.float32 else cu._is_bf16(logits_local)
        cu._check(cu.lib().telb_argmax_merge(
            cu._p(logits_local), ctypes.c_longlong(logits_local.stride(0)), cu._p(local), st.c_keys, st.c_flags, cu._p(st.epoch), cu._p(out),
            ctypes.c_int(self.rank), ctypes.c_int(self.world_size), ctypes.c_int(rows), ctypes.c_int(MAX_ARGMAX_ROWS), ctypes.c_int(vloc),
            ctypes.c_int(dt), cu._p(ws.status), cu._stream()), "argmax_merge")
        return out
