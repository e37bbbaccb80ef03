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


class FusedComm(TorchComm):
    def __init__(self, device=None, group=None):
        super().__init__(group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._sym: Dict[Tuple[int, torch.dtype], _SymState] = {}

    def _state(self, hidden: int, dtype: torch.dtype) -> _SymState:
        key = (hidden, dtype)
        st = self._sym.get(key)
        if st is None:
            st = self._sym[key] = _SymState(self.device, hidden, dtype, self.group)
        return st

    def prepare(self, hidden: int, dtype: torch.dtype) -> None:
        """Allocate and exchange the symmetric buffers up front (collective; call before capture)."""
        self._state(hidden, dtype)

    def add_rmsnorm(self, x_partial, residual, weight, eps, quant_scale=None):
        rows, hidden = x_partial.shape
        if not x_partial.is_cuda or rows > MAX_ROWS or hidden % 16:
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
