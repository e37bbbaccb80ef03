"""Communicators: the seam between model code and collectives.

``LocalComm``   one rank; every collective is the identity and ``add_rmsnorm`` is the local kernel.
``TorchComm``   ``torch.distributed`` process group (NCCL on GPUs, gloo on CPU): the *baseline*
                composition "collective, then kernel" that the fused kernels are measured against,
                and the CPU multi-process test path.
``FusedComm``   (``parallel/fused.py``) symmetric peer memory + in-kernel P2P / multimem
                reductions; it derives from ``TorchComm`` and overrides the hot entries.

Parity: ``cpp/runtime/multiDevice/collectiveGroup.{h,cpp}`` (broadcastInt32 / allGather /
allReduceSum) and ``cpp/plugins/allReducePlugin/allReducePlugin.cpp:64-110`` (identity when
tp_size ≤ 1, else ncclAllReduce).  The reference has no reduce-scatter or all-to-all.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .. import ops


class LocalComm:
    world_size = 1
    rank = 0

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def all_gather_cols(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def all_gather_rows(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def reduce_scatter_rows(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def broadcast_tokens(self, ids: torch.Tensor, src: int = 0) -> torch.Tensor:
        return ids

    def all_to_all(self, send: torch.Tensor, send_counts: List[int], recv_counts: List[int]) -> torch.Tensor:
        return send

    def add_rmsnorm(self, x_partial, residual, weight, eps, quant_scale=None, defer_gather=False) -> Tuple[torch.Tensor, torch.Tensor]:
        """``defer_gather`` is a hint that the normalised output feeds exactly one GEMM, which may then
        wait for the gathered rows itself; communicators without a fused gather ignore it."""
        return ops.add_rmsnorm(x_partial, residual, weight, eps, quant_scale)

    def barrier(self) -> None:
        pass


class TorchComm(LocalComm):
    """Collectives through ``torch.distributed`` (NCCL / gloo)."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world_size = dist.get_world_size(group)
        self.rank = dist.get_rank(group)

    def all_reduce(self, x):
        if x.dtype == torch.bfloat16 and not x.is_cuda:       # gloo has no bf16 sum
            y = x.float()
            self.dist.all_reduce(y, group=self.group)
            return y.to(x.dtype)
        self.dist.all_reduce(x, group=self.group)
        return x

    def all_gather_cols(self, x):
        parts = [torch.empty_like(x) for _ in range(self.world_size)]
        self.dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def all_gather_rows(self, x):
        parts = [torch.empty_like(x) for _ in range(self.world_size)]
        self.dist.all_gather(parts, x.contiguous(), group=self.group)
        return torch.cat(parts, dim=0)

    def reduce_scatter_rows(self, x):
        rows = x.shape[0] // self.world_size
        if not x.is_cuda:                                      # gloo: emulate with all-reduce
            y = self.all_reduce(x.clone())
            return y[self.rank * rows:(self.rank + 1) * rows].contiguous()
        out = torch.empty(rows, *x.shape[1:], dtype=x.dtype, device=x.device)
        self.dist.reduce_scatter_tensor(out, x.contiguous(), group=self.group)
        return out

    def broadcast_tokens(self, ids, src=0):
        self.dist.broadcast(ids, src=src, group=self.group)
        return ids

    def all_to_all(self, send, send_counts, recv_counts):
        out = torch.empty(sum(recv_counts), *send.shape[1:], dtype=send.dtype, device=send.device)
        if not send.is_cuda:                                   # gloo lacks all_to_all_single on some builds
            gathered: List[Optional[list]] = [None] * self.world_size
            offs = [0]
            for c in send_counts:
                offs.append(offs[-1] + c)
            chunks = [send[offs[i]:offs[i + 1]].clone() for i in range(self.world_size)]
            self.dist.all_gather_object(gathered, chunks, group=self.group)
            return torch.cat([gathered[src][self.rank] for src in range(self.world_size)], dim=0)
        self.dist.all_to_all_single(out, send.contiguous(), recv_counts, send_counts, group=self.group)
        return out

    def add_rmsnorm(self, x_partial, residual, weight, eps, quant_scale=None, defer_gather=False):
        return ops.add_rmsnorm(self.all_reduce(x_partial), residual, weight, eps, quant_scale)

    def argmax_sharded(self, logits_local: torch.Tensor) -> torch.Tensor:
        """Greedy token per row from vocabulary-sharded logits ``[rows, vocab / world]`` (rank r holds columns
        ``[r * vocab / world, ...)``): every rank contributes its best (value, global id) per row, the largest value
        wins and the lowest id among equals — the arg-max of the gathered logits without gathering them."""
        vloc = logits_local.shape[1]
        lf = logits_local.float()
        vals = lf.max(dim=-1).values
        # the first maximum of the shard (torch.max does not promise which of several equal maxima it reports)
        ids = ((lf == vals[:, None]).to(torch.int32).argmax(dim=-1) + self.rank * vloc).to(torch.int64)
        parts_v = [torch.empty_like(vals) for _ in range(self.world_size)]
        parts_i = [torch.empty_like(ids) for _ in range(self.world_size)]
        self.dist.all_gather(parts_v, vals.contiguous(), group=self.group)
        self.dist.all_gather(parts_i, ids.contiguous(), group=self.group)
        v, i = torch.stack(parts_v), torch.stack(parts_i)            # [world, rows]
        best = v.max(dim=0).values
        masked = torch.where(v == best[None, :], i, torch.full_like(i, torch.iinfo(torch.int64).max))
        return masked.min(dim=0).values.to(torch.int32)

    def barrier(self):
        self.dist.barrier(group=self.group)
