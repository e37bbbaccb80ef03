"""Tensor / expert parallel plumbing: communicators, symmetric peer memory, fused collectives."""
from .comm import LocalComm, TorchComm


def make_comm(kind: str, device=None):
    """``"nccl"`` → collectives through torch.distributed only (the baseline composition);
    ``"fused"`` → peer-memory kernels for the hot paths, NCCL for the rest."""
    if kind == "nccl":
        return TorchComm()
    from .fused import FusedComm
    return FusedComm(device)


__all__ = ["LocalComm", "TorchComm", "make_comm"]
