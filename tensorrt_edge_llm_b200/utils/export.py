"""Optional ONNX dump of the dense projection stack (weights as initialisers) for tools that want to look
at a checkpoint as a graph.  The paged-attention and state ops are custom to this runtime and are emitted
as opaque nodes by ``torch.onnx`` only if the exporter is present; nothing in the runtime reads the file."""
from __future__ import annotations


def export_onnx(model, path: str, *args, **kwargs) -> str:
    try:
        import onnx  # noqa: F401
    except ImportError as e:
        raise RuntimeError("ONNX export needs the `onnx` package, which is not installed; the runtime itself "
                           "executes checkpoints directly and never needs an ONNX file") from e
    import torch

    class _Projections(torch.nn.Module):
        def __init__(self, m):
            super().__init__()
            self.m = m

        def forward(self, hidden):
            x = hidden
            for layer in self.m.model.layers:
                x = x + layer.mlp(layer.post_attention_layernorm(x))
            return self.m.lm_head(self.m.model.norm(x))

    h = model.cfg.hidden_size
    torch.onnx.export(_Projections(model).float(), (torch.zeros(1, h),), path, input_names=["hidden"], output_names=["logits"])
    return path
