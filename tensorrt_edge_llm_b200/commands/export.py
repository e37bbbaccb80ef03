"""``trtedge export``: optional ONNX dump of a checkpoint's decoder for interoperability.  The execution
path never needs it (``tensorrt_edgellm/onnx/`` is the reference's route into TensorRT)."""
import argparse
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge export")
    p.add_argument("model_dir")
    p.add_argument("--output", required=True)
    a = p.parse_args(argv)
    from .. import AutoModel, export_onnx
    export_onnx(AutoModel.from_pretrained(a.model_dir), a.output)
    return 0


if __name__ == "__main__":
    sys.exit(main())
