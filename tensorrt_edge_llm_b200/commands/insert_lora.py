"""``trtedge insert-lora``: in the reference this rewrites an ONNX graph so engines expose LoRA inputs.
Here adapters bind at run time, so the command only reports where an adapter would attach."""
import argparse
import json
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge insert-lora")
    p.add_argument("--lora_dir", "--lora-dir", required=True)
    a = p.parse_args(argv)
    from ..lora import lora_target_modules
    print(json.dumps({"modules": lora_target_modules(a.lora_dir), "note": "no graph rewrite needed: adapters bind at run time"}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
