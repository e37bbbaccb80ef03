"""``trtedge process-lora --input_dir … --output_dir …``: PEFT adapter → runtime adapter file."""
import argparse
import json
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge process-lora")
    p.add_argument("--input_dir", "--input-dir", required=True)
    p.add_argument("--output_dir", "--output-dir", required=True)
    p.add_argument("--dtype", default="float16", choices=["float16", "bfloat16"])
    a = p.parse_args(argv)
    import torch
    from ..lora import process_lora_weights
    print(json.dumps(process_lora_weights(a.input_dir, a.output_dir, getattr(torch, a.dtype))))
    return 0


if __name__ == "__main__":
    sys.exit(main())
