"""``trtedge merge-lora --model_dir … --lora_dir … --output_dir …``."""
import argparse
import json
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge merge-lora")
    p.add_argument("--model_dir", "--model-dir", required=True)
    p.add_argument("--lora_dir", "--lora-dir", required=True)
    p.add_argument("--output_dir", "--output-dir", required=True)
    a = p.parse_args(argv)
    from ..lora import merge_lora
    print(json.dumps(merge_lora(a.model_dir, a.lora_dir, a.output_dir)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
