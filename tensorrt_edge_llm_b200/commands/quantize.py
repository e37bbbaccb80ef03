"""``trtedge quantize llm --model_dir … --output_dir … --quantization nvfp4`` (``tensorrt_edgellm/scripts/quantize.py``)."""
import argparse
import json
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge quantize")
    p.add_argument("kind", nargs="?", default="llm", choices=["llm", "draft"])
    p.add_argument("--model_dir", "--model-dir", required=True)
    p.add_argument("--output_dir", "--output-dir", required=True)
    p.add_argument("--quantization", default="nvfp4", choices=["nvfp4", "int4_awq", "int4_gptq", "fp8", "int8_sq", "mxfp8", "q8_0"])
    p.add_argument("--kv-cache-quantization", "--kv_cache_quantization", default=None, choices=[None, "fp8"])
    p.add_argument("--exclude", nargs="*", default=["lm_head"])
    p.add_argument("--calib-ids", default="", help="JSON file with a list of token-id lists; default: seeded uniform ids")
    p.add_argument("--no-calibration", action="store_true")
    p.add_argument("--group-size", type=int, default=128)
    p.add_argument("--device", default="cpu")
    a = p.parse_args(argv)
    import torch
    from ..quantization import quantize_and_export
    ids = None
    if a.calib_ids:
        with open(a.calib_ids, "r", encoding="utf-8") as f:
            rows = json.load(f)
        n = min(len(r) for r in rows)
        ids = torch.tensor([r[:n] for r in rows])
    r = quantize_and_export(a.model_dir, a.output_dir, a.quantization, a.exclude, a.kv_cache_quantization, ids, not a.no_calibration,
                            a.device, a.group_size)
    print(json.dumps({"output_dir": a.output_dir, **{k: v for k, v in r.items() if k != "config"}}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
