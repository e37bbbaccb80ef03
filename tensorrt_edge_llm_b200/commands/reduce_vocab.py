"""``trtedge reduce-vocab --model_dir … --output_dir … --keep N [--corpus-ids file.json]``."""
import argparse
import json
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge reduce-vocab")
    p.add_argument("--model_dir", "--model-dir", required=True)
    p.add_argument("--output_dir", "--output-dir", required=True)
    p.add_argument("--keep", type=int, required=True, help="number of vocabulary entries to keep")
    p.add_argument("--corpus-ids", default="", help="JSON file with token-id lists used to rank tokens by frequency")
    p.add_argument("--always-keep", type=int, nargs="*", default=[])
    a = p.parse_args(argv)
    from ..config import load_config_dict
    from ..vocab_reduction import build_vocab_map, count_tokens, reduce_vocab
    hf = load_config_dict(a.model_dir)
    vocab = int(hf.get("text_config", hf)["vocab_size"])
    counts = None
    if a.corpus_ids:
        with open(a.corpus_ids, "r", encoding="utf-8") as f:
            counts = count_tokens(json.load(f), vocab)
    special = [t for t in (hf.get("bos_token_id"), hf.get("eos_token_id")) if isinstance(t, int)]
    vm = build_vocab_map(vocab, counts, a.keep, list(a.always_keep) + special)
    print(json.dumps(reduce_vocab(a.model_dir, a.output_dir, vm)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
