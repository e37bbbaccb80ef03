"""Offline generation: `python examples/offline_inference.py /path/to/checkpoint "Hello"` (random weights without a path).

Run from the repository root (or with the package on PYTHONPATH)."""
import sys

from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams


def main():
    if len(sys.argv) > 1:
        from tensorrt_edge_llm_b200.runtime import native as rt
        model = sys.argv[1]
        tok = rt.Tokenizer.load_from_hf(model)
        llm = LLM(model, tokenizer=tok, max_batch_size=8, enable_in_flight_batching=True, enable_prefix_cache=True)
        prompts = sys.argv[2:] or ["Hello"]
    else:
        llm = LLM(tiny_llama_config(num_hidden_layers=2, vocab_size=256), max_batch_size=4, page_size=64)
        prompts = [[1, 2, 3, 4], [5, 6, 7]]
    for out in llm.generate(prompts, SamplingParams(max_tokens=32, temperature=0.7, top_p=0.9, seed=1)):
        print(out.text if out.text is not None else out.token_ids, f"[{out.finish_reason}]")
    llm.close()


if __name__ == "__main__":
    main()
