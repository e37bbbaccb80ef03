"""Speculative decoding with random weights: an EAGLE-3 tree draft and a DFlash block draft on the same target.

`python examples/speculative_decoding.py` prints the mean number of tokens each verification round produced."""
from tensorrt_edge_llm_b200.config import tiny_llama_config
from tensorrt_edge_llm_b200.runtime.llm import LLM, SamplingParams


def main():
    target = tiny_llama_config(num_hidden_layers=4, vocab_size=512)
    prompts = [[3, 1, 4, 1, 5, 9, 2, 6], [2, 7, 1, 8, 2, 8]]
    eagle = tiny_llama_config(num_hidden_layers=1, vocab_size=512)
    eagle.draft_type = "eagle3"
    dflash = tiny_llama_config(num_hidden_layers=2, vocab_size=512)
    dflash.draft_type, dflash.dflash_block_size, dflash.dflash_mask_token_id = "dflash", 8, 511
    plain = LLM(target, max_batch_size=2, page_size=64).generate(prompts, SamplingParams(max_tokens=48, ignore_eos=True))
    for name, draft in (("eagle3", eagle), ("dflash", dflash)):
        llm = LLM(target, max_batch_size=2, page_size=64, draft_model=draft)
        outs = llm.generate(prompts, SamplingParams(max_tokens=48, ignore_eos=True))
        same = all(a.token_ids == b.token_ids for a, b in zip(outs, plain))
        print(name, "lossless" if same else "differs (bf16 near-ties)", outs[0].spec_stats)


if __name__ == "__main__":
    main()
