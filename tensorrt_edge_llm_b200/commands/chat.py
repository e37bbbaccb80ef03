"""``trtedge chat <checkpoint>``: terminal chat with a local checkpoint (``experimental/frontend`` in the reference)."""
import argparse
import os
import sys


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trtedge chat")
    p.add_argument("model_dir")
    p.add_argument("--max-tokens", type=int, default=256)
    p.add_argument("--temperature", type=float, default=0.7)
    p.add_argument("--system", default="")
    p.add_argument("--prompt", default="", help="answer this one prompt and exit")
    a = p.parse_args(argv)
    from ..chat_template import ChatTemplate
    from ..runtime import native as rt
    from ..runtime.llm import LLM
    from ..runtime.runner import SamplingParams
    tok = rt.Tokenizer.load_from_hf(a.model_dir)
    llm = LLM(a.model_dir, max_batch_size=1, tokenizer=tok, enable_in_flight_batching=True)
    template = ChatTemplate.load(a.model_dir)
    history = [{"role": "system", "content": a.system}] if a.system else []
    sp = SamplingParams(max_tokens=a.max_tokens, temperature=a.temperature, top_k=50, top_p=0.9)
    try:
        while True:
            user = a.prompt or input("> ")
            history.append({"role": "user", "content": user})
            answer = ""
            for _, text in llm.generate_stream(template.apply(history, True), sp):
                if text:
                    answer += text
                    sys.stdout.write(text)
                    sys.stdout.flush()
            sys.stdout.write(os.linesep)
            history.append({"role": "assistant", "content": answer})
            if a.prompt:
                return 0
    except (EOFError, KeyboardInterrupt):
        return 0
    finally:
        llm.close()


if __name__ == "__main__":
    sys.exit(main())
