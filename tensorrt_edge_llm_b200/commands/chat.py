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
    p.add_argument("--image", action="append", default=[], help="image file shown with the first user turn (vision-language checkpoints; repeatable)")
    a = p.parse_args(argv)
    from ..chat_template import ChatTemplate
    from ..runtime import native as rt
    from ..runtime.llm import LLM
    from ..runtime.runner import SamplingParams
    tok = rt.Tokenizer.load_from_hf(a.model_dir)
    llm = LLM(a.model_dir, max_batch_size=1, tokenizer=tok, enable_in_flight_batching=True)
    template = ChatTemplate.load(a.model_dir)
    multimodal = None
    if a.image:
        from ..runtime.multimodal import MultimodalInputs, MultimodalRunner
        multimodal = MultimodalRunner.from_pretrained(llm, a.model_dir)
        if multimodal is None:
            print("error: this checkpoint names no vision tower this runtime builds", file=sys.stderr)
            return 2
    images = [open(path, "rb").read() for path in a.image]
    mark = "\x00IMG\x00"
    history = [{"role": "system", "content": a.system}] if a.system else []
    sp = SamplingParams(max_tokens=a.max_tokens, temperature=a.temperature, top_k=50, top_p=0.9)
    try:
        while True:
            user = a.prompt or input("> ")
            history.append({"role": "user", "content": (mark * len(images) if len(history) <= 1 else "") + user})
            answer = ""
            prompt = template.apply(history, True)
            if images:                       # the rendered prompt keeps one marker per image: text pieces and images in order
                req, rest = MultimodalInputs(), iter(images)
                for k, piece in enumerate(prompt.split(mark)):
                    if k:
                        req.image(next(rest))
                    if piece:
                        req.text(list(tok.encode(piece)))
                prompt = multimodal.prepare(req)
            for _, text in llm.generate_stream(prompt, sp):
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
