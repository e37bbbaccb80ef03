"""``trtedge action``: vision-language-action inference — reason over the scene with the language model, then roll the
flow-matching action expert over its KV cache and write the trajectories.

Counterpart of the reference's ``examples/cpp/action_inference.cpp``.  Input file::

    {"requests": [{"messages": [{"role": "user", "content": [{"type": "image", "image": "front.png"},
                                                              {"type": "text", "text": "Plan the next 6 seconds."}]}],
                   "trajectory_history": [[x, y, z], ...],        # optional: becomes trajectory tokens appended to the prompt
                   "max_generate_length": 64, "seed": 0}]}

Output file: one entry per request with the generated ``text`` / ``token_ids`` and ``trajectory`` = ``n_diffusion_tokens``
rows of (acceleration, curvature)."""
from __future__ import annotations

import argparse
import json
import sys
from typing import List


def run_requests(llm, expert, body, multimodal=None, template=None, num_steps: int = 10) -> List[dict]:
    """Library form of the command (the tests call it with in-memory models)."""
    import torch
    from ..runtime.action import ActionRunner, trajectory_to_token_ids
    from ..runtime.multimodal import MultimodalInputs
    runner, kv = llm.runner, llm.kv
    act = ActionRunner(runner, expert, num_steps=num_steps)
    ac = expert.action_cfg
    out = []
    for req in body["requests"]:
        seat = 0
        kv.free(seat)
        max_new = int(req.get("max_generate_length", body.get("max_generate_length", 32)))
        history = trajectory_to_token_ids(req.get("trajectory_history", []), ac.num_traj_tokens, ac.traj_token_start)
        pieces = MultimodalInputs()
        if "prompt_token_ids" in req:
            pieces.text([int(t) for t in req["prompt_token_ids"]])
        else:
            from ..server.app import _split_media, _IMG, _AUD
            flat, media = _split_media(req["messages"])
            text = template.apply(flat, add_generation_prompt=True) if template is not None else "\n".join(str(m["content"]) for m in flat)
            if llm.tokenizer is None:
                raise ValueError("requests with messages need a tokenizer; send prompt_token_ids instead")
            media = list(media)
            for chunk in text.replace(_AUD, _IMG).split(_IMG):
                pieces.text(list(llm.tokenizer.encode(chunk)))
                if media:
                    kind, data = media.pop(0)
                    pieces.image(data) if kind == "image" else pieces.audio(*_wav(data))
        pieces.text(history)
        if multimodal is not None and any(k != "text" for k, _ in pieces.pieces):
            ids, emb, pos3, delta = multimodal.build(pieces)
            kv.reserve(seat, len(ids) + max_new + act.kv_headroom())
            logits = runner.prefill_embeds([seat], [emb], positions3=None if pos3 is None else [pos3],
                                           rope_deltas=None if pos3 is None else [delta], deepstack=multimodal.deepstack)
        else:
            ids = [t for k, p in pieces.pieces if k == "text" for t in p]
            kv.reserve(seat, len(ids) + max_new + act.kv_headroom())
            logits = runner.prefill([seat], [ids])
        first = runner.pick(logits)
        toks = [int(first[0])]
        if max_new > 1:
            toks += runner.decode_greedy([seat], first, max_new - 1)[0].tolist()
        eos = llm.cfg.eos_token_id
        eos = set(eos if isinstance(eos, (list, tuple)) else [eos]) - {None}
        cut = next((i + 1 for i, t in enumerate(toks) if t in eos), len(toks))
        if cut < len(toks):                       # the cache holds rows past the end token: drop them before the expert reads it
            kv.rewind(seat, len(ids) + cut - 1)
        toks = toks[:cut]
        traj = act.sample([seat], seed=int(req.get("seed", body.get("seed", 0))))[0]
        text = llm.tokenizer.decode(toks) if llm.tokenizer is not None else None
        if isinstance(text, (bytes, bytearray)):
            text = text.decode("utf-8", "replace")
        out.append({"token_ids": toks, "text": text, "trajectory": [[float(a), float(c)] for a, c in traj.tolist()]})
        kv.free(seat)
    return out


def _wav(data: bytes):
    from ..runtime import native as rt
    clip = rt.parse_audio(data)
    import numpy as np
    return np.asarray(clip.samples, dtype=np.float32), clip.sample_rate


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trtedge action", description=__doc__.split("\n\n")[0])
    ap.add_argument("model", help="vision-language checkpoint directory")
    ap.add_argument("--expert", required=True, help="action expert directory (config.json + safetensors)")
    ap.add_argument("--input-file", required=True)
    ap.add_argument("--output-file", required=True)
    ap.add_argument("--denoise-steps", type=int, default=10)
    ap.add_argument("--max-input-len", type=int, default=8192)
    ap.add_argument("--max-kv-cache-capacity", type=int, default=16384)
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)
    from ..chat_template import ChatTemplate
    from ..models.action_expert import ActionExpert
    from ..server import app as server_app
    server_app._MEDIA_ROOT["path"] = "/"          # an offline command reads the files its own input names
    from ..runtime import native as rt
    from ..runtime.llm import LLM
    from ..runtime.multimodal import MultimodalRunner
    with open(a.input_file, "r", encoding="utf-8") as f:
        body = json.load(f)
    if not isinstance(body.get("requests"), list) or not body["requests"]:
        print("error: the input file needs a non-empty 'requests' array", file=sys.stderr)
        return 2
    try:
        tok = rt.Tokenizer.load_from_hf(a.model)
    except Exception:
        tok = None
    llm = LLM(a.model, device=a.device, tokenizer=tok, max_batch_size=1, max_input_len=a.max_input_len, max_kv_cache_capacity=a.max_kv_cache_capacity)
    expert = ActionExpert.from_pretrained(a.expert, device=llm.device)
    results = run_requests(llm, expert, body, MultimodalRunner.from_pretrained(llm, a.model), ChatTemplate.load(a.model), a.denoise_steps)
    with open(a.output_file, "w", encoding="utf-8") as f:
        json.dump({"responses": results}, f, indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
