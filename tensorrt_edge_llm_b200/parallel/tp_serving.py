"""In-flight batching with tensor parallelism: rank 0 schedules, the other ranks follow.

The reference keeps tensor-parallel deployments on its one-request-at-a-time path (``docs/source/user_guide/examples/
server.md:634-636``).  Here the request engine runs on rank 0 only; every state change of its session that touches the
model — a seat reserved, a step executed, a seat released — is mirrored to the other ranks as a small broadcast *before*
rank 0 runs it, and the followers replay it on their own shard (their own KV pool and page ids; only seats, token ids and
lengths have to agree).  The collectives inside the model step then meet on all ranks.  Sampling happens on rank 0; the
followers never look at logits.  Steps that hold a chunk of a multimodal prompt ship their embedding rows along
(``step_embeds``): the media encoders run on rank 0 only."""
from __future__ import annotations

from typing import List, Sequence

import torch.distributed as dist


class StepMirror:
    """Rank 0 → all: ordered stream of session operations (``broadcast_object_list`` over the given group)."""

    def __init__(self, group=None, src: int = 0):
        # A group of its own (gloo, host memory) with a week-long timeout: followers sit in this broadcast while the
        # server is idle, which must not trip the watchdog of the group the model's collectives use.  Every rank has to
        # construct the mirror (creating a group is collective).
        if group is None:
            import datetime
            group = dist.new_group(backend="gloo", timeout=datetime.timedelta(days=7))
        self.group, self.src = group, src
        self.sent = 0

    def send(self, op: tuple) -> None:
        dist.broadcast_object_list([op], src=self.src, group=self.group)
        self.sent += 1

    def recv(self) -> tuple:
        box = [None]
        dist.broadcast_object_list(box, src=self.src, group=self.group)
        return box[0]


def serve_follower(runner, mirror: StepMirror, enable_prefix_cache: bool = False, max_records: int = 4096) -> int:
    """Replay rank 0's session on this rank until it says stop; returns the number of steps executed.

    ``enable_prefix_cache`` / ``max_records`` must equal rank 0's: the follower then keeps a prefix index of its own and repeats
    every lookup, adoption, insertion and eviction, so its pages and reference counts stay in step with rank 0's."""
    kv, steps = runner.kv, 0
    prefix = None
    if enable_prefix_cache and getattr(kv, "native", None) is not None and not kv.bounded_swa and not runner.model.cfg.is_hybrid:
        from ..runtime import native as rt
        prefix = rt.PrefixCache(kv.native.allocator(), kv.page_size, max_records)
    while True:
        op = mirror.recv()
        kind = op[0]
        if kind == "stop":
            return steps
        if kind == "noop":                 # keep-alive while the engine is idle
            continue
        if kind == "reserve":
            _, slot, need = op
            kv.free(slot)
            kv.reserve(slot, need)
        elif kind == "admit":
            _, slot, prompt_ids, need, ok, seed = op
            kv.free(slot)
            try:
                if prefix is not None and prompt_ids is not None:
                    m = prefix.lookup(list(prompt_ids), seed)
                    if m.tokens:
                        kv.adopt_prefix(slot, list(m.pages), m.tokens)
                if ok:
                    kv.reserve(slot, need)
            except (MemoryError, RuntimeError):
                ok = False
            if not ok:                         # rank 0 gave the seat back and made room: do the same
                kv.free(slot)
                if prefix is not None:
                    prefix.evict(8)
        elif kind == "prefix_insert":
            _, slot, tokens, n, seed = op
            if prefix is not None:
                prefix.insert(list(tokens), n, kv.pages_of(slot), seed)
        elif kind == "step":
            _, seats, token_lists = op
            runner.step(list(seats), [list(t) for t in token_lists])
            steps += 1
        elif kind == "decode_graph":
            _, seats, tokens = op
            if runner.can_graph_step(list(seats)):
                runner.decode_step_graph(list(seats), list(tokens))
            else:                              # CPU ranks (tests): the same step, eagerly
                runner.step(list(seats), [[int(t)] for t in tokens])
            steps += 1
        elif kind == "step_embeds":
            # a step that carries a multimodal prompt chunk: rank 0 ships the embedding rows (host tensors) with the plan
            _, seats, embeds, pos3, deepstack, deltas = op
            runner.step_embeds(list(seats), [e.to(runner.device) for e in embeds], pos3, deepstack)
            for slot, d in deltas:
                runner.rope_delta[slot] = d
            steps += 1
        elif kind == "release":
            kv.free(op[1])
        else:
            raise RuntimeError(f"unknown mirrored operation {kind!r}")
