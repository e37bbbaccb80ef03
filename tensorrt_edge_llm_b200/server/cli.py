"""``trtedge serve <checkpoint>``: load the model, start the request engine, run uvicorn.

Parity: ``tensorrt_edgellm/server/cli.py`` / ``__main__.py``.  There is no engine build or cache step:
the checkpoint is loaded straight into device memory."""
from __future__ import annotations

import os
import sys
from typing import Optional, Sequence

from .config import ServerConfig, ServerConfigError, parse_server_config


def build_llm(cfg: ServerConfig):
    from ..chat_template import ChatTemplate
    from ..runtime.llm import LLM
    m = cfg.model
    tok = None
    try:
        from ..runtime import native as rt
        if os.path.exists(os.path.join(m.model, "tokenizer.json")):
            tok = rt.Tokenizer.load_from_hf(m.model)
    except ImportError:
        tok = None
    spec_kw = {}
    if m.speculative_config is not None and m.speculative_config.draft_model:
        from ..runtime.speculative import SpecConfig
        sc = m.speculative_config
        spec_kw = {"draft_model": sc.draft_model,
                   "speculative": SpecConfig(draft_steps=sc.num_speculative_tokens or 4, top_k=sc.draft_top_k or 8,
                                             verify_tokens=sc.verify_tokens or 32,
                                             # block drafts: an explicit draft_top_k above 1 asks for tree verification
                                             block_tree_top_k=min(sc.draft_top_k, 8) if (sc.draft_top_k or 1) > 1 and sc.method in ("dflash", "jetspec") else 1)}
    tp_kw = {}
    if m.tensor_parallel_size > 1:
        # one process per GPU (launched with ``python -m torch.distributed.run --nproc-per-node N -m … serve …``): rank 0
        # serves HTTP and schedules, the other ranks follow its steps (parallel/tp_serving.py)
        import torch
        import torch.distributed as dist
        from ..config import Mapping
        from ..parallel import make_comm
        from ..parallel.tp_serving import StepMirror
        rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
        if world != m.tensor_parallel_size:
            raise ServerConfigError(f"--tensor-parallel-size {m.tensor_parallel_size} needs that many ranks (WORLD_SIZE is {world})")
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        cuda = torch.cuda.is_available() and (m.device or "cuda").startswith("cuda")
        if cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        if not dist.is_initialized():
            dist.init_process_group("nccl" if cuda else "gloo")
        dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
        tp_kw = {"comm": make_comm("fused" if cuda else "nccl", dev), "mapping": Mapping(tp_size=world, tp_rank=rank),
                 "tp_mirror": None}
        build_llm.mirror = StepMirror()             # collective: every rank creates the mirror's group here
        if rank == 0 and m.enable_in_flight_batching:
            tp_kw["tp_mirror"] = build_llm.mirror
        m.device = str(dev)
    llm = LLM(m.model, device=m.device or None, **spec_kw, **tp_kw, max_batch_size=m.max_batch_size, max_input_len=m.max_input_len,
              max_kv_cache_capacity=m.max_kv_cache_capacity, kv_cache_dtype=m.kv_cache_dtype, page_size=m.kv_page_size, max_num_tokens=m.max_num_tokens or 8192,
              tokenizer=tok, enable_in_flight_batching=m.enable_in_flight_batching and int(os.environ.get("RANK", "0")) == 0,
              enable_prefix_cache=m.context_cache_config.enabled, context_cache_max_records=m.context_cache_config.max_records,
              context_cache_max_snapshots=m.context_cache_config.max_snapshots, scheduling=m.scheduling_dict() if m.enable_in_flight_batching else None)
    return llm, ChatTemplate.load(m.model)


def main(argv: Optional[Sequence[str]] = None) -> int:
    try:
        cfg = parse_server_config(argv)
    except ServerConfigError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    if cfg.model.tensor_parallel_size > 1 and not cfg.model.enable_in_flight_batching:
        print("error: tensor-parallel serving needs --enable-in-flight-batching (rank 0 schedules, the others follow)", file=sys.stderr)
        return 2
    import uvicorn
    from .app import create_app
    llm, template = build_llm(cfg)
    if cfg.model.tensor_parallel_size > 1 and int(os.environ.get("RANK", "0")) != 0:
        from ..parallel.tp_serving import serve_follower
        cc = cfg.model.context_cache_config
        serve_follower(llm.runner, build_llm.mirror, enable_prefix_cache=cc.enabled, max_records=cc.max_records)
        return 0
    multimodal = None
    if os.path.isdir(cfg.model.model):                   # vision-language checkpoints bring their tower along
        from ..runtime.multimodal import MultimodalRunner
        mc = cfg.model.multimodal_config
        multimodal = MultimodalRunner.from_pretrained(llm, cfg.model.model, cache_bytes=mc.encoder_cache_budget_bytes)
        if multimodal is not None and mc.max_image_tokens_per_image and hasattr(multimodal.vision.cfg, "spatial_merge_size"):
            vc = multimodal.vision.cfg                      # rows per image × pixels per row (patch × merge, squared)
            multimodal.max_pixels = mc.max_image_tokens_per_image * (vc.patch_size * vc.spatial_merge_size) ** 2
    tts = None
    if cfg.model.tts_model:
        from ..runtime.tts import TTS
        tts = TTS(cfg.model.tts_model, device=cfg.model.device or "cpu")
    app = create_app(llm, cfg.api, template, model_name=os.path.basename(os.path.normpath(cfg.model.model)), multimodal=multimodal, tts=tts)
    try:
        uvicorn.run(app, host=cfg.api.host, port=cfg.api.port, log_level=cfg.api.log_level)
    finally:
        llm.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
