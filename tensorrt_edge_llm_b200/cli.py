"""``trtedge`` command dispatcher.

Same sub-commands as ``tensorrt_edgellm/cli.py:23-40``: chat, serve, build, export, quantize, insert-lora,
process-lora, merge-lora, reduce-vocab.  Each maps to a module with ``main(argv) -> int``."""
from __future__ import annotations

import argparse
import importlib
import sys
from typing import Optional, Sequence

from ._version import __version__

COMMANDS = {
    "chat": ("tensorrt_edge_llm_b200.commands.chat", "Chat with a local checkpoint"),
    "serve": ("tensorrt_edge_llm_b200.server.cli", "Launch an OpenAI-compatible server"),
    "build": ("tensorrt_edge_llm_b200.commands.build", "Validate a checkpoint and write runtime artifacts"),
    "export": ("tensorrt_edge_llm_b200.commands.export", "Export a checkpoint to ONNX"),
    "quantize": ("tensorrt_edge_llm_b200.commands.quantize", "Quantize a checkpoint or draft model"),
    "insert-lora": ("tensorrt_edge_llm_b200.commands.insert_lora", "Report where a LoRA adapter attaches"),
    "process-lora": ("tensorrt_edge_llm_b200.commands.process_lora_weights", "Process LoRA adapter weights"),
    "merge-lora": ("tensorrt_edge_llm_b200.commands.merge_lora", "Merge a LoRA adapter into a checkpoint"),
    "reduce-vocab": ("tensorrt_edge_llm_b200.commands.reduce_vocab", "Generate reduced-vocabulary artifacts"),
    "infer": ("tensorrt_edge_llm_b200.commands.infer", "Run a request file and write predictions"),
    "stream": ("tensorrt_edge_llm_b200.commands.stream", "Run a request file and print the answers while they are generated"),
    "tts": ("tensorrt_edge_llm_b200.commands.tts", "Text to speech from a request file (talker, code predictor, vocoder)"),
    "multistage": ("tensorrt_edge_llm_b200.commands.multistage", "Run requests through a multi-stage graph"),
    "action": ("tensorrt_edge_llm_b200.commands.action", "Vision-language-action inference: reasoning text + trajectory"),
    "bench": ("tensorrt_edge_llm_b200.benchmarks.llm_bench", "Offline benchmark writing report.json"),
}


def main(argv: Optional[Sequence[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    parser = argparse.ArgumentParser(prog="trtedge", description="B200-native Edge-LLM tools", add_help=False)
    parser.add_argument("command", nargs="?", choices=sorted(COMMANDS))
    parser.add_argument("--version", action="store_true")
    parser.add_argument("-h", "--help", action="store_true")
    ns, rest = parser.parse_known_args(argv[:1])
    if ns.version:
        print(__version__)
        return 0
    if ns.command is None:
        print("usage: trtedge <command> [options]\n\ncommands:")
        for name in sorted(COMMANDS):
            print(f"  {name:<14}{COMMANDS[name][1]}")
        return 0 if ns.help else 2
    module = importlib.import_module(COMMANDS[ns.command][0])
    rc = module.main(argv[1:])
    return int(rc or 0)


if __name__ == "__main__":
    sys.exit(main())
