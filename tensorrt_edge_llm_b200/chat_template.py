"""Chat-template handling: turn a list of chat messages into the prompt string a checkpoint expects.

Order of preference: the checkpoint's own Jinja template (``chat_template.jinja`` or the
``chat_template`` field of ``tokenizer_config.json``) rendered with jinja2 in a sandbox; the native
template families of the C++ runtime (``csrc/runtime/tokenizer.cpp``); a ChatML fallback.

Parity: ``tensorrt_edgellm/chat_template.py`` (template extraction at export time) and
``cpp/chatTemplate/chatTemplate.{h,cpp}`` (``ChatTemplate::load / apply / optionsFrom``)."""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional, Sequence


def extract_chat_template(model_dir: str) -> Optional[str]:
    """The checkpoint's Jinja chat template text, or None."""
    p = os.path.join(model_dir, "chat_template.jinja")
    if os.path.exists(p):
        with open(p, "r", encoding="utf-8") as f:
            return f.read()
    p = os.path.join(model_dir, "tokenizer_config.json")
    if os.path.exists(p):
        with open(p, "r", encoding="utf-8") as f:
            cfg = json.load(f)
        t = cfg.get("chat_template")
        if isinstance(t, list):                      # named templates: [{"name": "default", "template": ...}, ...]
            named = {e.get("name"): e.get("template") for e in t if isinstance(e, dict)}
            t = named.get("default") or next(iter(named.values()), None)
        if isinstance(t, str) and t.strip():
            return t
    return None


def _special_tokens(model_dir: str) -> Dict[str, str]:
    out = {"bos_token": "", "eos_token": ""}
    p = os.path.join(model_dir, "tokenizer_config.json")
    if os.path.exists(p):
        with open(p, "r", encoding="utf-8") as f:
            cfg = json.load(f)
        for k in out:
            v = cfg.get(k)
            if isinstance(v, dict):
                v = v.get("content")
            if isinstance(v, str):
                out[k] = v
    return out


def _content_text(content: Any) -> str:
    """OpenAI content parts → plain text (non-text parts are dropped here; media goes another way)."""
    if isinstance(content, str) or content is None:
        return content or ""
    return "".join(str(p.get("text", "")) for p in content if isinstance(p, dict) and p.get("type") in ("text", "input_text"))


class ChatTemplate:
    def __init__(self, jinja_text: Optional[str] = None, special: Optional[Dict[str, str]] = None, native=None):
        self.special = special or {"bos_token": "", "eos_token": ""}
        self._native = native
        self._jinja = None
        self.source = jinja_text or ""
        if jinja_text:
            from jinja2.sandbox import ImmutableSandboxedEnvironment

            def raise_exception(msg):
                raise ValueError(msg)

            env = ImmutableSandboxedEnvironment(trim_blocks=True, lstrip_blocks=True)
            env.globals["raise_exception"] = raise_exception
            env.filters["tojson"] = lambda v, **kw: json.dumps(v, ensure_ascii=False, **kw)
            self._jinja = env.from_string(jinja_text)

    @classmethod
    def load(cls, model_dir: str) -> "ChatTemplate":
        text = extract_chat_template(model_dir)
        native = None
        if text is None:
            try:
                from .runtime import native as rt
                native = rt.ChatTemplate.load(model_dir)
            except Exception:       # no native module or no recognisable family: ChatML fallback below
                native = None
        return cls(text, _special_tokens(model_dir), native)

    def apply(self, messages: Sequence[Dict[str, Any]], add_generation_prompt: bool = True, tools: Optional[List[dict]] = None,
              enable_thinking: bool = True) -> str:
        msgs = [{**m, "content": _content_text(m.get("content"))} for m in messages]
        if self._jinja is not None:
            return self._jinja.render(messages=msgs, add_generation_prompt=add_generation_prompt, tools=tools or None,
                                      enable_thinking=enable_thinking, **self.special)
        if self._native is not None:
            from .runtime import native as rt
            return self._native.apply([rt.ChatMessage(m["role"], m["content"]) for m in msgs], add_generation_prompt, enable_thinking)
        out = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in msgs)
        return out + ("<|im_start|>assistant\n" if add_generation_prompt else "")
