"""Guided (constrained) decoding: a matcher turns "what may come next" into a token bitmask per step.

Supported request types (``GuidedDecodingParams.type``): ``choice`` (one of a list of strings), ``regex`` (full match
of a regular expression), ``json_object`` (any syntactically valid JSON object, nesting bounded) and ``json_schema``
for flat objects of string / number / integer / boolean / enum properties (compiled to a regex).  A token is allowed
when the text so far plus the token's text can still be completed to a match; the end-of-sequence token is allowed
once the text is a complete match.  The bitmask feeds ``ops.apply_token_bitmask`` before sampling.

Parity: ``cpp/runtime/decoding/guidedDecoder.cpp`` (XGrammar matcher → token bitmask, ``GuidedDecodingParams`` types of
``cpp/runtime/llmRuntimeUtils.h``).  The matcher here is this package's own: partial regular-expression matching
(the ``regex`` module), an incremental JSON recogniser, and for ``ebnf`` / ``structural_tag`` the Earley recogniser and tag
scanner of ``runtime/grammar.py``."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch


@dataclass
class GuidedDecodingParams:
    type: str                                  # "choice" | "regex" | "json_object" | "json_schema" | "ebnf" | "structural_tag"
    choices: Sequence[str] = ()
    pattern: str = ""
    json_schema: Optional[dict] = None
    max_depth: int = 8
    jump_forward: bool = False                 # append grammar-forced tokens without a forward pass each (ebnf only)
    grammar: str = ""                          # EBNF text ("ebnf")
    structural_tag: Optional[dict] = None      # {"structures": [...], "triggers": [...]} ("structural_tag")

    def __post_init__(self):
        if self.type not in ("choice", "regex", "json_object", "json_schema", "ebnf", "structural_tag"):
            raise ValueError(f"unsupported guided decoding type {self.type!r}")
        if self.type == "ebnf" and not self.grammar:
            raise ValueError("ebnf needs a grammar")
        if self.type == "structural_tag" and not isinstance(self.structural_tag, dict):
            raise ValueError("structural_tag needs a specification object")
        if self.type == "choice" and not self.choices:
            raise ValueError("choice needs a non-empty list")
        if self.type == "regex" and not self.pattern:
            raise ValueError("regex needs a pattern")
        if self.type == "json_schema" and not isinstance(self.json_schema, dict):
            raise ValueError("json_schema needs a schema object")


# ---- matchers: state = the text generated so far -------------------------------------------------------------------

class _RegexMatcher:
    def __init__(self, pattern: str):
        import regex
        self._re = regex.compile(pattern, regex.DOTALL)

    def viable(self, text: str) -> bool:
        return self._re.fullmatch(text, partial=True) is not None

    def complete(self, text: str) -> bool:
        return self._re.fullmatch(text) is not None


class _ChoiceMatcher:
    def __init__(self, choices: Sequence[str]):
        self.choices = list(choices)

    def viable(self, text: str) -> bool:
        return any(c.startswith(text) for c in self.choices)

    def complete(self, text: str) -> bool:
        return text in self.choices


class _JsonObjectMatcher:
    """Incremental JSON recogniser: accepts every prefix of a valid JSON object (whitespace allowed between tokens)."""

    def __init__(self, max_depth: int = 8):
        self.max_depth = max_depth

    def _scan(self, text: str):
        """Returns (ok, complete).  A small pushdown automaton over characters."""
        stack: List[str] = []           # '{' or '['
        state = "start"                 # start | value | key_or_end | key | colon | comma_or_end | string | str_esc | number | literal | done
        lit, lit_pos, in_key = "", 0, False
        i, n = 0, len(text)
        while i < n:
            ch = text[i]
            if state == "string":
                if ch == "\\":
                    state = "str_esc"
                elif ch == '"':
                    state = "colon" if in_key else "comma_or_end"
                elif ch < " ":
                    return False, False
                i += 1
                continue
            if state == "str_esc":
                if ch not in '"\\/bfnrtu':
                    return False, False
                state = "string"
                i += 1
                continue
            if state == "number":
                if ch.isdigit() or ch in "+-.eE":
                    i += 1
                    continue
                state = "comma_or_end"          # re-scan this character
                continue
            if state == "literal":
                if lit_pos < len(lit) and ch == lit[lit_pos]:
                    lit_pos += 1
                    i += 1
                    if lit_pos == len(lit):
                        state = "comma_or_end"
                    continue
                return False, False
            if ch in " \t\r\n":
                i += 1
                continue
            if state == "start":
                if ch != "{":
                    return False, False
                stack.append("{")
                state = "key_or_end"
            elif state == "key_or_end":
                if ch == '"':
                    state, in_key = "string", True
                elif ch == "}":
                    stack.pop()
                    state = "comma_or_end" if stack else "done"
                else:
                    return False, False
            elif state == "key":
                if ch != '"':
                    return False, False
                state, in_key = "string", True
            elif state == "colon":
                if ch != ":":
                    return False, False
                state = "value"
            elif state == "value":
                in_key = False
                if ch == '"':
                    state = "string"
                elif ch == "{" or ch == "[":
                    if len(stack) >= self.max_depth:
                        return False, False
                    stack.append(ch)
                    state = "key_or_end" if ch == "{" else "value_or_end"
                elif ch == "-" or ch.isdigit():
                    state = "number"
                elif ch in "tfn":
                    lit, lit_pos, state = {"t": "true", "f": "false", "n": "null"}[ch], 1, "literal"
                else:
                    return False, False
            elif state == "value_or_end":
                if ch == "]":
                    stack.pop()
                    state = "comma_or_end" if stack else "done"
                else:
                    state = "value"
                    continue
            elif state == "comma_or_end":
                if not stack:
                    return False, False
                if ch == ",":
                    state = "key" if stack[-1] == "{" else "value"
                elif ch == "}" and stack[-1] == "{" or ch == "]" and stack[-1] == "[":
                    stack.pop()
                    state = "comma_or_end" if stack else "done"
                else:
                    return False, False
            elif state == "done":
                return False, False
            i += 1
        return True, state == "done"

    def viable(self, text: str) -> bool:
        return self._scan(text)[0]

    def complete(self, text: str) -> bool:
        ok, done = self._scan(text)
        return ok and done


def schema_to_regex(schema: dict) -> str:
    """Flat object schemas → a regular expression (properties in declaration order, all required)."""
    import regex

    def value(s: dict) -> str:
        if "enum" in s:
            return "(?:" + "|".join(regex.escape(json.dumps(v)) for v in s["enum"]) + ")"
        t = s.get("type")
        if t == "string":
            return r'"(?:[^"\\\x00-\x1f]|\\["\\/bfnrt])*"'
        if t == "integer":
            return r"-?(?:0|[1-9][0-9]{0,17})"
        if t == "number":
            return r"-?(?:0|[1-9][0-9]{0,17})(?:\.[0-9]{1,17})?(?:[eE][+-]?[0-9]{1,3})?"
        if t == "boolean":
            return r"(?:true|false)"
        if t == "null":
            return "null"
        raise ValueError(f"unsupported schema fragment {s!r}")

    if schema.get("type") != "object" or not isinstance(schema.get("properties"), dict):
        raise ValueError("only flat object schemas are supported")
    ws = r"[ \n]?"          # bounded: an unconstrained model must not be able to pad for ever
    parts = [ws + regex.escape(json.dumps(k)) + ws + ":" + ws + value(v) for k, v in schema["properties"].items()]
    return r"\{" + ("," .join(parts)) + ws + r"\}"


def make_matcher(params: GuidedDecodingParams):
    if params.type == "choice":
        return _ChoiceMatcher(params.choices)
    if params.type == "regex":
        return _RegexMatcher(params.pattern)
    if params.type == "json_schema":
        return _RegexMatcher(schema_to_regex(params.json_schema))
    if params.type == "ebnf":
        from .grammar import EbnfMatcher
        return EbnfMatcher(params.grammar)
    if params.type == "structural_tag":
        from .grammar import StructuralTagMatcher
        return StructuralTagMatcher(params.structural_tag)
    return _JsonObjectMatcher(params.max_depth)


class GuidedDecoder:
    """Per-request matcher state + bitmask construction over a tokenizer's vocabulary."""

    def __init__(self, params: GuidedDecodingParams, token_texts: Sequence[Optional[str]], eos_token_ids: Sequence[int]):
        self.matcher = make_matcher(params)
        self.token_texts = list(token_texts)          # None = token that can never be produced under a constraint (specials)
        self.eos = set(int(t) for t in eos_token_ids)
        self.text = ""
        self.finished = False
        self.jump_forward = bool(params.jump_forward) and hasattr(self.matcher, "forced_continuation")

    @staticmethod
    def vocabulary(tokenizer, vocab_size: int) -> List[Optional[str]]:
        out: List[Optional[str]] = []
        for i in range(vocab_size):
            try:
                b = bytes(tokenizer.id_to_bytes(i))
                out.append(b.decode("utf-8") if b else None)
            except (UnicodeDecodeError, ValueError, IndexError):
                out.append(None)                      # partial UTF-8 sequences are not offered
        return out

    def bitmask(self) -> torch.Tensor:
        """int32 ``[ceil(V / 32)]``: bit t set ⇔ token t may come next."""
        v = len(self.token_texts)
        bits = torch.zeros((v + 31) // 32 * 32, dtype=torch.bool)
        if self.matcher.complete(self.text):
            for e in self.eos:
                if e < v:
                    bits[e] = True
        seen = {}
        for t, piece in enumerate(self.token_texts):
            if piece is None or t in self.eos:
                continue
            ok = seen.get(piece)
            if ok is None:
                ok = seen[piece] = self.matcher.viable(self.text + piece)
            bits[t] = ok
        if not bits.any():
            for e in self.eos:                         # dead end: let the request stop rather than emit anything
                if e < v:
                    bits[e] = True
        w = bits.view(-1, 32).to(torch.int64)
        packed = (w << torch.arange(32)).sum(-1)
        return torch.where(packed >= 2 ** 31, packed - 2 ** 32, packed).to(torch.int32)

    def forced_tokens(self, tokenizer, budget: int) -> List[int]:
        """Tokens the constraint forces next (``cpp/runtime/decoding/jumpForward.cpp`` in the reference): the grammar allows
        exactly one continuation for a stretch of characters, so its tokens are appended — and the matcher advanced —
        without sampling them one forward pass at a time.  At most ``budget`` tokens; never a partial character run that
        the tokenizer would split differently from the matcher's view (every token is re-checked against the grammar)."""
        if not self.jump_forward or self.finished or budget <= 0:
            return []
        forced = self.matcher.forced_continuation(self.text)
        if not forced:
            return []
        out: List[int] = []
        for t in tokenizer.encode(forced):
            t = int(t)
            piece = self.token_texts[t] if 0 <= t < len(self.token_texts) else None
            if piece is None or len(out) >= budget or not forced.startswith(piece):
                break
            self.advance(t)
            forced = forced[len(piece):]
            out.append(t)
        return out

    def advance(self, token: int) -> None:
        if token in self.eos:
            self.finished = True
            return
        piece = self.token_texts[token] if 0 <= token < len(self.token_texts) else None
        if piece is None or not self.matcher.viable(self.text + piece):
            if not self.eos and self.matcher.complete(self.text):      # nothing can follow and the model has no end token: done
                self.finished = True
                return
            raise ValueError(f"token {token} violates the constraint after {self.text!r}")
        self.text += piece
        if hasattr(self.matcher, "commit"):            # grammar matchers keep the chart of the accepted text
            self.matcher.commit(self.text)


@torch.no_grad()
def generate_guided(llm, prompt_ids: Sequence[int], params: GuidedDecodingParams, max_tokens: int = 128,
                    sample: Optional[Callable[[torch.Tensor], int]] = None, seat: int = 0) -> List[int]:
    """Constrained generation of one request on the static-batch path: mask → sample → advance, step by step."""
    from .. import ops
    if llm.tokenizer is None:
        raise ValueError("guided decoding needs a tokenizer (token texts)")
    eos = llm.cfg.eos_token_id
    eos_ids = [int(t) for t in (eos if isinstance(eos, (list, tuple)) else [eos]) if t is not None]
    dec = GuidedDecoder(params, GuidedDecoder.vocabulary(llm.tokenizer, llm.cfg.vocab_size), eos_ids)
    runner, kv = llm.runner, llm.kv
    kv.free(seat)
    kv.reserve(seat, len(prompt_ids) + max_tokens)
    was = runner.use_cuda_graphs
    runner.use_cuda_graphs = False
    logits = runner.prefill([seat], [list(prompt_ids)])
    out: List[int] = []
    try:
        for _ in range(max_tokens):
            mask = dec.bitmask().to(logits.device)[None]
            masked = ops.apply_token_bitmask(logits[:1].float().clone(), mask)
            tok = int(sample(masked[0]) if sample is not None else masked[0].argmax())
            dec.advance(tok)
            if dec.finished:
                break
            out.append(tok)
            logits = runner.step([seat], [[tok]])
    finally:
        runner.use_cuda_graphs = was
        kv.free(seat)
    return out
