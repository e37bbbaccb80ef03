"""Grammar-constrained decoding: EBNF grammars (an Earley recogniser over characters) and structural tags.

An EBNF grammar in the GBNF / XGrammar style —

    root   ::= "{" ws pair ("," ws pair)* "}"
    pair   ::= string ":" ws value
    string ::= "\\"" [a-z]* "\\""
    value  ::= [0-9]+ | string | "true" | "false"
    ws     ::= " "?

— is compiled to plain productions whose terminals are character sets; the matcher answers "can this text still be
completed to a sentence of the grammar" (``viable``) and "is it a sentence" (``complete``) by running an Earley
recogniser, caching the chart of the last accepted text so that per-token probes only pay for the token's characters.

Structural tags (``{"structures": [{"begin": "<function=f>", "schema": {...}, "end": "</function>"}], "triggers":
["<function="]}``) leave the text free until a trigger appears, then require one of the ``begin`` strings, a JSON value
of that structure's schema, and its ``end`` string, after which the text is free again.

Parity: the grammar modes of ``cpp/runtime/decoding/guidedDecoder.cpp`` (XGrammar ``Ebnf`` / ``StructuralTag``) and the
forced-continuation idea of ``jumpForward.cpp`` (:meth:`EbnfMatcher.forced_continuation`)."""
from __future__ import annotations

from typing import Dict, FrozenSet, List, Optional, Sequence, Set, Tuple


class GrammarError(ValueError):
    pass


# ---- EBNF → productions ----------------------------------------------------------------------------------------------

class _CharSet:
    __slots__ = ("ranges", "negated")

    def __init__(self, ranges: Sequence[Tuple[int, int]], negated: bool = False):
        self.ranges, self.negated = tuple(ranges), negated

    def __contains__(self, ch: str) -> bool:
        c = ord(ch)
        hit = any(lo <= c <= hi for lo, hi in self.ranges)
        return hit != self.negated

    def sample(self) -> Optional[str]:
        """The only member, if the set has exactly one (used for forced continuations)."""
        if self.negated or len(self.ranges) != 1 or self.ranges[0][0] != self.ranges[0][1]:
            return None
        return chr(self.ranges[0][0])


_ESC = {"n": "\n", "t": "\t", "r": "\r", "\\": "\\", '"': '"', "'": "'", "]": "]", "[": "[", "-": "-", "^": "^"}


class _Parser:
    """Recursive-descent parser of the grammar text; emits productions ``name → [symbols]`` where a symbol is a rule
    name (str) or a :class:`_CharSet`."""

    def __init__(self, text: str):
        self.s, self.i = text, 0
        self.rules: Dict[str, List[List[object]]] = {}
        self.fresh = 0

    def _ws(self, newlines: bool = True):
        while self.i < len(self.s):
            c = self.s[self.i]
            if c == "#":
                while self.i < len(self.s) and self.s[self.i] != "\n":
                    self.i += 1
            elif c in " \t\r" or (newlines and c == "\n"):
                self.i += 1
            else:
                break

    def _name(self) -> str:
        j = self.i
        while j < len(self.s) and (self.s[j].isalnum() or self.s[j] in "_-"):
            j += 1
        if j == self.i:
            raise GrammarError(f"expected a rule name at offset {self.i}")
        name, self.i = self.s[self.i:j], j
        return name

    def _new(self, alts: List[List[object]]) -> str:
        self.fresh += 1
        name = f"%{self.fresh}"
        self.rules[name] = alts
        return name

    def parse(self) -> Dict[str, List[List[object]]]:
        self._ws()
        while self.i < len(self.s):
            name = self._name()
            self._ws()
            if not self.s.startswith("::=", self.i):
                raise GrammarError(f"expected '::=' after {name!r}")
            self.i += 3
            alts = self._alternatives()
            self.rules.setdefault(name, []).extend(alts)
            self._ws()
        if "root" not in self.rules:
            raise GrammarError("the grammar needs a 'root' rule")
        for alts in list(self.rules.values()):
            for alt in alts:
                for sym in alt:
                    if isinstance(sym, str) and sym not in self.rules:
                        raise GrammarError(f"undefined rule {sym!r}")
        return self.rules

    def _at_rule_start(self) -> bool:
        """True when the upcoming tokens are ``name ::=`` (the next rule), which ends the current alternative list."""
        j = self.i
        while j < len(self.s) and (self.s[j].isalnum() or self.s[j] in "_-"):
            j += 1
        if j == self.i:
            return False
        while j < len(self.s) and self.s[j] in " \t":
            j += 1
        return self.s.startswith("::=", j)

    def _alternatives(self) -> List[List[object]]:
        alts = [self._sequence()]
        while True:
            self._ws()
            if self.i < len(self.s) and self.s[self.i] == "|":
                self.i += 1
                alts.append(self._sequence())
            else:
                return alts

    def _sequence(self) -> List[object]:
        seq: List[object] = []
        while True:
            self._ws()
            if self.i >= len(self.s) or self.s[self.i] in "|)" or self._at_rule_start():
                return seq
            seq.extend(self._repeated(self._atom()))

    def _atom(self) -> List[object]:
        c = self.s[self.i]
        if c == '"':
            return [_CharSet([(ord(ch), ord(ch))]) for ch in self._string()]
        if c == "[":
            return [self._charclass()]
        if c == "(":
            self.i += 1
            alts = self._alternatives()
            self._ws()
            if self.i >= len(self.s) or self.s[self.i] != ")":
                raise GrammarError("unbalanced parenthesis")
            self.i += 1
            return [self._new(alts)]
        if c == ".":
            self.i += 1
            return [_CharSet([(0, 0x10FFFF)])]
        return [self._name()]

    def _repeated(self, atom: List[object]) -> List[object]:
        if self.i >= len(self.s) or self.s[self.i] not in "*+?{":
            return atom
        op = self.s[self.i]
        unit = atom[0] if len(atom) == 1 else self._new([atom])
        if op == "{":
            j = self.s.index("}", self.i)
            body = self.s[self.i + 1:j]
            self.i = j + 1
            lo, _, hi = body.partition(",")
            lo_n = int(lo)
            hi_n = lo_n if "," not in body else (int(hi) if hi.strip() else None)
            out: List[object] = [unit] * lo_n
            if hi_n is None:
                out.append(self._new([[], [unit, None]]))
                self.rules[out[-1]][1][1] = out[-1]
            else:
                opt = self._new([[], [unit]])
                out += [opt] * (hi_n - lo_n)
            return out
        self.i += 1
        if op == "?":
            return [self._new([[], [unit]])]
        star = self._new([[], [unit, None]])
        self.rules[star][1][1] = star                    # star → ε | unit star
        return [star] if op == "*" else [unit, star]

    def _string(self) -> str:
        self.i += 1
        out = []
        while self.i < len(self.s) and self.s[self.i] != '"':
            c = self.s[self.i]
            if c == "\\":
                self.i += 1
                e = self.s[self.i]
                if e == "x":
                    out.append(chr(int(self.s[self.i + 1:self.i + 3], 16)))
                    self.i += 2
                elif e == "u":
                    out.append(chr(int(self.s[self.i + 1:self.i + 5], 16)))
                    self.i += 4
                else:
                    out.append(_ESC.get(e, e))
            else:
                out.append(c)
            self.i += 1
        if self.i >= len(self.s):
            raise GrammarError("unterminated string literal")
        self.i += 1
        return "".join(out)

    def _charclass(self) -> _CharSet:
        self.i += 1
        neg = self.s[self.i] == "^"
        if neg:
            self.i += 1
        ranges = []

        def one() -> int:
            c = self.s[self.i]
            if c == "\\":
                self.i += 1
                e = self.s[self.i]
                if e == "x":
                    v = int(self.s[self.i + 1:self.i + 3], 16)
                    self.i += 3
                    return v
                if e == "u":
                    v = int(self.s[self.i + 1:self.i + 5], 16)
                    self.i += 5
                    return v
                self.i += 1
                return ord(_ESC.get(e, e))
            self.i += 1
            return ord(c)
        while self.i < len(self.s) and self.s[self.i] != "]":
            lo = one()
            if self.s[self.i] == "-" and self.s[self.i + 1] != "]":
                self.i += 1
                hi = one()
            else:
                hi = lo
            ranges.append((lo, hi))
        if self.i >= len(self.s):
            raise GrammarError("unterminated character class")
        self.i += 1
        return _CharSet(ranges, neg)


# ---- Earley recogniser -----------------------------------------------------------------------------------------------

_Item = Tuple[str, int, int, int]          # (rule, alternative index, dot, origin set)


class EbnfMatcher:
    def __init__(self, grammar: str):
        self.rules = _Parser(grammar).parse()
        self.nullable = self._nullable()
        self._text = ""
        self._chart: List[FrozenSet[_Item]] = [self._close({("root", a, 0, 0) for a in range(len(self.rules["root"]))}, [], 0)]

    def _nullable(self) -> Set[str]:
        out: Set[str] = set()
        changed = True
        while changed:
            changed = False
            for name, alts in self.rules.items():
                if name not in out and any(all(isinstance(s, str) and s in out for s in alt) for alt in alts):
                    out.add(name)
                    changed = True
        return out

    def _close(self, seed: Set[_Item], chart: List[FrozenSet[_Item]], k: int) -> FrozenSet[_Item]:
        """Predict / complete to a fixed point for set ``k`` (``chart`` holds sets 0..k-1)."""
        items, work = set(seed), list(seed)
        while work:
            rule, a, dot, origin = work.pop()
            rhs = self.rules[rule][a]
            if dot < len(rhs):
                sym = rhs[dot]
                if isinstance(sym, str):
                    for b in range(len(self.rules[sym])):
                        it = (sym, b, 0, k)
                        if it not in items:
                            items.add(it)
                            work.append(it)
                    if sym in self.nullable:
                        it = (rule, a, dot + 1, origin)
                        if it not in items:
                            items.add(it)
                            work.append(it)
            else:
                parents = items if origin == k else chart[origin]
                for pr, pa, pd, po in list(parents):
                    prhs = self.rules[pr][pa]
                    if pd < len(prhs) and prhs[pd] == rule:
                        it = (pr, pa, pd + 1, po)
                        if it not in items:
                            items.add(it)
                            work.append(it)
        return frozenset(items)

    def _step(self, chart: List[FrozenSet[_Item]], ch: str) -> Optional[FrozenSet[_Item]]:
        k = len(chart)
        seed = set()
        for rule, a, dot, origin in chart[-1]:
            rhs = self.rules[rule][a]
            if dot < len(rhs) and not isinstance(rhs[dot], str) and ch in rhs[dot]:
                seed.add((rule, a, dot + 1, origin))
        if not seed:
            return None
        return self._close(seed, chart, k)

    def _chart_for(self, text: str) -> Optional[List[FrozenSet[_Item]]]:
        if text.startswith(self._text):
            chart, rest = list(self._chart), text[len(self._text):]
        else:
            chart, rest = [self._chart[0]], text
            if self._text.startswith(text):                       # a shorter prefix of what we hold
                return self._chart[:len(text) + 1]
        for ch in rest:
            nxt = self._step(chart, ch)
            if nxt is None:
                return None
            chart.append(nxt)
        return chart

    def viable(self, text: str) -> bool:
        return self._chart_for(text) is not None

    def complete(self, text: str) -> bool:
        chart = self._chart_for(text)
        if chart is None:
            return False
        return any(rule == "root" and origin == 0 and dot == len(self.rules[rule][a]) for rule, a, dot, origin in chart[-1])

    def commit(self, text: str) -> None:
        """Remember the chart of ``text`` (the decoder calls this after a token is accepted)."""
        chart = self._chart_for(text)
        if chart is None:
            raise GrammarError(f"text {text!r} is not a prefix of the grammar's language")
        self._text, self._chart = text, chart

    def next_chars(self, text: str) -> Optional[List[_CharSet]]:
        chart = self._chart_for(text)
        if chart is None:
            return None
        out = []
        for rule, a, dot, _ in chart[-1]:
            rhs = self.rules[rule][a]
            if dot < len(rhs) and not isinstance(rhs[dot], str):
                out.append(rhs[dot])
        return out

    def forced_continuation(self, text: str, limit: int = 256) -> str:
        """Characters the grammar forces after ``text`` (exactly one possible next character, repeatedly, and the text
        is not already a complete sentence): they can be appended without asking the model."""
        out = ""
        while len(out) < limit and not self.complete(text + out):
            sets = self.next_chars(text + out)
            if not sets:
                break
            singles = {s.sample() for s in sets}
            if len(singles) != 1 or None in singles:
                break
            out += singles.pop()
        return out


# ---- structural tags -------------------------------------------------------------------------------------------------

class StructuralTagMatcher:
    def __init__(self, spec: dict):
        from .guided import _RegexMatcher, schema_to_regex
        self.structs = []
        for st in spec.get("structures") or []:
            if "begin" not in st or "end" not in st:
                raise GrammarError("every structure needs 'begin' and 'end'")
            body = _RegexMatcher(schema_to_regex(st["schema"])) if st.get("schema") else None
            self.structs.append((st["begin"], body, st["end"]))
        self.triggers = list(spec.get("triggers") or [])
        if not self.structs or not self.triggers:
            raise GrammarError("a structural tag needs structures and triggers")
        for b, _, _ in self.structs:
            if not any(b.startswith(t) for t in self.triggers):
                raise GrammarError(f"structure {b!r} starts with none of the triggers")

    def _walk(self, text: str) -> Tuple[bool, bool]:
        """(viable, complete).  Free text may not contain a trigger except as the start of a structure."""
        i = 0
        while True:
            hit = min((j for j in (text.find(t, i) for t in self.triggers) if j != -1), default=-1)
            if hit == -1:
                return True, True                      # free text (a partial trigger at the end is still free text)
            rest = text[hit:]
            progressed = False
            partial = False
            for begin, body, end in self.structs:
                if rest.startswith(begin):
                    inner = rest[len(begin):]
                    # the body ends at the first position where the body is complete and the end string follows
                    done_at = -1
                    if body is None:
                        e = inner.find(end)
                        if e != -1:
                            done_at = e
                    else:
                        for e in range(len(inner) + 1):
                            if inner.startswith(end, e) and body.complete(inner[:e]):
                                done_at = e
                                break
                    if done_at >= 0:
                        i = hit + len(begin) + done_at + len(end)
                        progressed = True
                        break
                    # still inside: the body (plus possibly a partial end string) must be viable
                    for e in range(len(inner), -1, -1):
                        tail = inner[e:]
                        if end.startswith(tail) and (body.complete(inner[:e]) if (body is not None and tail) else
                                                     (body.viable(inner[:e]) if body is not None else True)):
                            partial = True
                            break
                    if body is None:
                        partial = True
                elif begin.startswith(rest):
                    partial = True                     # the begin string itself is still being written
            if progressed:
                continue
            return partial, False

    def viable(self, text: str) -> bool:
        return self._walk(text)[0]

    def complete(self, text: str) -> bool:
        return self._walk(text)[1]
