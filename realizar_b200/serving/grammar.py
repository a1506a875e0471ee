"""Constrained generation: GBNF grammars, JSON-schema → grammar, an incremental matcher over
characters, and per-step token masks for the sampler; tool-call schemas on top.

The matcher keeps a set of parse stacks (a nondeterministic push-down automaton).  Each stack is a
tuple of frames ``(rule_id, alt_index, position)``; advancing by one character expands
non-terminals until every stack's next element is a terminal, then keeps the stacks whose
terminal accepts the character.  A token is allowed when all of its characters can be consumed in
sequence.  Reference parity: ``Grammar`` / ``GrammarStateMachine`` / ``GrammarTokenMasker`` /
``JsonSchemaType`` / ``ToolDefinition`` (src/grammar/mod.rs:21-262 and siblings)."""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Dict, FrozenSet, List, Optional, Sequence, Tuple, Union

import numpy as np

# elements: ("char", frozenset|None, ranges, negated) | ("ref", rule_name)
CharEl = Tuple[str, Tuple[Tuple[int, int], ...], bool]


@dataclass(frozen=True)
class El:
    kind: str                                   # "chars" | "ref"
    ranges: Tuple[Tuple[int, int], ...] = ()
    negated: bool = False
    ref: str = ""

    def accepts(self, ch: str) -> bool:
        c = ord(ch)
        hit = any(lo <= c <= hi for lo, hi in self.ranges)
        return hit != self.negated


class GrammarError(ValueError):
    pass


class Grammar:
    def __init__(self, root: str = "root"):
        self.rules: Dict[str, List[List[El]]] = {}
        self.root = root
        self._anon = 0

    def add_rule(self, name: str, alternatives: List[List[El]]) -> None:
        self.rules.setdefault(name, []).extend(alternatives)

    def fresh(self, base: str) -> str:
        self._anon += 1
        return f"{base}_{self._anon}"

    def validate(self) -> None:
        if self.root not in self.rules:
            raise GrammarError(f"grammar has no '{self.root}' rule")
        for name, alts in self.rules.items():
            for alt in alts:
                for el in alt:
                    if el.kind == "ref" and el.ref not in self.rules:
                        raise GrammarError(f"rule '{name}' references undefined rule '{el.ref}'")

    # -- GBNF ---------------------------------------------------------------------------------
    @classmethod
    def from_gbnf(cls, text: str, root: str = "root") -> "Grammar":
        g = cls(root)
        _GbnfParser(text, g).parse()
        g.validate()
        return g


def lit(s: str) -> List[El]:
    return [El("chars", ((ord(c), ord(c)),)) for c in s]


def ref(name: str) -> El:
    return El("ref", ref=name)


class _GbnfParser:
    def __init__(self, text: str, g: Grammar):
        self.s, self.i, self.g = text, 0, g

    def ws(self, newlines: bool = True) -> None:
        while self.i < len(self.s):
            c = self.s[self.i]
            if c == "#":
                while self.i < len(self.s) and self.s[self.i] != "\n":
                    self.i += 1
            elif c in " \t" or (newlines and c in "\r\n"):
                self.i += 1
            else:
                break

    def name(self) -> str:
        j = self.i
        while self.i < len(self.s) and (self.s[self.i].isalnum() or self.s[self.i] in "-_"):
            self.i += 1
        if j == self.i:
            raise GrammarError(f"expected a rule name at offset {j}")
        return self.s[j:self.i]

    def parse(self) -> None:
        self.ws()
        while self.i < len(self.s):
            n = self.name()
            self.ws(False)
            if not self.s.startswith("::=", self.i):
                raise GrammarError(f"expected '::=' after '{n}'")
            self.i += 3
            self.g.add_rule(n, self.alternatives(n))
            self.ws()

    def alternatives(self, rule: str) -> List[List[El]]:
        alts = [self.sequence(rule)]
        while True:
            self.ws(False)
            # a line break ends the rule unless the next non-blank token is '|'
            save = self.i
            self.ws(True)
            if self.i < len(self.s) and self.s[self.i] == "|":
                self.i += 1
                alts.append(self.sequence(rule))
            else:
                self.i = save
                return alts

    def escape(self) -> str:
        c = self.s[self.i]
        self.i += 1
        if c != "\\":
            return c
        e = self.s[self.i]
        self.i += 1
        if e == "x":
            v = self.s[self.i:self.i + 2]; self.i += 2
            return chr(int(v, 16))
        if e == "u":
            v = self.s[self.i:self.i + 4]; self.i += 4
            return chr(int(v, 16))
        return {"n": "\n", "r": "\r", "t": "\t"}.get(e, e)

    def sequence(self, rule: str) -> List[El]:
        seq: List[El] = []
        while True:
            self.ws(False)
            if self.i >= len(self.s):
                return seq
            c = self.s[self.i]
            start = len(seq)
            if c == '"':
                self.i += 1
                while self.s[self.i] != '"':
                    ch = self.escape()
                    seq.append(El("chars", ((ord(ch), ord(ch)),)))
                self.i += 1
            elif c == "[":
                self.i += 1
                neg = self.s[self.i] == "^"
                self.i += neg
                ranges = []
                while self.s[self.i] != "]":
                    lo = self.escape()
                    hi = lo
                    if self.s[self.i] == "-" and self.s[self.i + 1] != "]":
                        self.i += 1
                        hi = self.escape()
                    ranges.append((ord(lo), ord(hi)))
                self.i += 1
                seq.append(El("chars", tuple(ranges), neg))
            elif c == ".":
                self.i += 1
                seq.append(El("chars", ((0, 0x10FFFF),)))
            elif c == "(":
                self.i += 1
                sub = self.g.fresh(rule)
                self.g.add_rule(sub, self.alternatives(rule))
                self.ws()
                if self.s[self.i] != ")":
                    raise GrammarError(f"expected ')' at offset {self.i}")
                self.i += 1
                seq.append(ref(sub))
            elif c.isalnum() or c in "-_":
                save = self.i
                n = self.name()
                self.ws(False)
                if self.s.startswith("::=", self.i):        # start of the next rule
                    self.i = save
                    return seq
                seq.append(ref(n))
            else:
                return seq
            # postfix operators apply to the last item (a literal string counts as one group)
            if self.i < len(self.s) and self.s[self.i] in "*+?":
                op = self.s[self.i]
                self.i += 1
                item = seq[start:]
                del seq[start:]
                sub = self.g.fresh(rule)
                if op == "*":
                    self.g.add_rule(sub, [item + [ref(sub)], []])
                elif op == "+":
                    self.g.add_rule(sub, [item + [ref(sub)], item])
                else:
                    self.g.add_rule(sub, [item, []])
                seq.append(ref(sub))


Stack = Tuple[Tuple[str, int, int], ...]


class GrammarMatcher:
    """Incremental recogniser.  ``advance(text)`` consumes characters; ``is_complete`` tells whether
    the consumed text is a full sentence of the grammar; ``accepts(text)`` probes without consuming."""

    MAX_STACKS = 4096

    def __init__(self, grammar: Grammar):
        self.g = grammar
        self.stacks: FrozenSet[Stack] = self._expand({((grammar.root, a, 0),) for a in range(len(grammar.rules[grammar.root]))})

    def _expand(self, stacks) -> FrozenSet[Stack]:
        out, seen, todo = set(), set(), list(stacks)
        while todo:
            st = todo.pop()
            if st in seen:
                continue
            seen.add(st)
            if len(seen) > self.MAX_STACKS * 4:
                raise GrammarError("grammar expansion too large (left recursion?)")
            if not st:
                out.add(st)
                continue
            rule, alt, pos = st[-1]
            seq = self.g.rules[rule][alt]
            if pos >= len(seq):
                todo.append(self._pop(st))
                continue
            el = seq[pos]
            if el.kind == "chars":
                out.add(st)
            else:
                base = st[:-1] + ((rule, alt, pos + 1),)
                for a in range(len(self.g.rules[el.ref])):
                    todo.append(base + ((el.ref, a, 0),))
        return frozenset(out)

    @staticmethod
    def _pop(st: Stack) -> Stack:
        return st[:-1]

    def _step(self, stacks: FrozenSet[Stack], ch: str) -> FrozenSet[Stack]:
        nxt = set()
        for st in stacks:
            if not st:
                continue
            rule, alt, pos = st[-1]
            if self.g.rules[rule][alt][pos].accepts(ch):
                nxt.add(st[:-1] + ((rule, alt, pos + 1),))
        return self._expand(nxt) if nxt else frozenset()

    def accepts(self, text: str) -> bool:
        s = self.stacks
        for ch in text:
            s = self._step(s, ch)
            if not s:
                return False
        return True

    def advance(self, text: str) -> bool:
        s = self.stacks
        for ch in text:
            s = self._step(s, ch)
            if not s:
                return False
        self.stacks = s
        return True

    @property
    def is_complete(self) -> bool:
        return () in self.stacks

    @property
    def is_dead(self) -> bool:
        return not self.stacks

    def allowed_first_chars(self, probe: Sequence[str]) -> List[str]:
        return [c for c in probe if self._step(self.stacks, c)]


class GrammarTokenMasker:
    """Turns matcher state into a vocabulary mask.  Token strings are bucketed by first character so
    that a step only tests tokens whose first character is viable."""

    def __init__(self, grammar: Grammar, vocab: Sequence[str], eos_token_id: Optional[int] = None):
        self.matcher = GrammarMatcher(grammar)
        self.vocab = list(vocab)
        self.eos = eos_token_id
        self.by_first: Dict[str, List[int]] = {}
        for i, t in enumerate(self.vocab):
            if t and i != eos_token_id:
                self.by_first.setdefault(t[0], []).append(i)

    def mask(self) -> np.ndarray:
        m = np.zeros(len(self.vocab), dtype=bool)
        for ch, ids in self.by_first.items():
            if not self.matcher._step(self.matcher.stacks, ch):
                continue
            for i in ids:
                if len(self.vocab[i]) == 1 or self.matcher.accepts(self.vocab[i]):
                    m[i] = True
        if self.eos is not None and self.matcher.is_complete:
            m[self.eos] = True
        return m

    def apply(self, logits: np.ndarray) -> np.ndarray:
        m = self.mask()
        if not m.any():
            return logits
        out = np.where(m[: logits.shape[-1]], logits, -np.inf)
        return out

    def accept_token(self, token_id: int) -> bool:
        if token_id == self.eos:
            return self.matcher.is_complete
        return self.matcher.advance(self.vocab[token_id])


# -- JSON schema → grammar -----------------------------------------------------------------------
_JSON_PRIMS = r'''
ws ::= [ \t\n]*
string ::= "\"" char* "\""
char ::= [^"\\\x00-\x1f] | "\\" (["\\/bfnrt] | "u" hex hex hex hex)
hex ::= [0-9a-fA-F]
integer ::= "-"? ("0" | [1-9] [0-9]*)
number ::= integer ("." [0-9]+)? ([eE] [-+]? [0-9]+)?
boolean ::= "true" | "false"
null ::= "null"
value ::= object | array | string | number | boolean | null
object ::= "{" ws (string ws ":" ws value (ws "," ws string ws ":" ws value)*)? ws "}"
array ::= "[" ws (value (ws "," ws value)*)? ws "]"
'''


def json_schema_to_gbnf(schema: dict) -> str:
    rules: List[str] = []
    counter = [0]

    def emit(body: str) -> str:
        counter[0] += 1
        n = f"s{counter[0]}"
        rules.append(f"{n} ::= {body}")
        return n

    def q(s: str) -> str:
        return '"' + json.dumps(s).replace("\\", "\\\\").replace('"', '\\"') + '"'

    def visit(s: dict) -> str:
        if "enum" in s:
            return emit(" | ".join(q(v) if isinstance(v, str) else f'"{json.dumps(v)}"' for v in s["enum"]))
        if "const" in s:
            return emit(q(s["const"]) if isinstance(s["const"], str) else f'"{json.dumps(s["const"])}"')
        if "anyOf" in s or "oneOf" in s:
            return emit(" | ".join(visit(x) for x in s.get("anyOf", s.get("oneOf"))))
        t = s.get("type")
        if isinstance(t, list):
            return emit(" | ".join(visit({**s, "type": x}) for x in t))
        if t == "object":
            props = s.get("properties", {})
            if not props:
                return "object"
            req = set(s.get("required", list(props)))
            parts, first = [], True
            for k, v in props.items():
                item = f'{q(k)} ws ":" ws {visit(v)}'
                if k in req:
                    parts.append(item if first else f'ws "," ws {item}')
                    first = False
                else:
                    # optional properties are allowed only in declaration order
                    parts.append(f'({item})?' if first else f'(ws "," ws {item})?')
            return emit('"{" ws ' + " ".join(parts) + ' ws "}"')
        if t == "array":
            item = visit(s["items"]) if "items" in s else "value"
            return emit(f'"[" ws ({item} (ws "," ws {item})*)? ws "]"')
        return {"string": "string", "integer": "integer", "number": "number", "boolean": "boolean", "null": "null"}.get(t, "value")

    top = visit(schema)
    return f"root ::= ws {top} ws\n" + "\n".join(rules) + _JSON_PRIMS


def grammar_from_json_schema(schema: dict) -> Grammar:
    return Grammar.from_gbnf(json_schema_to_gbnf(schema))


# -- tool calls -----------------------------------------------------------------------------------------
@dataclass
class ToolDefinition:
    name: str
    description: str = ""
    parameters: dict = field(default_factory=lambda: {"type": "object", "properties": {}})


@dataclass
class ToolCall:
    name: str
    arguments: dict


def tool_call_grammar(tools: Sequence[ToolDefinition]) -> Grammar:
    """``{"name": "<tool>", "arguments": {...}}`` with the arguments constrained per tool."""
    schema = {"anyOf": [{"type": "object", "properties": {"name": {"const": t.name}, "arguments": t.parameters}, "required": ["name", "arguments"]} for t in tools]}
    return grammar_from_json_schema(schema)


def parse_tool_call(text: str, tools: Sequence[ToolDefinition]) -> Optional[ToolCall]:
    try:
        start = text.index("{")
        obj = json.loads(text[start:text.rindex("}") + 1])
    except ValueError:
        return None
    if not isinstance(obj, dict) or obj.get("name") not in {t.name for t in tools} or not isinstance(obj.get("arguments"), dict):
        return None
    return ToolCall(obj["name"], obj["arguments"])
