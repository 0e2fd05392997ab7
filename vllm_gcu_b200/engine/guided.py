"""Grammar-guided decoding: regular expressions and JSON schemas as token masks.

The reference serves guided requests through the structured-output backends of the vLLM it
plugs into and ships a benchmark for them (benchmarks/benchmark_guided.py); this engine has
its own small backend.  A pattern is compiled once into an automaton over characters
(Thompson construction, subset construction done lazily).  The vocabulary is indexed as a
trie, and for every automaton state that a request reaches the trie is walked once to find
the tokens whose whole text keeps the automaton alive, together with the state each of them
leads to.  The sampler then sees, per step, the list of permitted token ids
(``SamplingParams.allowed_next``): everything else is masked to -inf before sampling.

Supported syntax: literals, ``.``, escapes (``\\d \\w \\s \\D \\W \\S`` and escaped
punctuation), classes ``[a-z0-9_]`` / ``[^...]``, groups, ``|``, ``* + ?`` and ``{m}``,
``{m,}``, ``{m,n}``.  The match is anchored at both ends.  ``json_schema_to_regex`` covers
objects (properties in declaration order), arrays, strings (``enum``, ``pattern``,
``minLength`` / ``maxLength``), integers, numbers, booleans, null, ``const``, ``anyOf``.
"""
from __future__ import annotations

import json
import re as _re
from typing import Optional, Sequence

_MAXC = 0x10FFFF


class CharSet:
    """A set of characters as sorted, disjoint inclusive ranges."""
    __slots__ = ("ranges",)

    def __init__(self, ranges):
        rs = sorted((int(a), int(b)) for a, b in ranges if a <= b)
        out: list[tuple[int, int]] = []
        for a, b in rs:
            if out and a <= out[-1][1] + 1:
                out[-1] = (out[-1][0], max(out[-1][1], b))
            else:
                out.append((a, b))
        self.ranges = tuple(out)

    def negate(self) -> "CharSet":
        out, prev = [], 0
        for a, b in self.ranges:
            if a > prev:
                out.append((prev, a - 1))
            prev = b + 1
        if prev <= _MAXC:
            out.append((prev, _MAXC))
        return CharSet(out)

    def union(self, other: "CharSet") -> "CharSet":
        return CharSet(self.ranges + other.ranges)

    def __contains__(self, ch: str) -> bool:
        c = ord(ch)
        lo, hi = 0, len(self.ranges)
        while lo < hi:
            mid = (lo + hi) >> 1
            a, b = self.ranges[mid]
            if c < a:
                hi = mid
            elif c > b:
                lo = mid + 1
            else:
                return True
        return False


_DIGIT = CharSet([(48, 57)])
_WORD = CharSet([(48, 57), (65, 90), (95, 95), (97, 122)])
_SPACE = CharSet([(9, 13), (32, 32)])
_ANY = CharSet([(0, 9), (11, _MAXC)])            # '.' does not match a newline
_ESC_CLASS = {"d": _DIGIT, "w": _WORD, "s": _SPACE, "D": _DIGIT.negate(), "W": _WORD.negate(),
              "S": _SPACE.negate()}
_ESC_CHAR = {"n": "\n", "t": "\t", "r": "\r", "f": "\f", "v": "\v", "0": "\0"}


class RegexSyntaxError(ValueError):
    pass


# --- parser: pattern -> tree ----------------------------------------------------------------
# nodes: ("set", CharSet) | ("cat", [nodes]) | ("alt", [nodes]) | ("rep", node, lo, hi|None)
class _Parser:
    def __init__(self, pattern: str):
        self.p, self.i = pattern, 0

    def parse(self):
        node = self._alt()
        if self.i != len(self.p):
            raise RegexSyntaxError(f"unexpected {self.p[self.i]!r} at {self.i}")
        return node

    def _peek(self) -> Optional[str]:
        return self.p[self.i] if self.i < len(self.p) else None

    def _alt(self):
        parts = [self._cat()]
        while self._peek() == "|":
            self.i += 1
            parts.append(self._cat())
        return parts[0] if len(parts) == 1 else ("alt", parts)

    def _cat(self):
        items = []
        while self._peek() is not None and self._peek() not in "|)":
            items.append(self._repeat())
        return ("cat", items)

    def _repeat(self):
        node = self._atom()
        while True:
            c = self._peek()
            if c == "*":
                node, self.i = ("rep", node, 0, None), self.i + 1
            elif c == "+":
                node, self.i = ("rep", node, 1, None), self.i + 1
            elif c == "?":
                node, self.i = ("rep", node, 0, 1), self.i + 1
            elif c == "{":
                m = _re.compile(r"\{(\d+)(,(\d*))?\}").match(self.p, self.i)
                if not m:
                    raise RegexSyntaxError(f"bad quantifier at {self.i}")
                lo = int(m.group(1))
                hi = lo if m.group(2) is None else (int(m.group(3)) if m.group(3) else None)
                if hi is not None and hi < lo:
                    raise RegexSyntaxError(f"bad quantifier bounds at {self.i}")
                node, self.i = ("rep", node, lo, hi), m.end()
            else:
                return node
            if self._peek() == "?":          # lazy quantifiers accept the same language
                self.i += 1

    def _escape(self) -> CharSet:
        c = self._peek()
        if c is None:
            raise RegexSyntaxError("dangling backslash")
        self.i += 1
        if c in _ESC_CLASS:
            return _ESC_CLASS[c]
        if c == "x":
            h = self.p[self.i:self.i + 2]
            self.i += 2
            return CharSet([(int(h, 16),) * 2])
        if c == "u":
            h = self.p[self.i:self.i + 4]
            self.i += 4
            return CharSet([(int(h, 16),) * 2])
        ch = _ESC_CHAR.get(c, c)
        return CharSet([(ord(ch), ord(ch))])

    def _atom(self):
        c = self._peek()
        self.i += 1
        if c == "(":
            if self.p.startswith("?:", self.i):
                self.i += 2
            elif self._peek() == "?":
                raise RegexSyntaxError("look-around and named groups are not supported")
            node = self._alt()
            if self._peek() != ")":
                raise RegexSyntaxError("missing )")
            self.i += 1
            return node
        if c == "[":
            return ("set", self._klass())
        if c == ".":
            return ("set", _ANY)
        if c == "\\":
            return ("set", self._escape())
        if c in "^$":
            return ("cat", [])               # the match is anchored anyway
        if c in "*+?{":
            raise RegexSyntaxError(f"nothing to repeat at {self.i - 1}")
        return ("set", CharSet([(ord(c), ord(c))]))

    def _klass(self) -> CharSet:
        neg = self._peek() == "^"
        if neg:
            self.i += 1
        acc = CharSet([])
        first = True
        while True:
            c = self._peek()
            if c is None:
                raise RegexSyntaxError("missing ]")
            if c == "]" and not first:
                self.i += 1
                break
            first = False
            self.i += 1
            if c == "\\":
                cs = self._escape()
                if len(cs.ranges) != 1 or cs.ranges[0][0] != cs.ranges[0][1]:
                    acc = acc.union(cs)
                    continue
                lo = cs.ranges[0][0]
            else:
                lo = ord(c)
            if self._peek() == "-" and self.i + 1 < len(self.p) and self.p[self.i + 1] != "]":
                self.i += 1
                d = self._peek()
                self.i += 1
                if d == "\\":
                    hs = self._escape()
                    hi = hs.ranges[0][0]
                else:
                    hi = ord(d)
                if hi < lo:
                    raise RegexSyntaxError("bad range in class")
                acc = acc.union(CharSet([(lo, hi)]))
            else:
                acc = acc.union(CharSet([(lo, lo)]))
        return acc.negate() if neg else acc


# --- automaton --------------------------------------------------------------------------------
class _NFA:
    def __init__(self):
        self.eps: list[list[int]] = []
        self.edges: list[list[tuple[CharSet, int]]] = []

    def new(self) -> int:
        self.eps.append([])
        self.edges.append([])
        return len(self.eps) - 1

    def build(self, node, max_states: int) -> tuple[int, int]:
        if len(self.eps) > max_states:
            raise RegexSyntaxError("pattern too large (bounded repetitions expand)")
        kind = node[0]
        if kind == "set":
            a, b = self.new(), self.new()
            self.edges[a].append((node[1], b))
            return a, b
        if kind == "cat":
            a = b = self.new()
            for it in node[1]:
                s, e = self.build(it, max_states)
                self.eps[b].append(s)
                b = e
            return a, b
        if kind == "alt":
            a, b = self.new(), self.new()
            for it in node[1]:
                s, e = self.build(it, max_states)
                self.eps[a].append(s)
                self.eps[e].append(b)
            return a, b
        _, sub, lo, hi = node
        a = b = self.new()
        for _i in range(lo):
            s, e = self.build(sub, max_states)
            self.eps[b].append(s)
            b = e
        if hi is None:
            s, e = self.build(sub, max_states)
            loop = self.new()
            self.eps[b].append(loop)
            self.eps[loop].append(s)
            self.eps[e].append(loop)
            b = loop
        else:
            end = self.new()
            for _i in range(hi - lo):
                s, e = self.build(sub, max_states)
                self.eps[b].append(end)
                self.eps[b].append(s)
                b = e
            self.eps[b].append(end)
            b = end
        return a, b


class _Trie:
    __slots__ = ("children", "tokens")

    def __init__(self):
        self.children: dict[str, _Trie] = {}
        self.tokens: list[int] = []


class RegexGuide:
    """Compiled pattern + vocabulary.  Shared by all requests that use the same pattern; the
    per-request position is a ``GuideCursor``."""

    def __init__(self, pattern: str, vocab: Sequence[Optional[str]], eos_token_id: Optional[int],
                 max_nfa_states: int = 200_000):
        self.pattern = pattern
        self.eos = eos_token_id
        nfa = _NFA()
        start, accept = nfa.build(_Parser(pattern).parse(), max_nfa_states)
        self._nfa, self._accept = nfa, accept
        self._ids: dict[frozenset, int] = {}
        self._sets: list[frozenset] = []
        self._step: list[dict[str, int]] = []          # per state: char -> next state (-1 dead)
        self._tok: list[Optional[dict[int, int]]] = [] # per state: token id -> next state
        self.start = self._intern(self._closure({start}))
        self._root = _Trie()
        for tid, text in enumerate(vocab):
            if not text or tid == eos_token_id:
                continue
            node = self._root
            for ch in text:
                nxt = node.children.get(ch)
                if nxt is None:
                    nxt = node.children[ch] = _Trie()
                node = nxt
            node.tokens.append(tid)

    # subset construction, on demand
    def _closure(self, states) -> frozenset:
        seen, stack = set(states), list(states)
        while stack:
            s = stack.pop()
            for t in self._nfa.eps[s]:
                if t not in seen:
                    seen.add(t)
                    stack.append(t)
        return frozenset(seen)

    def _intern(self, st: frozenset) -> int:
        i = self._ids.get(st)
        if i is None:
            i = self._ids[st] = len(self._sets)
            self._sets.append(st)
            self._step.append({})
            self._tok.append(None)
        return i

    def step_char(self, state: int, ch: str) -> int:
        memo = self._step[state]
        nxt = memo.get(ch)
        if nxt is None:
            tgt = {t for s in self._sets[state] for cs, t in self._nfa.edges[s] if ch in cs}
            nxt = memo[ch] = self._intern(self._closure(tgt)) if tgt else -1
        return nxt

    def accepting(self, state: int) -> bool:
        return state >= 0 and self._accept in self._sets[state]

    def token_moves(self, state: int) -> dict[int, int]:
        """token id -> next state for every token whose text the automaton can consume."""
        moves = self._tok[state]
        if moves is None:
            moves = {}
            stack = [(self._root, state)]
            while stack:
                node, st = stack.pop()
                for ch, child in node.children.items():
                    nx = self.step_char(st, ch)
                    if nx < 0:
                        continue
                    for tid in child.tokens:
                        moves[tid] = nx
                    if child.children:
                        stack.append((child, nx))
            self._tok[state] = moves
        return moves

    def allowed(self, state: int) -> list[int]:
        if state < 0:
            return [self.eos] if self.eos is not None else []
        ids = sorted(self.token_moves(state))
        if self.accepting(state) and self.eos is not None:
            ids.append(self.eos)
        if not ids and self.eos is not None:
            ids = [self.eos]
        return ids

    def advance(self, state: int, token_id: int) -> int:
        if state < 0 or token_id == self.eos:
            return state
        return self.token_moves(state).get(token_id, -1)

    def exhausted(self, state: int) -> bool:
        """The pattern is matched and nothing can follow."""
        return state < 0 or (self.accepting(state) and not self.token_moves(state))

    def matches(self, text: str) -> bool:
        st = self.start
        for ch in text:
            st = self.step_char(st, ch)
            if st < 0:
                return False
        return self.accepting(st)


class GuideCursor:
    """Position of one request inside a ``RegexGuide``; follows the request's output."""

    def __init__(self, guide: RegexGuide):
        self.guide = guide
        self.n = 0
        self.state = guide.start

    def _sync(self, output_token_ids) -> None:
        if len(output_token_ids) < self.n:                 # request was rolled back
            self.n, self.state = 0, self.guide.start
        for t in output_token_ids[self.n:]:
            self.state = self.guide.advance(self.state, int(t))
        self.n = len(output_token_ids)

    def allowed_next(self, output_token_ids) -> list[int]:
        self._sync(output_token_ids)
        return self.guide.allowed(self.state)

    def finished(self, output_token_ids) -> bool:
        self._sync(output_token_ids)
        return self.guide.exhausted(self.state)


# --- JSON schema -> pattern ---------------------------------------------------------------------
_WS = r"[ \n\t]{0,2}"
_STR_INNER = r'([^"\\\x00-\x1f]|\\["\\/bfnrt]|\\u[0-9a-fA-F]{4})'
_INT = r"-?(0|[1-9][0-9]*)"
_NUM = _INT + r"(\.[0-9]+)?([eE][+-]?[0-9]+)?"


def _lit(value) -> str:
    return _re.escape(json.dumps(value, ensure_ascii=False))


def json_schema_to_regex(schema, depth: int = 0) -> str:
    """A pattern that accepts the JSON documents described by ``schema`` (dict or JSON text)."""
    if isinstance(schema, str):
        schema = json.loads(schema)
    if depth > 16:
        raise ValueError("schema nests too deeply")
    if schema is True or schema == {}:
        raise ValueError("an unconstrained sub-schema cannot be expressed as a regular pattern")
    if "$ref" in schema:
        raise ValueError("$ref is not supported")
    if "const" in schema:
        return _lit(schema["const"])
    if "enum" in schema:
        return "(" + "|".join(_lit(v) for v in schema["enum"]) + ")"
    for key in ("anyOf", "oneOf"):
        if key in schema:
            return "(" + "|".join(json_schema_to_regex(s, depth + 1) for s in schema[key]) + ")"
    t = schema.get("type")
    if isinstance(t, list):
        return "(" + "|".join(json_schema_to_regex({**schema, "type": x}, depth + 1)
                              for x in t) + ")"
    if t == "string":
        if "pattern" in schema:
            return '"' + schema["pattern"].lstrip("^").rstrip("$") + '"'
        lo, hi = schema.get("minLength"), schema.get("maxLength")
        if lo is None and hi is None:
            return '"' + _STR_INNER + '*"'
        return '"' + _STR_INNER + "{" + str(lo or 0) + "," + ("" if hi is None else str(hi)) + '}"'
    if t == "integer":
        return _INT
    if t == "number":
        return _NUM
    if t == "boolean":
        return "(true|false)"
    if t == "null":
        return "null"
    if t == "array":
        item = json_schema_to_regex(schema.get("items", {"type": "string"}), depth + 1)
        lo, hi = int(schema.get("minItems", 0)), schema.get("maxItems")
        more = "(" + _WS + "," + _WS + item + ")"
        if lo == 0:
            rest = "{0," + ("" if hi is None else str(max(int(hi) - 1, 0))) + "}"
            body = "(" + item + more + rest + ")?" if hi != 0 else ""
        else:
            rest = "{" + str(lo - 1) + "," + ("" if hi is None else str(int(hi) - 1)) + "}"
            body = item + more + rest
        return r"\[" + _WS + body + _WS + r"\]"
    if t == "object" or "properties" in schema:
        props = schema.get("properties", {})
        if not props:
            return r"\{" + _WS + r"\}"
        required = set(schema.get("required", props.keys()))
        if len(props) - len(required & set(props)) > 6:     # every optional one doubles the
            required = set(props.keys())                    # pattern: then all are emitted
        parts = []
        for i, (name, sub) in enumerate(props.items()):
            kv = _lit(name) + _WS + ":" + _WS + json_schema_to_regex(sub, depth + 1)
            parts.append((name in required, kv))
        # Optional properties may be left out; declaration order is kept.  The separator
        # belongs to the property that follows another one, so every subset is well formed
        # as long as the first emitted property carries no comma: expand on the first one.
        def seq(items, first: bool) -> str:
            if not items:
                return ""
            req, kv = items[0]
            head = kv if first else _WS + "," + _WS + kv
            with_it = head + seq(items[1:], False)
            if req:
                return with_it
            without = seq(items[1:], first)
            return "(" + with_it + "|" + without + ")"
        return r"\{" + _WS + seq(parts, True) + _WS + r"\}"
    raise ValueError(f"unsupported schema: {schema!r}")


def check_guided(guided_regex=None, guided_json=None) -> None:
    """Raises ValueError (``RegexSyntaxError``) for a pattern or schema the guide cannot be
    built from; cheap, so that a server can refuse the request before it reaches the engine."""
    if guided_json is not None:
        guided_regex = json_schema_to_regex(guided_json)
    if guided_regex is not None:
        _Parser(guided_regex).parse()


def vocabulary_of(tokenizer, vocab_size: int) -> list:
    """Token texts of a tokenizer, index = token id (None where a token cannot be used as
    text: specials, ids past the tokenizer's table, pieces that are not valid UTF-8 alone)."""
    out: list = [None] * vocab_size
    special = set(getattr(tokenizer, "all_special_ids", []) or [])
    n = min(vocab_size, int(getattr(tokenizer, "vocab_size", vocab_size)) or vocab_size)
    for tid in range(n):
        if tid in special:
            continue
        try:
            text = tokenizer.decode([tid])
        except Exception:
            continue
        if text and "�" not in text:
            out[tid] = text
    return out
