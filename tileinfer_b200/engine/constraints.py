"""Constrained decoding: logit bias, allow/deny lists, guided choice / JSON / regex.

Capabilities follow the reference (engine/constraints.py:1-914): additive logit bias, hard token
allow- and deny-lists, output restricted to one of several strings, to syntactically valid JSON, or
to a regular expression (literals, classes, \\d \\w \\s, ., * + ? {m,n}, groups, alternation), all
applied to the vocabulary shard a tensor-parallel rank owns (vocab_offset / vocab_shard).

The construction differs.  Every grammar is a *character automaton* with hashable states
(`start`, `step(state, ch)`, `accepting(state)`); one generic engine walks a trie of the decoded
vocabulary under that automaton to obtain the set of admissible tokens of a state, and memoises the
resulting mask per state.  Regular expressions compile to a Thompson NFA that is determinised lazily,
JSON is a small push-down automaton whose state is (stack, phase), and a choice list is a trie of the
choices.  As in the reference a `guided_json` schema (dict) selects JSON mode but is not enforced.
"""
from __future__ import annotations

import torch

NEG_INF = float("-inf")


# =============================================================================== vocabulary trie
class VocabIndex:
    """Decoded text of every token and a character trie over it (built once per tokenizer)."""
    _cache = {}

    def __init__(self, tokenizer):
        n = getattr(tokenizer, "vocab_size", None) or len(tokenizer)
        try:
            n = max(n, len(tokenizer))
        except TypeError:
            pass
        self.size = n
        special = set(getattr(tokenizer, "all_special_ids", []) or [])
        self.text = [""] * n
        for i in range(n):
            if i in special:
                continue
            try:
                s = tokenizer.decode([i], skip_special_tokens=False)
            except Exception:
                s = ""
            if "�" in s:
                s = ""
            self.text[i] = s
        # trie: node = [children dict, token id list]
        self.root = [{}, []]
        for i, s in enumerate(self.text):
            if not s:
                continue
            node = self.root
            for ch in s:
                nxt = node[0].get(ch)
                if nxt is None:
                    nxt = node[0][ch] = [{}, []]
                node = nxt
            node[1].append(i)

    @classmethod
    def get(cls, tokenizer) -> "VocabIndex":
        key = id(tokenizer)
        if key not in cls._cache:
            cls._cache[key] = cls(tokenizer)
        return cls._cache[key]

    def admissible(self, fsm, state) -> list:
        """Token ids whose whole text the automaton can consume from `state`."""
        out = []
        stack = [(self.root, state)]
        while stack:
            node, st = stack.pop()
            for ch, child in node[0].items():
                nst = fsm.step(st, ch)
                if nst is None:
                    continue
                if child[1]:
                    out.extend(child[1])
                if child[0]:
                    stack.append((child, nst))
        return out


# =============================================================================== regex automaton
class _Parser:
    """Recursive-descent regex parser producing a small AST of tuples."""

    def __init__(self, pattern: str):
        self.p, self.i = pattern, 0

    def peek(self):
        return self.p[self.i] if self.i < len(self.p) else None

    def take(self):
        ch = self.p[self.i]
        self.i += 1
        return ch

    def parse(self):
        node = self.alt()
        if self.i != len(self.p):
            raise ValueError(f"unbalanced ')' at {self.i} in regex {self.p!r}")
        return node

    def alt(self):
        branches = [self.concat()]
        while self.peek() == "|":
            self.take()
            branches.append(self.concat())
        return branches[0] if len(branches) == 1 else ("alt", branches)

    def concat(self):
        items = []
        while self.peek() is not None and self.peek() not in "|)":
            items.append(self.repeat())
        return ("cat", items)

    def repeat(self):
        atom = self.atom()
        while True:
            ch = self.peek()
            if ch == "*":
                self.take(); atom = ("rep", atom, 0, None)
            elif ch == "+":
                self.take(); atom = ("rep", atom, 1, None)
            elif ch == "?":
                self.take(); atom = ("rep", atom, 0, 1)
            elif ch == "{":
                j = self.p.find("}", self.i)
                body = self.p[self.i + 1:j] if j > 0 else ""
                parts = body.split(",")
                if j < 0 or not all(x.strip().isdigit() or x.strip() == "" for x in parts) or not parts[0].strip():
                    break
                self.i = j + 1
                lo = int(parts[0])
                hi = lo if len(parts) == 1 else (int(parts[1]) if parts[1].strip() else None)
                atom = ("rep", atom, lo, hi)
            else:
                break
            if self.peek() == "?":      # lazy quantifiers match the same language
                self.take()
        return atom

    _CLASSES = {
        "d": (False, [("0", "9")]),
        "w": (False, [("a", "z"), ("A", "Z"), ("0", "9"), ("_", "_")]),
        "s": (False, [(" ", " "), ("\t", "\t"), ("\n", "\n"), ("\r", "\r"), ("\f", "\f"), ("\v", "\v")]),
    }
    _ESC = {"n": "\n", "t": "\t", "r": "\r", "f": "\f", "v": "\v", "0": "\0"}

    def escape(self):
        ch = self.take()
        if ch.lower() in self._CLASSES and ch.lower() in "dws":
            neg, ranges = self._CLASSES[ch.lower()]
            return ("set", ch.isupper(), ranges)
        if ch in self._ESC:
            return ("set", False, [(self._ESC[ch],) * 2])
        if ch == "x":
            h = self.p[self.i:self.i + 2]
            self.i += 2
            return ("set", False, [(chr(int(h, 16)),) * 2])
        if ch == "u":
            h = self.p[self.i:self.i + 4]
            self.i += 4
            return ("set", False, [(chr(int(h, 16)),) * 2])
        return ("set", False, [(ch, ch)])

    def atom(self):
        ch = self.take()
        if ch == "(":
            if self.p.startswith("?:", self.i):
                self.i += 2
            elif self.p.startswith("?P<", self.i):
                self.i = self.p.index(">", self.i) + 1
            node = self.alt()
            if self.peek() != ")":
                raise ValueError(f"missing ')' in regex {self.p!r}")
            self.take()
            return node
        if ch == "[":
            neg = self.peek() == "^"
            if neg:
                self.take()
            ranges, first = [], True
            while True:
                if self.peek() is None:
                    raise ValueError(f"missing ']' in regex {self.p!r}")
                c = self.take()
                if c == "]" and not first:
                    break
                first = False
                if c == "\\":
                    _, n2, r2 = self.escape()
                    if n2:
                        raise ValueError("negated class escapes inside [] are not supported")
                    ranges.extend(r2)
                    continue
                if self.peek() == "-" and self.i + 1 < len(self.p) and self.p[self.i + 1] != "]":
                    self.take()
                    hi = self.take()
                    if hi == "\\":
                        hi = self.escape()[2][0][0]
                    ranges.append((c, hi))
                else:
                    ranges.append((c, c))
            return ("set", neg, ranges)
        if ch == ".":
            return ("set", True, [("\n", "\n")])
        if ch == "\\":
            return self.escape()
        if ch in "^$":
            return ("cat", [])          # anchors: the whole output is always matched
        return ("set", False, [(ch, ch)])


class RegexFSM:
    """Thompson NFA, determinised on demand.  A state is a frozenset of NFA node ids."""

    def __init__(self, pattern: str):
        self.pattern = pattern
        self.eps, self.edges = [], []       # per node: list of eps targets; list of (neg, ranges, target)
        ast = _Parser(pattern).parse()
        s, e = self._build(ast)
        self.final = e
        self.start = self._closure({s})
        self._trans = {}
        self._alive = {}

    def _node(self):
        self.eps.append([])
        self.edges.append([])
        return len(self.eps) - 1

    def _build(self, ast):
        kind = ast[0]
        if kind == "set":
            s, e = self._node(), self._node()
            self.edges[s].append((ast[1], ast[2], e))
            return s, e
        if kind == "cat":
            s = e = self._node()
            for item in ast[1]:
                s2, e2 = self._build(item)
                self.eps[e].append(s2)
                e = e2
            return s, e
        if kind == "alt":
            s, e = self._node(), self._node()
            for br in ast[1]:
                s2, e2 = self._build(br)
                self.eps[s].append(s2)
                self.eps[e2].append(e)
            return s, e
        if kind == "rep":
            _, sub, lo, hi = ast
            s = e = self._node()
            for _ in range(lo):
                s2, e2 = self._build(sub)
                self.eps[e].append(s2)
                e = e2
            if hi is None:
                s2, e2 = self._build(sub)
                self.eps[e].append(s2)
                self.eps[e2].append(s2)
                out = self._node()
                self.eps[e].append(out)
                self.eps[e2].append(out)
                e = out
            else:
                out = self._node()
                self.eps[e].append(out)
                for _ in range(hi - lo):
                    s2, e2 = self._build(sub)
                    self.eps[e].append(s2)
                    self.eps[e2].append(out)
                    e = e2
                e = out
            return s, e
        raise ValueError(kind)

    def _closure(self, nodes) -> frozenset:
        seen, todo = set(nodes), list(nodes)
        while todo:
            n = todo.pop()
            for t in self.eps[n]:
                if t not in seen:
                    seen.add(t)
                    todo.append(t)
        return frozenset(seen)

    @staticmethod
    def _in(neg, ranges, ch) -> bool:
        hit = any(lo <= ch <= hi for lo, hi in ranges)
        return hit != neg

    def step(self, state, ch):
        key = (state, ch)
        r = self._trans.get(key, 0)
        if r != 0:
            return r
        nxt = set()
        for n in state:
            for neg, ranges, t in self.edges[n]:
                if self._in(neg, ranges, ch):
                    nxt.add(t)
        r = self._closure(nxt) if nxt else None
        self._trans[key] = r
        return r

    def accepting(self, state) -> bool:
        return self.final in state

    def can_continue(self, state) -> bool:
        return any(self.edges[n] for n in state)


# =============================================================================== choice automaton
class ChoiceFSM:
    """State = the text produced so far (must stay a prefix of a choice)."""

    def __init__(self, choices):
        self.choices = [c for c in choices if c]
        if not self.choices:
            raise ValueError("guided_choice needs at least one non-empty string")
        self.prefixes = {c[:i] for c in self.choices for i in range(len(c) + 1)}
        self.full = set(self.choices)
        self.start = ""

    def step(self, state, ch):
        s = state + ch
        return s if s in self.prefixes else None

    def accepting(self, state) -> bool:
        return state in self.full

    def can_continue(self, state) -> bool:
        return any(c != state and c.startswith(state) for c in self.choices)


# =============================================================================== JSON automaton
class JsonFSM:
    """Push-down automaton for one JSON object.  State = (stack, phase, aux).

    stack is a string of 'O'/'A' (open containers).  Whitespace is limited to single characters
    between structural tokens so that a model cannot pad forever.  Nesting depth is capped.
    """
    MAX_DEPTH = 12
    WS = " \n\t"
    DIGITS = "0123456789"
    HEX = "0123456789abcdefABCDEF"

    def __init__(self, top_level: str = "object"):
        self.top = top_level
        self.start = ("", "top", 0)

    def accepting(self, state) -> bool:
        return state[1] == "done"

    def can_continue(self, state) -> bool:
        return state[1] != "done"

    # -- helpers
    def _after_value(self, stack):
        if not stack:
            return ("", "done", 0)
        return (stack, "after_o" if stack[-1] == "O" else "after_a", 0)

    def _value_start(self, stack, ch):
        if ch == '"':
            return (stack, "str", 0)
        if ch == "{":
            return (stack + "O", "obj_start", 0) if len(stack) < self.MAX_DEPTH else None
        if ch == "[":
            return (stack + "A", "arr_start", 0) if len(stack) < self.MAX_DEPTH else None
        if ch == "-":
            return (stack, "num_minus", 0)
        if ch == "0":
            return (stack, "num_zero", 0)
        if ch in "123456789":
            return (stack, "num_int", 0)
        for lit in ("true", "false", "null"):
            if ch == lit[0]:
                return (stack, "lit", lit[1:])
        return None

    def _end_number(self, stack, ch):
        """A number ends implicitly at the next structural character."""
        return self.step(self._after_value(stack), ch)

    def step(self, state, ch):
        stack, ph, aux = state
        ws = ch in self.WS
        if ph == "top":
            if ch == "{":
                return ("O", "obj_start", 0)
            if ch == "[" and self.top != "object":
                return ("A", "arr_start", 0)
            return None
        if ph == "done":
            return None
        if ph in ("str", "key"):
            if ch == '"':
                return (stack, "colon", 0) if ph == "key" else self._after_value(stack)
            if ch == "\\":
                return (stack, ph + "_esc", 0)
            return state if ch >= " " else None
        if ph in ("str_esc", "key_esc"):
            base = ph[:-4]
            if ch in '"\\/bfnrt':
                return (stack, base, 0)
            if ch == "u":
                return (stack, base + "_u", 4)
            return None
        if ph in ("str_u", "key_u"):
            if ch in self.HEX:
                return (stack, ph, aux - 1) if aux > 1 else (stack, ph[:-2], 0)
            return None
        if ph == "lit":
            if aux and ch == aux[0]:
                return (stack, "lit", aux[1:]) if len(aux) > 1 else self._after_value(stack)
            return None
        if ph == "num_minus":
            if ch == "0":
                return (stack, "num_zero", 0)
            return (stack, "num_int", 0) if ch in "123456789" else None
        if ph in ("num_zero", "num_int"):
            if ch in self.DIGITS and ph == "num_int":
                return state
            if ch == ".":
                return (stack, "num_frac0", 0)
            if ch in "eE":
                return (stack, "num_e", 0)
            return self._end_number(stack, ch)
        if ph == "num_frac0":
            return (stack, "num_frac", 0) if ch in self.DIGITS else None
        if ph == "num_frac":
            if ch in self.DIGITS:
                return state
            if ch in "eE":
                return (stack, "num_e", 0)
            return self._end_number(stack, ch)
        if ph == "num_e":
            if ch in "+-":
                return (stack, "num_esign", 0)
            return (stack, "num_exp", 0) if ch in self.DIGITS else None
        if ph == "num_esign":
            return (stack, "num_exp", 0) if ch in self.DIGITS else None
        if ph == "num_exp":
            return state if ch in self.DIGITS else self._end_number(stack, ch)
        # structural phases: one optional whitespace character (aux == 1 once used)
        if ws:
            return (stack, ph, 1) if aux == 0 else None
        if ph == "obj_start":
            if ch == '"':
                return (stack, "key", 0)
            if ch == "}":
                return self._after_value(stack[:-1])
            return None
        if ph == "need_key":
            return (stack, "key", 0) if ch == '"' else None
        if ph == "colon":
            return (stack, "value", 0) if ch == ":" else None
        if ph == "value":
            return self._value_start(stack, ch)
        if ph == "arr_start":
            if ch == "]":
                return self._after_value(stack[:-1])
            return self._value_start(stack, ch)
        if ph == "after_o":
            if ch == ",":
                return (stack, "need_key", 0)
            return self._after_value(stack[:-1]) if ch == "}" else None
        if ph == "after_a":
            if ch == ",":
                return (stack, "value", 0)
            return self._after_value(stack[:-1]) if ch == "]" else None
        return None


# =============================================================================== constraints
class Constraint:
    """Base class.  `apply` edits the logits row of one sequence IN PLACE.

    `logits` is the rank-local vocabulary shard [vocab_shard]; token id t lives at
    index t - vocab_offset."""
    stateful = False

    def initial_state(self):
        return None

    def apply(self, logits: torch.Tensor, state, vocab_offset: int = 0, eos_ids=()):
        raise NotImplementedError

    def advance(self, state, token_id: int):
        return state

    def is_complete(self, state) -> bool:
        return False


def _local(ids, vocab_offset, n):
    return [i - vocab_offset for i in ids if 0 <= i - vocab_offset < n]


class LogitBiasConstraint(Constraint):
    def __init__(self, bias: dict):
        self.bias = {int(k): float(v) for k, v in bias.items()}

    def apply(self, logits, state, vocab_offset=0, eos_ids=()):
        n = logits.shape[-1]
        for tok, b in self.bias.items():
            j = tok - vocab_offset
            if 0 <= j < n:
                logits[j] += b


class TokenMaskConstraint(Constraint):
    def __init__(self, allowed=None, banned=None):
        self.allowed = sorted(set(int(t) for t in (allowed or [])))
        self.banned = sorted(set(int(t) for t in (banned or [])))

    def apply(self, logits, state, vocab_offset=0, eos_ids=()):
        n = logits.shape[-1]
        if self.allowed:
            keep = torch.zeros(n, dtype=torch.bool, device=logits.device)
            idx = _local(self.allowed, vocab_offset, n)
            if idx:
                keep[torch.tensor(idx, device=logits.device)] = True
            logits.masked_fill_(~keep, NEG_INF)
        idx = _local(self.banned, vocab_offset, n)
        if idx:
            logits[torch.tensor(idx, device=logits.device)] = NEG_INF


class GrammarConstraint(Constraint):
    """Any character automaton driven through the vocabulary trie."""
    stateful = True

    def __init__(self, fsm, tokenizer):
        self.fsm = fsm
        self.vocab = VocabIndex.get(tokenizer)
        self._tokens = {}       # state -> sorted admissible token ids
        self._masks = {}        # (state, offset, n, device) -> bool mask

    def initial_state(self):
        return self.fsm.start

    def tokens_for(self, state) -> list:
        t = self._tokens.get(state)
        if t is None:
            t = self._tokens[state] = sorted(self.vocab.admissible(self.fsm, state))
        return t

    def apply(self, logits, state, vocab_offset=0, eos_ids=()):
        n = logits.shape[-1]
        key = (state, vocab_offset, n, str(logits.device))
        mask = self._masks.get(key)
        if mask is None:
            ids = list(self.tokens_for(state))
            if self.fsm.accepting(state):
                ids.extend(eos_ids)
            mask = torch.zeros(n, dtype=torch.bool)
            idx = _local(ids, vocab_offset, n)
            if idx:
                mask[torch.tensor(idx)] = True
            mask = mask.to(logits.device)
            if len(self._masks) > 4096:
                self._masks.clear()
            self._masks[key] = mask
        logits.masked_fill_(~mask, NEG_INF)

    def advance(self, state, token_id: int):
        if state is None:
            return None
        text = self.vocab.text[token_id] if 0 <= token_id < self.vocab.size else ""
        if not text:
            return state        # EOS / special token: the grammar does not move
        for ch in text:
            state = self.fsm.step(state, ch)
            if state is None:
                return None     # left the language (only possible with un-masked sampling)
        return state

    def is_complete(self, state) -> bool:
        if state is None:
            return True
        return self.fsm.accepting(state) and not (self.fsm.can_continue(state) and self.tokens_for(state))


class ChoiceConstraint(GrammarConstraint):
    def __init__(self, choices, tokenizer):
        super().__init__(ChoiceFSM(choices), tokenizer)


class JsonConstraint(GrammarConstraint):
    def __init__(self, schema, tokenizer):
        super().__init__(JsonFSM("object"), tokenizer)
        self.schema = schema if isinstance(schema, dict) else None   # stored, not enforced


class RegexConstraint(GrammarConstraint):
    def __init__(self, pattern: str, tokenizer):
        super().__init__(RegexFSM(pattern), tokenizer)


class CompositeConstraint(Constraint):
    def __init__(self, parts):
        self.parts = parts
        self.stateful = any(p.stateful for p in parts)

    def initial_state(self):
        return [p.initial_state() for p in self.parts]

    def apply(self, logits, state, vocab_offset=0, eos_ids=()):
        for p, s in zip(self.parts, state):
            p.apply(logits, s, vocab_offset, eos_ids)

    def advance(self, state, token_id):
        return [p.advance(s, token_id) for p, s in zip(self.parts, state)]

    def is_complete(self, state):
        return any(p.is_complete(s) for p, s in zip(self.parts, state) if p.stateful)


def make_constraint(sp, tokenizer):
    """Build the constraint of a request from its SamplingParams (None when unconstrained)."""
    parts = []
    if getattr(sp, "logit_bias", None):
        parts.append(LogitBiasConstraint(sp.logit_bias))
    if getattr(sp, "allowed_token_ids", None) or getattr(sp, "bad_token_ids", None):
        parts.append(TokenMaskConstraint(sp.allowed_token_ids, sp.bad_token_ids))
    grammars = [bool(getattr(sp, "guided_choice", None)), getattr(sp, "guided_json", None) not in (None, False),
                bool(getattr(sp, "guided_regex", None))]
    if sum(grammars) > 1:
        raise ValueError("use at most one of guided_choice, guided_json, guided_regex")
    if grammars[0]:
        parts.append(ChoiceConstraint(sp.guided_choice, tokenizer))
    elif grammars[1]:
        parts.append(JsonConstraint(sp.guided_json, tokenizer))
    elif grammars[2]:
        parts.append(RegexConstraint(sp.guided_regex, tokenizer))
    if not parts:
        return None
    return parts[0] if len(parts) == 1 else CompositeConstraint(parts)


def init_constraint_state(seq):
    if seq.constraint is not None and seq.constraint_state is None:
        seq.constraint_state = seq.constraint.initial_state()


def advance_constraint(seq, token_id: int):
    c = getattr(seq, "constraint", None)
    if c is not None and c.stateful:
        init_constraint_state(seq)
        seq.constraint_state = c.advance(seq.constraint_state, token_id)


def constraint_complete(seq) -> bool:
    c = getattr(seq, "constraint", None)
    if c is None or not c.stateful:
        return False
    init_constraint_state(seq)
    return c.is_complete(seq.constraint_state)
