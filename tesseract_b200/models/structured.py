"""Grammar-constrained decoding: a byte-level regex automaton and the token mask built on it.

``RegexAutomaton`` compiles a practical regex subset (literals, ``.``, escapes ``\\d \\D \\w \\W \\s \\S \\n \\t
\\r \\f \\v`` and escaped punctuation, classes ``[a-z0-9]`` / ``[^...]``, groups, alternation, ``* + ?`` and
counted ``{m} {m,} {m,n}``) into a Thompson NFA and walks it through lazy subset construction (a DFA state
is an epsilon-closed set of NFA states, memoised). Matching is anchored at both ends.

``GrammarConstraint`` maps that byte language onto a token vocabulary: a token is allowed iff its non-empty
byte string keeps the automaton live; EOS is allowed iff the current state is accepting; no allowed token
at all is an error; committing EOS does not move the state (include/tesseract/models/StructuredDecoding.hpp:47-138,
src/models/StructuredDecoding.cpp:400-468).
"""
from __future__ import annotations

from typing import Dict, FrozenSet, List, Optional, Sequence, Tuple

import numpy as np

K_DEAD = -1


class ByteAutomaton:
    def start(self) -> int:  # pragma: no cover - interface
        raise NotImplementedError

    def step(self, state: int, byte: int) -> int:  # pragma: no cover - interface
        raise NotImplementedError

    def accepting(self, state: int) -> bool:  # pragma: no cover - interface
        raise NotImplementedError

    def walk(self, state: int, data: bytes) -> int:
        for b in data:
            if state == K_DEAD:
                return K_DEAD
            state = self.step(state, b)
        return state


_ALL = frozenset(range(256))
_DIGIT = frozenset(range(48, 58))
_WORD = frozenset(list(range(48, 58)) + list(range(65, 91)) + list(range(97, 123)) + [95])
_SPACE = frozenset([32, 9, 10, 13, 11, 12])
_SIMPLE_ESC = {"n": 10, "t": 9, "r": 13, "f": 12, "v": 11}


class _Nfa:
    def __init__(self):
        self.eps: List[List[int]] = []
        self.trans: List[List[Tuple[FrozenSet[int], int]]] = []

    def new(self) -> int:
        self.eps.append([])
        self.trans.append([])
        return len(self.eps) - 1


class _Parser:
    """Recursive descent: alt := cat ('|' cat)*; cat := rep*; rep := atom quantifier*. Builds NFA fragments
    (start, end) directly."""

    def __init__(self, pattern: str, nfa: _Nfa):
        self.p, self.i, self.nfa = pattern, 0, nfa

    def _peek(self) -> Optional[str]:
        return self.p[self.i] if self.i < len(self.p) else None

    def parse(self) -> Tuple[int, int]:
        frag = self._alt()
        if self.i != len(self.p):
            raise ValueError(f"regex: unexpected {self.p[self.i]!r} at {self.i}")
        return frag

    def _alt(self):
        frags = [self._cat()]
        while self._peek() == "|":
            self.i += 1
            frags.append(self._cat())
        if len(frags) == 1:
            return frags[0]
        s, e = self.nfa.new(), self.nfa.new()
        for fs, fe in frags:
            self.nfa.eps[s].append(fs)
            self.nfa.eps[fe].append(e)
        return s, e

    def _cat(self):
        s = self.nfa.new()
        cur = s
        while self._peek() is not None and self._peek() not in "|)":
            fs, fe = self._rep()
            self.nfa.eps[cur].append(fs)
            cur = fe
        return s, cur

    def _rep(self):
        start_i = self.i
        frag = self._atom()
        atom_src = (start_i, self.i)
        while self._peek() is not None and self._peek() in "*+?{":
            c = self._peek()
            if c == "{":
                j = self.p.find("}", self.i)
                if j < 0:
                    raise ValueError("regex: unterminated {")
                body = self.p[self.i + 1:j]
                self.i = j + 1
                if "," in body:
                    lo_s, hi_s = body.split(",", 1)
                    lo = int(lo_s)
                    hi = int(hi_s) if hi_s.strip() else None
                else:
                    lo = hi = int(body)
                if hi is not None and hi < lo:
                    raise ValueError("regex: bad counted quantifier")
                frag = self._counted(atom_src, lo, hi)
                continue
            self.i += 1
            fs, fe = frag
            s, e = self.nfa.new(), self.nfa.new()
            self.nfa.eps[s].append(fs)
            self.nfa.eps[fe].append(e)
            if c in "*?":
                self.nfa.eps[s].append(e)
            if c in "*+":
                self.nfa.eps[fe].append(fs)
            frag = (s, e)
        return frag

    def _reparse_atom(self, src):
        sub = _Parser(self.p[src[0]:src[1]], self.nfa)
        return sub._atom()

    def _counted(self, src, lo, hi):
        s = self.nfa.new()
        cur = s
        for _ in range(lo):
            fs, fe = self._reparse_atom(src)
            self.nfa.eps[cur].append(fs)
            cur = fe
        if hi is None:
            fs, fe = self._reparse_atom(src)
            self.nfa.eps[cur].append(fs)
            self.nfa.eps[fe].append(fs)
            e = self.nfa.new()
            self.nfa.eps[cur].append(e)
            self.nfa.eps[fe].append(e)
            return s, e
        e = self.nfa.new()
        self.nfa.eps[cur].append(e)
        for _ in range(hi - lo):
            fs, fe = self._reparse_atom(src)
            self.nfa.eps[cur].append(fs)
            cur = fe
            self.nfa.eps[cur].append(e)
        return s, e

    def _escape_set(self, c: str) -> FrozenSet[int]:
        if c == "d":
            return _DIGIT
        if c == "D":
            return _ALL - _DIGIT
        if c == "w":
            return _WORD
        if c == "W":
            return _ALL - _WORD
        if c == "s":
            return _SPACE
        if c == "S":
            return _ALL - _SPACE
        if c in _SIMPLE_ESC:
            return frozenset([_SIMPLE_ESC[c]])
        return frozenset(c.encode("utf-8")) if len(c.encode("utf-8")) == 1 else frozenset()

    def _byte_edge(self, byteset: FrozenSet[int]):
        s, e = self.nfa.new(), self.nfa.new()
        self.nfa.trans[s].append((byteset, e))
        return s, e

    def _literal_bytes(self, data: bytes):
        s = self.nfa.new()
        cur = s
        for b in data:
            nxt = self.nfa.new()
            self.nfa.trans[cur].append((frozenset([b]), nxt))
            cur = nxt
        return s, cur

    def _atom(self):
        c = self._peek()
        if c is None:
            raise ValueError("regex: unexpected end of pattern")
        if c == "(":
            self.i += 1
            frag = self._alt()
            if self._peek() != ")":
                raise ValueError("regex: missing )")
            self.i += 1
            return frag
        if c == "[":
            return self._byte_edge(self._klass())
        if c == ".":
            self.i += 1
            return self._byte_edge(_ALL)
        if c == "\\":
            if self.i + 1 >= len(self.p):
                raise ValueError("regex: dangling backslash")
            e = self.p[self.i + 1]
            self.i += 2
            return self._byte_edge(self._escape_set(e))
        if c in "*+?{":
            raise ValueError(f"regex: nothing to repeat at {self.i}")
        self.i += 1
        return self._literal_bytes(c.encode("utf-8"))

    def _klass(self) -> FrozenSet[int]:
        self.i += 1  # [
        neg = self._peek() == "^"
        if neg:
            self.i += 1
        items = set()
        first = True
        while True:
            c = self._peek()
            if c is None:
                raise ValueError("regex: unterminated [")
            if c == "]" and not first:
                self.i += 1
                break
            first = False
            if c == "\\":
                e = self.p[self.i + 1]
                self.i += 2
                es = self._escape_set(e)
                if len(es) != 1:
                    items |= es
                    continue
                lo = next(iter(es))
            else:
                self.i += 1
                enc = c.encode("utf-8")
                if len(enc) != 1:
                    items |= set(enc)
                    continue
                lo = enc[0]
            if self._peek() == "-" and self.i + 1 < len(self.p) and self.p[self.i + 1] != "]":
                self.i += 1
                hc = self._peek()
                if hc == "\\":
                    hs = self._escape_set(self.p[self.i + 1])
                    self.i += 2
                    hi = next(iter(hs))
                else:
                    self.i += 1
                    hi = hc.encode("utf-8")[0]
                if hi < lo:
                    raise ValueError("regex: reversed range in class")
                items |= set(range(lo, hi + 1))
            else:
                items.add(lo)
        return frozenset(_ALL - items) if neg else frozenset(items)


MAX_DFA_STATES = 65536


def _host_module():
    from .sampler import _host_module as hm
    return hm()


class RegexAutomaton(ByteAutomaton):
    """Anchored byte-level regex. With the native host runtime the pattern is compiled in C++ (csrc/host/regex.cpp)
    into a complete DFA table -- states numbered breadth first, state 0 the start state -- and ``step`` is a table
    lookup; the token mask of a vocabulary is then one native walk over all token bytes (``GrammarConstraint``).
    Without it (or when the DFA would exceed ``MAX_DFA_STATES``) the Python implementation below runs lazily:
    a DFA state is an epsilon-closed set of NFA states, interned on first sight. ``dfa_table()`` of the Python
    implementation builds the same table as the native compiler, entry for entry."""

    def __init__(self, pattern: str, native: Optional[bool] = None):
        self.pattern = pattern
        self._table: Optional[np.ndarray] = None        # int32 [states, 256], -1 = dead (native mode)
        self._accepting: Optional[np.ndarray] = None
        host = _host_module() if native in (None, True) else None
        if native is True and host is None:
            raise RuntimeError("RegexAutomaton: the native host runtime is not available")
        if host is not None and hasattr(host, "compile_regex"):
            try:
                self._table, self._accepting, _ = host.compile_regex(pattern.encode("utf-8"), MAX_DFA_STATES)
                return
            except ValueError as e:
                if "max_states" not in str(e):
                    raise                                  # a malformed pattern: the same error class as the twin
        self._nfa = _Nfa()
        self._start_nfa, self._accept_nfa = _Parser(pattern, self._nfa).parse()
        self._ids: Dict[FrozenSet[int], int] = {}
        self._sets: List[FrozenSet[int]] = []
        self._memo: Dict[Tuple[int, int], int] = {}
        self._start = self._intern(self._closure({self._start_nfa}))

    @property
    def is_native(self) -> bool:
        return self._table is not None

    def dfa_table(self, max_states: int = MAX_DFA_STATES) -> Tuple[np.ndarray, np.ndarray]:
        """The complete DFA as ``(table int32 [states, 256], accepting uint8 [states])``: state 0 is the start state,
        states are numbered in breadth-first discovery order with the bytes visited 0 .. 255."""
        if self._table is not None:
            return self._table, self._accepting
        fresh = RegexAutomaton(self.pattern, native=False)       # its lazy numbering starts from scratch
        rows: List[List[int]] = []
        q = 0
        while q < len(fresh._sets):
            if len(fresh._sets) > max_states:
                raise ValueError("regex: more DFA states than max_states")
            rows.append([fresh.step(q, b) for b in range(256)])
            q += 1
        table = np.asarray(rows, dtype=np.int32).reshape(len(rows), 256)
        acc = np.asarray([1 if fresh.accepting(s) else 0 for s in range(len(rows))], dtype=np.uint8)
        return table, acc

    def _closure(self, states) -> FrozenSet[int]:
        seen, stack = set(states), list(states)
        while stack:
            s = stack.pop()
            for t in self._nfa.eps[s]:
                if t not in seen:
                    seen.add(t)
                    stack.append(t)
        return frozenset(seen)

    def _intern(self, st: FrozenSet[int]) -> int:
        i = self._ids.get(st)
        if i is None:
            i = len(self._sets)
            self._ids[st] = i
            self._sets.append(st)
        return i

    def start(self) -> int:
        return 0 if self._table is not None else self._start

    def step(self, state: int, byte: int) -> int:
        if state == K_DEAD:
            return K_DEAD
        if self._table is not None:
            return int(self._table[state, byte])
        key = (state, byte)
        hit = self._memo.get(key)
        if hit is not None:
            return hit
        nxt = set()
        for s in self._sets[state]:
            for bs, t in self._nfa.trans[s]:
                if byte in bs:
                    nxt.add(t)
        res = self._intern(self._closure(nxt)) if nxt else K_DEAD
        self._memo[key] = res
        return res

    def accepting(self, state: int) -> bool:
        if state == K_DEAD:
            return False
        if self._table is not None:
            return bool(self._accepting[state])
        return self._accept_nfa in self._sets[state]

    def matches(self, s) -> bool:
        data = s.encode("utf-8") if isinstance(s, str) else bytes(s)
        return self.accepting(self.walk(self.start(), data))

    def num_dfa_states(self) -> int:
        """States of the complete DFA (native mode) or the states visited so far (lazy mode)."""
        return int(self._table.shape[0]) if self._table is not None else len(self._sets)


class GrammarConstraint:
    def __init__(self, automaton: ByteAutomaton, token_bytes: Sequence[bytes], eos_id: int = -1):
        self.automaton = automaton
        self.token_bytes = [bytes(b) for b in token_bytes]
        self.eos_id = eos_id
        self.state = automaton.start()
        self._mask_cache: Dict[int, np.ndarray] = {}
        # native mask: all token bytes in one buffer with offsets, walked over the DFA table in C++
        self._packed: Optional[Tuple[bytes, np.ndarray]] = None
        if getattr(automaton, "is_native", False) and _host_module() is not None:
            offs = np.zeros(len(self.token_bytes) + 1, dtype=np.int64)
            np.cumsum([len(b) for b in self.token_bytes], out=offs[1:])
            self._packed = (b"".join(self.token_bytes), offs)

    @classmethod
    def from_tokenizer(cls, automaton: ByteAutomaton, tokenizer, eos_id: Optional[int] = None) -> "GrammarConstraint":
        n = tokenizer.vocab_size()
        toks = [tokenizer.decode([i], skip_special_tokens=True).encode("utf-8") for i in range(n)]
        return cls(automaton, toks, tokenizer.eos_id if eos_id is None else eos_id)

    def reset(self) -> None:
        self.state = self.automaton.start()

    def allowed_mask(self) -> np.ndarray:
        m = self._mask_cache.get(self.state)
        if m is None and self._packed is not None:
            table, _ = self.automaton.dfa_table()
            m = _host_module().token_mask(table, int(self.state), self._packed[0], self._packed[1]).astype(bool)
            if 0 <= self.eos_id < m.shape[0]:
                m[self.eos_id] = self.automaton.accepting(self.state)
            self._mask_cache[self.state] = m
        if m is None:
            m = np.zeros(len(self.token_bytes), dtype=bool)
            for i, tb in enumerate(self.token_bytes):
                if i == self.eos_id:
                    m[i] = self.automaton.accepting(self.state)
                elif tb:
                    m[i] = self.automaton.walk(self.state, tb) != K_DEAD
            self._mask_cache[self.state] = m
        return m

    def apply(self, logits: np.ndarray) -> int:
        """Mask ``logits`` (fp32, length = vocabulary) in place; returns the number of allowed tokens."""
        m = self.allowed_mask()
        if logits.shape[0] != m.shape[0]:
            raise ValueError("GrammarConstraint.apply: logits length differs from the vocabulary")
        n = int(m.sum())
        if n == 0:
            raise RuntimeError("GrammarConstraint: no token is allowed in the current state")
        logits[~m] = -np.inf
        return n

    def accept(self, token_id: int) -> None:
        if token_id == self.eos_id:
            return
        self.state = self.automaton.walk(self.state, self.token_bytes[token_id])
        if self.state == K_DEAD:
            raise RuntimeError("GrammarConstraint.accept: token leaves the grammar")


def generate_structured(model, prompt_ids, tokenizer, regex: str, cfg=None, token_bytes: Optional[Sequence[bytes]] = None):
    """``LlamaModel.generate`` with every step's logits masked by the regular expression ``regex``
    (the reference wires the same constraint into its generate CLI, examples/llama_generate.cpp:133,
    through ``GrammarConstraint::apply`` / ``accept``). EOS is allowed only in accepting states; generation stops at
    EOS, at ``max_new_tokens``, or when the grammar allows no further token. Returns prompt + generated ids."""
    import torch

    from .llama import GenerateConfig
    from .sampler import Sampler
    cfg = cfg or GenerateConfig()
    V = model.config.vocab_size
    if token_bytes is None:
        token_bytes = [tokenizer.decode([i]).encode("utf-8") if i < 256 or hasattr(tokenizer, "vocab_size") else b""
                       for i in range(V)]
    if len(token_bytes) != V:
        token_bytes = (list(token_bytes) + [b""] * V)[:V]
    constraint = GrammarConstraint(RegexAutomaton(regex), token_bytes, cfg.eos_token_id)
    prompt = [int(t) for t in prompt_ids]
    total = len(prompt) + cfg.max_new_tokens
    caches = model.make_quantized_kv_caches(1, total) if cfg.kv_int8 else model.make_kv_caches(1, total)
    sampler = Sampler(cfg.sampling, cfg.seed) if cfg.do_sample else None
    out = list(prompt)
    dev = next(model.parameters()).device
    logits = model.forward_step(torch.tensor([prompt], dtype=torch.int64, device=dev), caches)
    for step in range(cfg.max_new_tokens):
        row = logits[0, -1].float().cpu().numpy().copy()
        try:
            constraint.apply(row)
        except RuntimeError:
            break                                   # the grammar is exhausted
        nxt = int(row.argmax()) if sampler is None else sampler.sample(row, out)
        out.append(nxt)
        if cfg.eos_token_id >= 0 and nxt == cfg.eos_token_id:
            break
        constraint.accept(nxt)
        if step + 1 < cfg.max_new_tokens:
            logits = model.forward_step(torch.tensor([[nxt]], dtype=torch.int64, device=dev), caches)
    return out
