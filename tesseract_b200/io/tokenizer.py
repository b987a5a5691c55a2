"""Tokenizers: a whitespace tokenizer over a fixed vocabulary and a byte-level BPE tokenizer that reads
Hugging Face ``tokenizer.json`` files.

BPE behaviour follows the reference (src/io/BpeTokenizer.cpp): GPT-2 byte <-> unicode table; an
ASCII-scoped GPT-2 pre-tokeniser (contractions 's 't 'm 'd 're 've 'll; an optional leading space followed
by a run of letters, of digits, or of other characters; whitespace runs that leave their last space to the
next piece; bytes >= 0x80 count as letters); merging = repeatedly take the lowest-rank adjacent pair and
merge ALL its occurrences; added tokens are matched longest-first as whole units; BOS / EOS are resolved
from the added tokens (<|begin_of_text|> or <s>; <|end_of_text|>, </s> or <|eot_id|>); merges may be
"a b" strings or ["a", "b"] pairs; ``decode`` can skip added ids.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


class Tokenizer:
    """Common interface (include/tesseract/io/Tokenizer.hpp)."""

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:  # pragma: no cover - interface
        raise NotImplementedError

    def decode(self, ids, skip_special_tokens: bool = True) -> str:  # pragma: no cover - interface
        raise NotImplementedError

    def vocab_size(self) -> int:  # pragma: no cover - interface
        raise NotImplementedError

    bos_id: int = -1
    eos_id: int = -1
    unk_id: int = -1

    # accessor spelling of the reference's Python module (python/_core.cpp:334-336)
    def bos_token_id(self) -> int:
        return self.bos_id

    def eos_token_id(self) -> int:
        return self.eos_id

    def unk_token_id(self) -> int:
        return self.unk_id


@dataclass
class WhitespaceTokenizerConfig:
    vocab: List[str] = field(default_factory=list)
    unk: str = "<unk>"
    bos: str = ""
    eos: str = ""


class WhitespaceTokenizer(Tokenizer):
    def __init__(self, cfg: WhitespaceTokenizerConfig):
        self.cfg = cfg
        self._id = {w: i for i, w in enumerate(cfg.vocab)}
        if cfg.unk not in self._id:
            raise ValueError("WhitespaceTokenizer: the unk token must be in the vocabulary")
        self.unk_id = self._id[cfg.unk]
        self.bos_id = self._id.get(cfg.bos, -1) if cfg.bos else -1
        self.eos_id = self._id.get(cfg.eos, -1) if cfg.eos else -1

    def encode(self, text, add_special_tokens=True):
        ids = [self._id.get(w, self.unk_id) for w in text.split()]
        if add_special_tokens:
            if self.bos_id >= 0:
                ids = [self.bos_id] + ids
            if self.eos_id >= 0:
                ids = ids + [self.eos_id]
        return ids

    def decode(self, ids, skip_special_tokens=True):
        special = {self.bos_id, self.eos_id} - {-1}
        words = [self.cfg.vocab[i] for i in ids if not (skip_special_tokens and i in special)]
        return " ".join(words)

    def vocab_size(self):
        return len(self.cfg.vocab)


def _bytes_to_unicode() -> Dict[int, str]:
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAC + 1)) + list(range(0xAE, 0xFF + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return {b: chr(c) for b, c in zip(bs, cs)}


_B2U = _bytes_to_unicode()
_U2B = {u: b for b, u in _B2U.items()}
_CONTRACTIONS = ("'s", "'t", "'m", "'d", "'re", "'ve", "'ll")


def _is_letter(b: int) -> bool:
    return (65 <= b <= 90) or (97 <= b <= 122) or b >= 0x80


def _is_digit(b: int) -> bool:
    return 48 <= b <= 57


def _is_space(b: int) -> bool:
    return b in (32, 9, 10, 13, 11, 12)


def pretokenize(data: bytes) -> List[bytes]:
    """GPT-2 pattern ``'s|'t|'re|'ve|'m|'ll|'d| ?L+| ?N+| ?[^\\sLN]+|\\s+(?!\\S)|\\s+`` on bytes."""
    out, i, n = [], 0, len(data)
    while i < n:
        matched = False
        if data[i] == 39:  # apostrophe
            for c in _CONTRACTIONS:
                cb = c.encode()
                if data.startswith(cb, i):
                    out.append(cb)
                    i += len(cb)
                    matched = True
                    break
        if matched:
            continue
        j = i
        if data[j] == 32 and j + 1 < n and not _is_space(data[j + 1]):
            j += 1
        if j < n and not _is_space(data[j]):
            k = j
            if _is_letter(data[k]):
                while k < n and _is_letter(data[k]):
                    k += 1
            elif _is_digit(data[k]):
                while k < n and _is_digit(data[k]):
                    k += 1
            else:
                while k < n and not _is_space(data[k]) and not _is_letter(data[k]) and not _is_digit(data[k]):
                    k += 1
            out.append(data[i:k])
            i = k
            continue
        k = i
        while k < n and _is_space(data[k]):
            k += 1
        if k < n and k - i > 1:
            k -= 1  # leave the last space to prefix the next piece
        out.append(data[i:k])
        i = k
    return out


class BpeTokenizer(Tokenizer):
    def __init__(self, vocab: Dict[str, int], merges: List[Tuple[str, str]], added: Dict[str, int]):
        self.vocab = dict(vocab)
        self.ranks = {pair: r for r, pair in enumerate(merges)}
        self.added = dict(added)
        self._added_sorted = sorted(self.added.keys(), key=len, reverse=True)
        self.id_to_tok: Dict[int, str] = {i: t for t, i in self.vocab.items()}
        for t, i in self.added.items():
            self.id_to_tok[i] = t
        self._added_ids = set(self.added.values())
        self.bos_id = next((self.added[t] for t in ("<|begin_of_text|>", "<s>") if t in self.added), -1)
        self.eos_id = next((self.added[t] for t in ("<|end_of_text|>", "</s>", "<|eot_id|>") if t in self.added), -1)
        self.unk_id = next((self.added[t] for t in ("<unk>", "<|unk|>") if t in self.added), -1)
        self._cache: Dict[bytes, List[int]] = {}
        self._core = None           # native merge loop (csrc/host/bpe_io.cpp), built on first use
        self._core_tried = False

    def _native_core(self):
        if not self._core_tried:
            self._core_tried = True
            import os
            if os.environ.get("TESSERACT_HOST", "") != "python":
                from .. import _native
                host = _native.host()
                if host is not None:
                    merges = sorted(self.ranks.items(), key=lambda kv: kv[1])
                    self._core = host.BpeCore(self.vocab, [pair for pair, _ in merges], [_B2U[b] for b in range(256)])
        return self._core

    @classmethod
    def from_json(cls, text: str) -> "BpeTokenizer":
        obj = json.loads(text)
        model = obj.get("model", {})
        if model.get("type", "BPE") != "BPE":
            raise ValueError("BpeTokenizer: tokenizer.json model type must be BPE")
        merges = []
        for m in model.get("merges", []):
            if isinstance(m, str):
                a, b = m.split(" ", 1)
            else:
                a, b = m
            merges.append((a, b))
        added = {t["content"]: int(t["id"]) for t in obj.get("added_tokens", [])}
        return cls(model.get("vocab", {}), merges, added)

    @classmethod
    def from_file(cls, path: str) -> "BpeTokenizer":
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_json(f.read())

    def vocab_size(self) -> int:
        return max(self.id_to_tok.keys(), default=-1) + 1

    def _bpe(self, piece: bytes) -> List[int]:
        hit = self._cache.get(piece)
        if hit is not None:
            return hit
        core = self._native_core()
        if core is not None:
            ids = list(core.encode_piece(bytes(piece)))
            if len(self._cache) < 65536:
                self._cache[piece] = ids
            return ids
        syms = [_B2U[b] for b in piece]
        while len(syms) > 1:
            best, best_rank = None, None
            for a, b in zip(syms[:-1], syms[1:]):
                r = self.ranks.get((a, b))
                if r is not None and (best_rank is None or r < best_rank):
                    best, best_rank = (a, b), r
            if best is None:
                break
            merged, i = [], 0
            while i < len(syms):
                if i + 1 < len(syms) and syms[i] == best[0] and syms[i + 1] == best[1]:
                    merged.append(best[0] + best[1])
                    i += 2
                else:
                    merged.append(syms[i])
                    i += 1
            syms = merged
        ids = []
        for s in syms:
            if s in self.vocab:
                ids.append(self.vocab[s])
            else:  # unknown multi-byte symbol: fall back to its bytes
                ids.extend(self.vocab[ch] for ch in s if ch in self.vocab)
        if len(self._cache) < 65536:
            self._cache[piece] = ids
        return ids

    def _encode_plain(self, text: str) -> List[int]:
        ids: List[int] = []
        for piece in pretokenize(text.encode("utf-8")):
            ids.extend(self._bpe(piece))
        return ids

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        ids: List[int] = []
        if add_special_tokens and self.bos_id >= 0:
            ids.append(self.bos_id)
        i, start, n = 0, 0, len(text)
        while i < n:
            hit = None
            if self._added_sorted:
                for t in self._added_sorted:
                    if text.startswith(t, i):
                        hit = t
                        break
            if hit is None:
                i += 1
                continue
            if start < i:
                ids.extend(self._encode_plain(text[start:i]))
            ids.append(self.added[hit])
            i += len(hit)
            start = i
        if start < n:
            ids.extend(self._encode_plain(text[start:]))
        if add_special_tokens and self.eos_id >= 0:      # BOS ... EOS, as src/io/BpeTokenizer.cpp:472,513
            ids.append(self.eos_id)
        return ids

    def decode(self, ids, skip_special_tokens: bool = True) -> str:
        buf = bytearray()
        for i in ids:
            i = int(i)
            if i in self._added_ids:
                if not skip_special_tokens:
                    buf.extend(self.id_to_tok[i].encode("utf-8"))
                continue
            tok = self.id_to_tok.get(i)
            if tok is None:
                continue
            for ch in tok:
                b = _U2B.get(ch)
                if b is not None:
                    buf.append(b)
                else:
                    buf.extend(ch.encode("utf-8"))
        return buf.decode("utf-8", errors="replace")
