"""Byte-level BPE against golden token ids produced by Hugging Face ``tokenizers``.

``tests/fixtures/hf_bpe/tokenizer.json`` is a small trained byte-level BPE model (400 entries, three special
tokens) and ``golden_ids.tsv`` holds, per line, the ids that the Hugging Face implementation produced for a text
(ids, a tab, the text as a JSON string literal). They are the data files of the reference project's tokenizer
parity test (tests/io/test_bpe_tokenizer.cpp:132-141, fixtures under tests/io/fixtures); both the Python
tokenizer and the native merge loop have to reproduce every line.
"""
import json
import os

import pytest

from tesseract_b200.io.tokenizer import BpeTokenizer

FIX = os.path.join(os.path.dirname(__file__), "fixtures", "hf_bpe")


def _golden():
    rows = []
    with open(os.path.join(FIX, "golden_ids.tsv"), encoding="utf-8") as f:
        for line in f:
            line = line.rstrip("\n")
            if not line.strip():
                continue
            ids, text = line.split("\t", 1)
            rows.append(([int(t) for t in ids.split()], json.loads(text)))
    return rows


@pytest.mark.parametrize("host", ["native", "python"])
def test_golden_ids_match_hugging_face(host, monkeypatch):
    monkeypatch.setenv("TESSERACT_HOST", host)
    tok = BpeTokenizer.from_file(os.path.join(FIX, "tokenizer.json"))
    rows = _golden()
    assert len(rows) >= 7
    for ids, text in rows:
        assert tok.encode(text, add_special_tokens=False) == ids, text


def test_vocab_specials_and_round_trip():
    tok = BpeTokenizer.from_file(os.path.join(FIX, "tokenizer.json"))
    assert tok.vocab_size() == 400
    assert tok.bos_token_id() >= 0 and tok.eos_token_id() >= 0 and tok.bos_token_id() != tok.eos_token_id()
    for text in ["the quick brown fox", "punctuation, like; colons: periods.", "numbers 12 34 567 here",
                 "  leading spaces", "CamelCase and snake_case"]:
        assert tok.decode(tok.encode(text, add_special_tokens=False), skip_special_tokens=True) == text
    plain = tok.encode("the quick brown fox", add_special_tokens=False)
    special = tok.encode("the quick brown fox", add_special_tokens=True)
    assert special == [tok.bos_token_id()] + plain + [tok.eos_token_id()]
