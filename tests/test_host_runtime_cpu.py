"""The native host runtime (csrc/host, pybind11 module _tsb_host) against its pure-Python twins: identical random
streams and sampled tokens, identical BPE ids, identical allocator behaviour, parallel file reads."""
import numpy as np
import pytest
import torch

from tesseract_b200 import _native

host = _native.host()
pytestmark = pytest.mark.skipif(host is None, reason="native host runtime not built")


def test_mt19937_64_stream_and_uniform_match_python():
    from tesseract_b200.models.sampler import MT19937_64
    for seed in (0, 1, 5489, 2 ** 63 + 12345):
        py, nat = MT19937_64(seed), host.HostSampler(seed=seed)
        assert [py.next_u64() for _ in range(700)] == [nat.next_u64() for _ in range(700)]   # crosses a twist
        assert [py.uniform_double() for _ in range(50)] == [nat.uniform_double() for _ in range(50)]
    assert host.HostSampler(seed=5489).next_u64() == 14514284786278117030        # std::mt19937_64 default seed, 1st draw


@pytest.mark.parametrize("params", [dict(temperature=0.8), dict(temperature=1.3, top_k=7),
                                    dict(temperature=0.7, top_p=0.9), dict(temperature=1.0, top_k=20, top_p=0.5,
                                                                           repetition_penalty=1.3),
                                    dict(temperature=0.0, repetition_penalty=2.0)])
def test_sampler_tokens_match_python(params):
    from tesseract_b200.models.sampler import Sampler, SamplingParams
    rng = np.random.default_rng(3)
    sp = SamplingParams(**params)
    a, b = Sampler(sp, seed=11, native=False), Sampler(sp, seed=11, native=True)
    hist = []
    for _ in range(60):
        logits = rng.standard_normal(997).astype(np.float32) * 3
        logits[rng.integers(0, 997, 5)] = logits.max()            # ties
        ta, tb = a.sample(logits, hist), b.sample(logits, hist)
        assert ta == tb
        hist.append(ta)
    a.reseed(5)
    b.reseed(5)
    assert a.sample(logits, hist) == b.sample(logits, hist)


def test_bpe_core_matches_python(monkeypatch):
    from tesseract_b200.io.tokenizer import _B2U, BpeTokenizer
    alphabet = [_B2U[b] for b in range(256)]
    vocab = {ch: i for i, ch in enumerate(alphabet)}
    merges = []
    def add(a, b):
        merges.append((a, b))
        vocab.setdefault(a + b, len(vocab))
    sp = _B2U[ord(" ")]
    add("t", "h"); add("th", "e"); add(sp, "the"); add("i", "n"); add("a", "n"); add(sp, "a"); add("e", "r"); add("in", "g")
    merges.append(("x", "y"))                                       # merged symbol missing from the vocabulary
    text = "the other thing in an xy anthem " * 3 + "naïve café 你好"
    monkeypatch.setenv("TESSERACT_HOST", "python")
    py_ids = BpeTokenizer(vocab, merges, {"<s>": 900}).encode("<s>" + text)
    monkeypatch.delenv("TESSERACT_HOST")
    tok = BpeTokenizer(vocab, merges, {"<s>": 900})
    nat_ids = tok.encode("<s>" + text)
    assert tok._core is not None and nat_ids == py_ids
    assert tok.decode(nat_ids) == text


def test_block_allocator_native_behaviour():
    from tesseract_b200.nn.kv_cache import BlockAllocator
    al = BlockAllocator(4)
    assert type(al).__module__ == "_tsb_host"
    assert [al.allocate() for _ in range(4)] == [0, 1, 2, 3] and al.num_free() == 0 and al.num_used() == 4
    with pytest.raises(RuntimeError):
        al.allocate()
    al.free(2)
    assert al.allocate() == 2
    al.free(1)
    with pytest.raises(RuntimeError):
        al.free(1)
    with pytest.raises(RuntimeError):
        al.free(17)
    with pytest.raises(ValueError):
        BlockAllocator(0)


def test_parallel_safetensors_load_matches_mmap_reader(tmp_path):
    from tesseract_b200.io import load_file, load_file_parallel, save_file
    g = torch.Generator().manual_seed(0)
    tensors = {"a": torch.randn(1000, 300, generator=g), "b": torch.randint(0, 100, (77,), generator=g),
               "c.bf16": torch.randn(5000, 64, generator=g).bfloat16(), "empty": torch.zeros(0, 3)}
    path = str(tmp_path / "m.safetensors")
    save_file(tensors, path, metadata={"format": "pt"})
    ref, got = load_file(path), load_file_parallel(path, threads=4, pin=False)
    assert list(ref) == list(got)
    for k in ref:
        assert ref[k].dtype == got[k].dtype and torch.equal(ref[k], got[k])
    hdr, off = host.safetensors_header(path)
    assert off % 8 == 0 and b'"__metadata__"' in hdr
    with pytest.raises(RuntimeError):
        host.read_ranges(path, [0], [10 ** 9], [0], 2) if False else host.safetensors_header(str(tmp_path / "missing"))


def test_token_mask_kernel():
    # automaton over bytes for [0-9]+ : state 0 --digit--> 1 --digit--> 1
    table = np.full((2, 256), -1, dtype=np.int32)
    table[:, ord("0"):ord("9") + 1] = 1
    toks = [b"12", b"a", b"", b"7", b"3x"]
    offs = np.cumsum([0] + [len(t) for t in toks]).astype(np.int64)
    mask = host.token_mask(table, 0, b"".join(toks), offs)
    assert mask.tolist() == [1, 0, 0, 1, 0]


REGEXES = [r"-?(0|[1-9]\d*)(\.\d+)?", r"(yes|no|maybe)", r"[a-c]{2,3}x?", r"[^0-9]+\s\w{2}", r"a{2,}", r"a{0,2}b{3}",
           r"\{\"name\": \"[a-z]+\", \"age\": [1-9]\d?\}", r"[]a-]+", r"(ab|a)(bc|c)*", r"\D\W\S.", r"héllo[é-ü]?",
           r"(\+|-)?\d{1,3}(,\d{3})*", r"[\d\s]+|x", r"((a|b)*c){2}", r""]


@pytest.mark.parametrize("pattern", REGEXES)
def test_regex_compiler_builds_the_same_dfa_as_the_python_twin(pattern):
    """csrc/host/regex.cpp against models/structured.py: the complete DFA tables are equal entry for entry (same
    breadth-first numbering), so are the accepting flags."""
    from tesseract_b200.models.structured import RegexAutomaton
    nat, twin = RegexAutomaton(pattern, native=True), RegexAutomaton(pattern, native=False)
    assert nat.is_native and not twin.is_native
    t_nat, a_nat = nat.dfa_table()
    t_py, a_py = twin.dfa_table()
    assert t_nat.shape == t_py.shape and np.array_equal(t_nat, t_py) and np.array_equal(a_nat, a_py)
    assert nat.num_dfa_states() == t_py.shape[0]


def test_regex_compiler_errors_and_matching_agree_with_the_twin():
    from tesseract_b200.models.structured import K_DEAD, RegexAutomaton
    for bad in ["(ab", "a)", "*a", "a{2", "a{3,1}", "[abc", "a\\", "[z-a]"]:
        with pytest.raises(ValueError):
            RegexAutomaton(bad, native=True)
        with pytest.raises((ValueError, IndexError)):
            RegexAutomaton(bad, native=False)
    rng = np.random.default_rng(7)
    alphabet = list(b"ab01 .-,x_c\xc3\xa9")
    for pattern in REGEXES:
        nat, twin = RegexAutomaton(pattern, native=True), RegexAutomaton(pattern, native=False)
        for _ in range(200):
            s = bytes(rng.choice(alphabet, size=int(rng.integers(0, 9))).tolist())
            assert nat.matches(s) == twin.matches(s), (pattern, s)
            live_n = nat.walk(nat.start(), s) != K_DEAD
            live_t = twin.walk(twin.start(), s) != K_DEAD
            assert live_n == live_t, (pattern, s)


def test_grammar_mask_native_walk_equals_python_loop(monkeypatch):
    """The vocabulary mask from one native walk over all token bytes equals the per-token Python loop, state by state
    along a constrained generation."""
    from tesseract_b200.models.structured import GrammarConstraint, RegexAutomaton
    rng = np.random.default_rng(1)
    pieces = [b"", b"0", b"1", b"12", b"7.", b".", b".5", b"-", b"-3", b"a", b"1a", b"00", b"<eos>"]
    vocab = pieces + [bytes(rng.choice(list(b"0123456789.-a"), size=int(rng.integers(1, 5))).tolist()) for _ in range(300)]
    eos = 12
    pattern = r"-?(0|[1-9]\d*)(\.\d+)?"
    g_nat = GrammarConstraint(RegexAutomaton(pattern, native=True), vocab, eos_id=eos)
    g_py = GrammarConstraint(RegexAutomaton(pattern, native=False), vocab, eos_id=eos)
    assert g_nat._packed is not None and g_py._packed is None
    for step in range(12):
        m_nat, m_py = g_nat.allowed_mask(), g_py.allowed_mask()
        assert np.array_equal(m_nat, m_py), step
        allowed = np.nonzero(m_py)[0]
        allowed = allowed[allowed != eos]
        if allowed.size == 0:
            break
        tok = int(allowed[int(rng.integers(0, allowed.size))])
        g_nat.accept(tok)
        g_py.accept(tok)


def _random_pattern(rng, depth=0):
    """A random pattern of the supported subset over the letters a .. c (valid for Python's ``re`` too)."""
    def atom():
        r = rng.integers(0, 10)
        if r < 4:
            return "abc"[int(rng.integers(0, 3))]
        if r == 4:
            return "."
        if r == 5:
            return ["[ab]", "[^a]", "[a-c]", "[b-c]", r"\w", r"\d"][int(rng.integers(0, 6))]
        if depth < 2:
            return "(" + _random_pattern(rng, depth + 1) + ")"
        return "abc"[int(rng.integers(0, 3))]

    def piece():
        a = atom()
        q = rng.integers(0, 8)
        if q == 0:
            return a + "*"
        if q == 1:
            return a + "+"
        if q == 2:
            return a + "?"
        if q == 3:
            lo = int(rng.integers(0, 3))
            return a + "{%d,%d}" % (lo, lo + int(rng.integers(0, 3)))
        if q == 4:
            return a + "{%d}" % int(rng.integers(1, 3))
        return a

    def cat():
        return "".join(piece() for _ in range(int(rng.integers(1, 4))))

    return "|".join(cat() for _ in range(int(rng.integers(1, 3))))


def test_regex_automata_agree_with_python_re_on_random_patterns():
    """An independent oracle: anchored matching of both automata equals ``re.fullmatch`` for random patterns of the
    supported subset and random strings."""
    import re
    from tesseract_b200.models.structured import RegexAutomaton
    rng = np.random.default_rng(11)
    checked = 0
    for _ in range(150):
        pattern = _random_pattern(rng)
        oracle = re.compile(pattern, re.DOTALL | re.ASCII)
        nat, twin = RegexAutomaton(pattern, native=True), RegexAutomaton(pattern, native=False)
        for _ in range(40):
            s = "".join("abc1_ "[int(i)] for i in rng.integers(0, 6, size=int(rng.integers(0, 7))))
            want = oracle.fullmatch(s) is not None
            assert nat.matches(s) == want, (pattern, s, want)
            assert twin.matches(s) == want, (pattern, s, want)
            checked += 1
    assert checked == 6000


def test_sampler_twins_agree_on_flat_tied_and_peaked_rows():
    """Nucleus sampling where the cut is decided by rounding (uniform rows, top_p next to 1), with many ties, and on a
    128 K vocabulary where only a prefix of the order is sorted: native and Python samplers draw the same tokens."""
    from tesseract_b200.models.sampler import Sampler, SamplingParams
    rng = np.random.default_rng(0)
    rows = [(rng.standard_normal(128256) * 3.0), (rng.standard_normal(128256) * 0.05), np.zeros(1000),
            np.round(rng.standard_normal(300) * 2) / 4, rng.standard_normal(777) * 2.0]
    settings = [dict(temperature=1.0, top_p=0.9), dict(temperature=0.7, top_k=40, top_p=0.5),
                dict(temperature=1.3, top_p=0.999), dict(temperature=1.0, top_p=0.01),
                dict(temperature=0.37, top_p=0.95, repetition_penalty=1.1)]
    for row in rows:
        logits = torch.from_numpy(row.astype(np.float32))
        for kw in settings:
            a, b = Sampler(SamplingParams(**kw), seed=7, native=True), Sampler(SamplingParams(**kw), seed=7, native=False)
            for _ in range(4):
                assert a.sample(logits, [1, 2, 3]) == b.sample(logits, [1, 2, 3]), (row.shape, kw)
