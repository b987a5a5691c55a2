"""safetensors, tokenizers, quantisation packers / layers, structured decoding, MoE, Mamba and the tesseract API."""
import json
import struct

import numpy as np
import pytest
import torch

from tesseract_b200.io import (BpeTokenizer, SafeTensors, SafeTensorsError, WhitespaceTokenizer,
                               WhitespaceTokenizerConfig, load_file, save_file)
from tesseract_b200.models import GenerateConfig, LlamaConfig, LlamaModel
from tesseract_b200.models.structured import K_DEAD, GrammarConstraint, RegexAutomaton
from tesseract_b200.nn.moe import MoEFeedForward
from tesseract_b200.quant import (QuantizedLinear, QuantizedLinearInt4G, Scheme, pack_int4_group, pack_int8_symmetric,
                                  unpack_int4_group)


def test_safetensors_roundtrip_and_validation(tmp_path):
    p = str(tmp_path / "a.safetensors")
    tensors = {"b.weight": torch.randn(3, 4), "a.ids": torch.arange(6, dtype=torch.int64).view(2, 3),
               "c.half": torch.randn(5).to(torch.bfloat16), "d.flag": torch.tensor([True, False])}
    save_file(tensors, p, {"format": "pt"})
    st = SafeTensors.open(p)
    assert st.keys() == sorted(tensors) and st.metadata == {"format": "pt"}
    for k, v in tensors.items():
        assert torch.equal(st.load(k), v)
    with pytest.raises(KeyError):
        st.load("missing")
    st.close()
    # corrupt: offsets beyond the data region
    raw = open(p, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    hdr = json.loads(raw[8:8 + hlen])
    hdr["b.weight"]["data_offsets"][1] += 4
    bad = json.dumps(hdr).encode()
    q = str(tmp_path / "bad.safetensors")
    open(q, "wb").write(struct.pack("<Q", len(bad)) + bad + raw[8 + hlen:])
    with pytest.raises(SafeTensorsError):
        SafeTensors.open(q)
    # trailing garbage after the header object
    junk = raw[8:8 + hlen].rstrip() + b"x"
    open(q, "wb").write(struct.pack("<Q", len(junk)) + junk + raw[8 + hlen:])
    with pytest.raises(SafeTensorsError):
        SafeTensors.open(q)


def test_llama_checkpoint_roundtrip_hf_names(tmp_path):
    cfg = LlamaConfig(vocab_size=40, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, intermediate_size=48, max_position_embeddings=32)
    m = LlamaModel(cfg, init_std=0.1, seed=1)
    p = str(tmp_path / "model.safetensors")
    m.save_safetensors(p)
    keys = SafeTensors.open(p).keys()
    assert "model.layers.1.self_attn.k_proj.weight" in keys and "model.layers.0.mlp.gate_proj.weight" in keys
    assert "model.norm.weight" in keys and "lm_head.weight" in keys
    m2 = LlamaModel.from_pretrained(p, cfg)
    tok = torch.randint(0, 40, (1, 9))
    assert torch.equal(m(tok), m2(tok))
    extra = dict(load_file(p))
    extra["model.rotary_emb.inv_freq"] = torch.zeros(4)
    assert m2.load_hf_state_dict(extra) == ["model.rotary_emb.inv_freq"]
    del extra["model.norm.weight"]
    with pytest.raises(KeyError):
        m2.load_hf_state_dict(extra)


def test_whitespace_tokenizer():
    cfg = WhitespaceTokenizerConfig(vocab=["<unk>", "hello", "world", "<s>", "</s>"], unk="<unk>", bos="<s>", eos="</s>")
    tk = WhitespaceTokenizer(cfg)
    assert tk.encode("hello world", add_special_tokens=False) == [1, 2]
    assert tk.encode("hello there") == [3, 1, 0, 4]
    assert tk.decode([3, 1, 2, 4]) == "hello world"


def _tiny_bpe():
    from tesseract_b200.io.tokenizer import _B2U
    vocab = {_B2U[b]: b for b in range(256)}
    merges = [("h", "e"), ("l", "l"), ("he", "ll"), ("hell", "o"), ("Ġ", "w"), ("o", "r"), ("Ġw", "or"), ("Ġwor", "l"),
              ("Ġworl", "d")]
    nid = 256
    for a, b in merges:
        vocab[a + b] = nid
        nid += 1
    spec = {"model": {"type": "BPE", "vocab": vocab, "merges": [f"{a} {b}" for a, b in merges]},
            "added_tokens": [{"id": nid, "content": "<|begin_of_text|>"}, {"id": nid + 1, "content": "<|end_of_text|>"}]}
    return BpeTokenizer.from_json(json.dumps(spec)), vocab, nid


def test_bpe_tokenizer_merges_specials_and_roundtrip():
    tk, vocab, nid = _tiny_bpe()
    ids = tk.encode("hello world", add_special_tokens=False)
    assert ids == [vocab["hello"], vocab["Ġworld"]]
    assert tk.bos_id == nid and tk.eos_id == nid + 1
    full = tk.encode("hello<|end_of_text|> world's 123  x")
    assert full[0] == nid and (nid + 1) in full
    assert tk.decode(full) == "hello world's 123  x"
    assert tk.decode(full, skip_special_tokens=False).startswith("<|begin_of_text|>hello<|end_of_text|>")
    for text in ["naïve café ☕", "a  b\n\tc", "it's we're I'll", "x=1,y=22;"]:
        assert tk.decode(tk.encode(text, add_special_tokens=False)) == text


def test_pack_int8_and_int4():
    w = torch.randn(6, 64)
    w[2] = 0
    q, s = pack_int8_symmetric(w)
    assert q.dtype == torch.int8 and int(q.abs().max()) <= 127 and float(s[2]) == 1.0
    assert (q.float() * s[:, None] - w).abs().max() <= s.max() / 2 + 1e-6
    p4, s4 = pack_int4_group(w, 32)
    assert p4.shape == (6, 32) and s4.shape == (6, 2)
    deq = unpack_int4_group(p4, s4, 32)
    assert (deq - w).abs().max() <= s4.max() / 2 + 1e-6
    # nibble order: low nibble = even k, two's complement
    row = torch.zeros(1, 32)
    row[0, 0], row[0, 1] = 7.0, -7.0
    pk, _ = pack_int4_group(row, 32)
    assert int(pk[0, 0]) == (7 | (9 << 4))
    with pytest.raises(ValueError):
        pack_int4_group(w, 48)


def test_quantized_linear_close_to_fp_and_buffers():
    from tesseract_b200.nn import Linear
    lin = Linear(64, 24, bias=True)
    x = torch.randn(5, 64)
    ref = lin(x)
    q8 = QuantizedLinear.from_linear(lin)
    q4 = QuantizedLinearInt4G.from_linear(lin, 32)
    assert (q8(x) - ref).abs().max() < 0.05 and (q4(x) - ref).abs().max() < 0.5
    assert {n for n, _ in q8.named_buffers()} == {"q_weight", "weight_scale"}
    assert [n for n, _ in q8.named_parameters()] == ["bias"]
    assert q8.weight_bytes() < 0.3 * lin.weight.numel() * 4 and q4.weight_bytes() < 0.18 * lin.weight.numel() * 4


def test_quantized_model_keeps_top1():
    cfg = LlamaConfig(vocab_size=50, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                      intermediate_size=128, max_position_embeddings=32)
    m = LlamaModel(cfg, init_std=0.1, seed=2)
    tok = torch.randint(0, 50, (1, 12))
    ref = m(tok)[0, -1]
    m.quantize_(Scheme.Int8Symmetric())
    q = m(tok)[0, -1]
    assert int(q.argmax()) == int(ref.argmax())
    m.quantize_(Scheme.Int8Symmetric())  # idempotent
    assert len(m.generate([1, 2, 3], GenerateConfig(max_new_tokens=3))) == 6


def test_regex_automaton():
    a = RegexAutomaton(r"-?(0|[1-9]\d*)(\.\d+)?")
    for s in ["0", "-12", "3.14", "100.001"]:
        assert a.matches(s)
    for s in ["", "01", "1.", "--1", "1.2.3", "a"]:
        assert not a.matches(s)
    assert RegexAutomaton(r"(yes|no|maybe)").matches("maybe") and not RegexAutomaton(r"(yes|no)").matches("yesno")
    assert RegexAutomaton(r"[a-c]{2,3}x?").matches("abcx") and not RegexAutomaton(r"[a-c]{2,3}").matches("abca")
    assert RegexAutomaton(r"[^0-9]+\s\w{2}").matches("ab c_") and RegexAutomaton(r"a{2,}").matches("aaaa")
    d = RegexAutomaton(r"ab")
    assert d.step(d.start(), ord("x")) == K_DEAD and d.step(K_DEAD, ord("a")) == K_DEAD
    with pytest.raises(ValueError):
        RegexAutomaton("(ab")


def test_grammar_constraint_masks_tokens():
    vocab = [b"", b"1", b"2", b"12", b".", b"a", b"<eos>"]
    g = GrammarConstraint(RegexAutomaton(r"\d+(\.\d+)?"), vocab, eos_id=6)
    logits = np.zeros(7, dtype=np.float32)
    n = g.apply(logits)
    assert n == 3 and np.isinf(logits[[0, 4, 5, 6]]).all()       # digits only; EOS not yet accepting
    g.accept(3)
    logits[:] = 0
    g.apply(logits)
    assert not np.isinf(logits[[1, 2, 3, 4, 6]]).any() and np.isinf(logits[5])
    g.accept(4)
    logits[:] = 0
    assert g.apply(logits) == 3                                   # after "12." only digits
    g.accept(6)                                                   # EOS does not move the state
    dead = GrammarConstraint(RegexAutomaton(r"z"), vocab, eos_id=6)
    with pytest.raises(RuntimeError):
        dead.apply(np.zeros(7, dtype=np.float32))


def test_moe_sparse_equals_dense_and_aux_loss():
    torch.manual_seed(0)
    moe = MoEFeedForward(32, 48, num_experts=4, num_experts_per_tok=2)
    x = torch.randn(3, 5, 32)
    out = moe(x)
    assert torch.allclose(out, moe.forward_dense_reference(x), atol=1e-5)
    assert moe.aux_loss is not None and float(moe.aux_loss) > 0
    names = [n for n, _ in moe.named_parameters()]
    assert names[0] == "gate.weight" and "experts.3.down_proj.weight" in names
    all_e = MoEFeedForward(32, 48, num_experts=3, num_experts_per_tok=0)
    assert all_e.top_k == 3
    out.sum().backward()
    assert moe.gate.weight.grad is not None and moe.experts[0].gate_proj.weight.grad is not None


def test_mamba_recurrent_equals_full_scan():
    from tesseract_b200.nn.mamba import Mamba
    torch.manual_seed(0)
    blk = Mamba(32, d_state=8, d_conv=4, expand=2)
    x = torch.randn(2, 10, 32)
    full = blk(x)
    cache = blk.make_state_cache(2)
    steps = torch.cat([blk.forward_step(x[:, t:t + 1], cache) for t in range(10)], dim=1)
    assert torch.allclose(full, steps, atol=1e-5)
    names = [n for n, _ in blk.named_parameters()]
    assert {"conv_weight", "conv_bias", "A_log", "D", "in_proj.weight", "dt_proj.bias"} <= set(names)


def test_tesseract_python_surface():
    import tesseract as ts
    a = np.arange(12, dtype=np.float32).reshape(3, 4)
    t = ts.Tensor(a)
    assert t.shape == [3, 4] and t.dtype == ts.float32 and t.ndim == 2 and t.numel == 12 and t.device.is_cpu()
    np.testing.assert_array_equal(t.numpy(), a)
    assert ts.Tensor.ones([2, 3]).numpy().sum() == 6.0 and ts.Tensor.full([2], 2.5).numpy().sum() == 5.0
    x = ts.Tensor(np.ones((2, 3), dtype=np.float32))
    x.requires_grad = True
    w = ts.Tensor(np.ones((3, 4), dtype=np.float32))
    w.requires_grad = True
    loss = ts.ops.cross_entropy(x @ w, ts.Tensor(np.array([0, 1], dtype=np.int64)))
    assert x.grad() is None
    loss.backward()
    assert x.grad().shape == [2, 3] and isinstance(loss.item(), float)
    with pytest.raises(ValueError):
        ts.ops.matmul(x, x)
    with pytest.raises(TypeError):
        ts.ops.add(x, ts.Tensor(np.ones((2, 3), dtype=np.float64)))
    rng = np.random.default_rng(0)
    xs = ts.Tensor(rng.standard_normal((16, 8)).astype(np.float32))
    ys = ts.Tensor(rng.integers(0, 4, size=16).astype(np.int64))
    model = ts.nn.Sequential([ts.nn.Linear(8, 32), ts.nn.ReLU(), ts.nn.Linear(32, 4)])
    opt = ts.optim.Adam(model.parameters(), lr=0.05)
    losses = []
    for _ in range(60):
        l = ts.ops.cross_entropy(model(xs), ys)
        opt.zero_grad()
        l.backward()
        opt.step()
        losses.append(l.item())
    assert losses[-1] < 0.5 * losses[0]
    cfg = ts.models.MambaConfig()
    cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers, cfg.d_state = 24, 16, 2, 8
    mm = ts.models.MambaModel(cfg)
    gc = ts.models.MambaGenerateConfig()
    gc.max_new_tokens = 4
    assert len(mm.generate([1, 4, 2], gc)) == 7


def test_tesseract_python_surface_models_and_tokenizer():
    """The model and io part of the drop-in frontend (the reference's python/_core.cpp:247-360 surface): dense and
    MoE Llama and Mamba generate greedily and deterministically from a bare config; the whitespace tokenizer
    round-trips."""
    import tesseract as ts
    assert ts.__version__ and hasattr(ts.nn, "Linear") and hasattr(ts.models, "LlamaModel")
    for experts in (0, 4):
        cfg = ts.models.LlamaConfig()
        cfg.vocab_size, cfg.hidden_size, cfg.num_hidden_layers = 40, 16, 2
        cfg.num_attention_heads = cfg.num_key_value_heads = 4
        cfg.intermediate_size, cfg.max_position_embeddings = 32, 64
        if experts:
            cfg.num_experts, cfg.num_experts_per_tok = experts, 2
        model = ts.models.LlamaModel(cfg)
        gc = ts.models.LlamaGenerateConfig()
        gc.max_new_tokens = 6
        first = model.generate([3, 7, 11], gc)
        assert len(first) == 9 and first[:3] == [3, 7, 11] and model.generate([3, 7, 11], gc) == first
        assert all(0 <= t < 40 for t in first)
    tcfg = ts.io.WhitespaceTokenizerConfig()
    tcfg.vocab = ["<unk>", "paged", "decode", "kernel"]
    tcfg.unk = "<unk>"
    tk = ts.io.WhitespaceTokenizer(tcfg)
    ids = tk.encode("decode kernel paged", add_special_tokens=False)
    assert ids == [2, 3, 1] and tk.decode(ids) == "decode kernel paged"
    assert tk.encode("decode nothing", add_special_tokens=False) == [2, 0]


def test_fp8_block_scaling_restatement_cpu():
    """1 x 128 / 128 x 128 E4M3 quantisation and the block-scaled matmul (torch restatement used as the oracle of
    the CUDA kernels): scales, zero blocks, ragged N, round trip error."""
    from tesseract_b200.ops import fp8
    torch.manual_seed(0)
    x = torch.randn(70, 256) * 2
    w = torch.randn(200, 256) * 0.05
    x[3, 128:] = 0
    qa, sa = fp8.quantize_act(x)
    qb, sb = fp8.quantize_weight(w)
    assert qa.dtype == torch.uint8 and sa.shape == (2, 70) and sb.shape == (2, 2)
    assert sa[1, 3] == 1.0
    assert torch.allclose(sa[0], x[:, :128].abs().amax(1) / 448.0)
    assert (fp8.dequantize_act(qa, sa) - x).abs().max() <= x.abs().max() / 8          # 3 mantissa bits
    y = fp8.fp8_gemm(qa, sa, qb, sb).float()
    ref = x @ w.t()
    assert ((y - ref).norm() / ref.norm()) < 6e-2
    lin = fp8.Fp8Linear(w, bias=torch.ones(200))
    assert torch.allclose(lin(x).float(), y + 1.0, atol=2e-2)
