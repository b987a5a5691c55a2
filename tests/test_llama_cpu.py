"""Tiny Llama on CPU (fp32): arena + fused loss parity with plain autograd, one Adam step, config parsing."""
import json

import torch

from tesseract_b200.models import LlamaConfig, LlamaModel, llama_local_to_hf_name
from tesseract_b200.optim import Adam, ParamArena
from tesseract_b200.training import TrainConfig, Trainer


def tiny_cfg(**kw):
    base = dict(vocab_size=512, hidden_size=256, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
                intermediate_size=688, max_position_embeddings=256, rope_theta=10000.0, rms_norm_eps=1e-5)
    base.update(kw)
    return LlamaConfig(**base)


def test_parameter_names_match_reference_layout():
    m = LlamaModel(tiny_cfg(num_hidden_layers=1))
    names = [n for n, _ in m.named_parameters()]
    assert names == ["embed_tokens.weight", "layers.0.norm_1.weight", "layers.0.attn.q_proj.weight",
                     "layers.0.attn.k_proj.weight", "layers.0.attn.v_proj.weight", "layers.0.attn.o_proj.weight",
                     "layers.0.norm_2.weight", "layers.0.ffn.gate_proj.weight", "layers.0.ffn.up_proj.weight",
                     "layers.0.ffn.down_proj.weight", "norm.weight", "lm_head.weight"]
    assert llama_local_to_hf_name("layers.3.attn.q_proj.weight") == "model.layers.3.self_attn.q_proj.weight"
    assert llama_local_to_hf_name("layers.0.norm_2.weight") == "model.layers.0.post_attention_layernorm.weight"
    assert llama_local_to_hf_name("lm_head.weight") == "lm_head.weight"


def test_fused_loss_and_arena_grads_match_autograd():
    torch.manual_seed(0)
    m = LlamaModel(tiny_cfg(), init_std=0.02)
    tok = torch.randint(0, 512, (4, 128))
    tgt = torch.randint(0, 512, (4, 128))
    ref_loss = torch.nn.functional.cross_entropy(m(tok).view(-1, 512), tgt.view(-1))
    ref_loss.backward()
    ref = {n: p.grad.clone() for n, p in m.named_parameters()}
    m.zero_grad()
    ParamArena.from_module(m)
    loss = m.loss(tok, tgt, chunk_rows=100)
    loss.backward()
    assert abs(loss.item() - ref_loss.item()) < 1e-5
    for n, p in m.named_parameters():
        assert p.grad is None
        assert torch.allclose(p.main_grad, ref[n], atol=1e-6), n


def test_train_step_reduces_loss_and_microbatching_is_equivalent():
    torch.manual_seed(1)
    batch = torch.randint(0, 512, (4, 65))
    losses = {}
    for mb in (4, 1):
        torch.manual_seed(2)
        m = LlamaModel(tiny_cfg(num_hidden_layers=2), init_std=0.02, seed=5)
        tr = Trainer(m, TrainConfig(lr=1e-3, micro_batch=mb))
        l0 = tr.train_step(batch)
        l1 = tr.train_step(batch)
        assert l1 < l0
        losses[mb] = (l0, l1)
    assert abs(losses[4][0] - losses[1][0]) < 1e-5
    assert abs(losses[4][1] - losses[1][1]) < 1e-4


def test_overfits_fixed_batch():
    """The reference's training contract: a fixed tiny batch is memorised (tests/models/test_llama_train.cpp:47-95)."""
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=64, hidden_size=64, num_hidden_layers=2, num_attention_heads=4,
                      intermediate_size=128, max_position_embeddings=32)
    m = LlamaModel(cfg, init_std=0.02, seed=1)
    tr = Trainer(m, TrainConfig(lr=3e-3, micro_batch=2))
    batch = torch.randint(0, 64, (2, 17))
    first = tr.train_step(batch)
    for _ in range(119):
        last = tr.train_step(batch)
    assert last < first and last < 0.1


def test_config_from_json():
    cfg = LlamaConfig.from_json(json.dumps({"vocab_size": 100, "hidden_size": 64, "num_local_experts": 4,
                                            "num_experts_per_tok": 2, "torch_dtype": "bfloat16", "rope_theta": 5e5,
                                            "tie_word_embeddings": True, "unknown": {"a": 1}, "eos_token_id": 7}))
    assert cfg.vocab_size == 100 and cfg.num_experts == 4 and cfg.dtype == torch.bfloat16
    assert cfg.rope_theta == 5e5 and cfg.tie_word_embeddings and cfg.eos_token_id == 7
    assert cfg.kv_heads() == cfg.num_attention_heads
