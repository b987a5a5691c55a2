"""Behavioural contracts of the serving stack on CPU: incremental == one-shot, paged == contiguous, INT8 close
to FP, scheduler == standalone generate, speculative == target greedy, disaggregated == monolithic."""
import numpy as np
import pytest
import torch

from tesseract_b200 import ops
from tesseract_b200.models import GenerateConfig, LlamaConfig, LlamaModel, Sampler, SamplingParams
from tesseract_b200.models.disaggregated import DisaggregatedEngine
from tesseract_b200.models.scheduler import ContinuousBatchingScheduler, EngineConfig
from tesseract_b200.models.speculative import SpeculativeDecoder
from tesseract_b200.nn.kv_cache import (BlockAllocator, KVCache, PagedKVCache, PagedKVPool, QuantizedKVCache,
                                        QuantizedPagedKVCache, QuantizedPagedKVPool, quantize_kv_per_token)


def make_model(seed=0, layers=2, vocab=96, d=64, heads=4, kv=2, ff=128, max_pos=128):
    cfg = LlamaConfig(vocab_size=vocab, hidden_size=d, num_hidden_layers=layers, num_attention_heads=heads,
                      num_key_value_heads=kv, intermediate_size=ff, max_position_embeddings=max_pos)
    return LlamaModel(cfg, init_std=0.2, seed=seed)


def test_forward_step_matches_full_forward():
    m = make_model()
    tok = torch.randint(0, 96, (2, 20))
    full = m(tok)
    caches = m.make_kv_caches(2, 32)
    a = m.forward_step(tok[:, :12], caches)
    parts = [a]
    for t in range(12, 20):
        parts.append(m.forward_step(tok[:, t:t + 1], caches))
    inc = torch.cat(parts, dim=1)
    assert torch.allclose(inc, full, atol=2e-4)


def test_chunked_prefill_matches_full_forward():
    m = make_model(seed=1)
    tok = torch.randint(0, 96, (1, 24))
    full = m(tok)
    caches = m.make_kv_caches(1, 32)
    parts = [m.forward_step(tok[:, :8], caches), m.forward_step(tok[:, 8:19], caches), m.forward_step(tok[:, 19:], caches)]
    assert torch.allclose(torch.cat(parts, dim=1), full, atol=2e-4)


def test_kv_cache_overflow_and_rewind():
    c = KVCache(1, 2, 4, 8)
    k = torch.randn(1, 2, 3, 8)
    c.append(k, k)
    assert c.current_len() == 3
    with pytest.raises(RuntimeError):
        c.append(k, k)
    c.set_current_len(1)
    assert c.keys_view().shape == (1, 2, 1, 8)
    with pytest.raises(ValueError):
        c.append(torch.randn(1, 3, 1, 8), torch.randn(1, 3, 1, 8))


def test_block_allocator_contract():
    a = BlockAllocator(3)
    assert [a.allocate(), a.allocate(), a.allocate()] == [0, 1, 2]
    with pytest.raises(RuntimeError):
        a.allocate()
    a.free(1)
    assert a.allocate() == 1
    a.free(0)
    with pytest.raises(RuntimeError):
        a.free(0)


def test_paged_cache_equals_contiguous_and_recycles_blocks():
    pool = PagedKVPool(8, 2, 4, 8)
    pc = PagedKVCache(pool, 20)
    cc = KVCache(1, 2, 20, 8)
    for n in (5, 1, 1, 6):
        k, v = torch.randn(1, 2, n, 8), torch.randn(1, 2, n, 8)
        pc.append(k, v)
        cc.append(k, v)
    assert torch.equal(pc.keys_view(), cc.keys_view()) and torch.equal(pc.values_view(), cc.values_view())
    assert pc.num_blocks_held() == 4 and pool.allocator.num_free() == 4
    pc.reset()
    assert pool.allocator.num_free() == 8


def test_int8_kv_roundtrip_error_bound():
    x = torch.randn(3, 2, 7, 16)
    q, s = quantize_kv_per_token(x)
    err = (q.float() * s[..., None] - x).abs()
    assert (err <= s[..., None] / 2 + 1e-5).all()
    zq, zs = quantize_kv_per_token(torch.zeros(1, 1, 1, 8))
    assert float(zs) == 1.0 and int(zq.abs().max()) == 0
    qc = QuantizedKVCache(3, 2, 8, 16)
    qc.append(x, x)
    assert (qc.keys_view() - x).abs().max() < 0.05


def test_paged_decode_op_matches_gather_attention():
    pool = PagedKVPool(16, 2, 4, 16)
    caches = [PagedKVCache(pool, 40) for _ in range(3)]
    lens = [9, 4, 13]
    for c, n in zip(caches, lens):
        c.append(torch.randn(1, 2, n, 16), torch.randn(1, 2, n, 16))
    q = torch.randn(3, 4, 16)
    tables = torch.zeros(3, 4, dtype=torch.int32)
    for i, c in enumerate(caches):
        tables[i, :len(c.block_table)] = torch.tensor(c.block_table, dtype=torch.int32)
    out = ops.paged_decode_attention(q, pool.k, pool.v, tables, torch.tensor(lens, dtype=torch.int32))
    for i, c in enumerate(caches):
        ref = ops.attention_ref(q[i][None, :, None, :], c.keys_view(), c.values_view(), causal=False)[0, :, 0]
        assert torch.allclose(out[i], ref, atol=1e-5)


def test_int8_paged_matches_fp_on_dequantised_pool():
    qpool = QuantizedPagedKVPool(8, 2, 4, 16)
    c = QuantizedPagedKVCache(qpool, 16)
    c.append(torch.randn(1, 2, 10, 16), torch.randn(1, 2, 10, 16))
    q = torch.randn(1, 4, 16)
    tables = torch.tensor([c.block_table + [0]], dtype=torch.int32)
    lens = torch.tensor([10], dtype=torch.int32)
    got = ops.paged_decode_attention_int8(q, qpool.k, qpool.v, qpool.k_scale, qpool.v_scale, tables, lens)
    ref = ops.attention_ref(q[:, :, None, :], c.keys_view(), c.values_view(), causal=False)[:, :, 0]
    assert torch.allclose(got, ref, atol=1e-5)


def test_batched_decode_equals_per_request():
    m = make_model(seed=3)
    pools = m.make_layer_pools(32, 4)
    prompts = [[1, 2, 3, 4, 5], [7, 8], [9, 10, 11]]
    per_seq = []
    for p in prompts:
        caches = m.make_paged_kv_caches(pools, 32)
        m.forward_step(torch.tensor([p]), caches)
        per_seq.append(caches)
    toks = torch.tensor([[11], [12], [13]])
    batched = m.forward_step_batched(toks, per_seq)
    for i, p in enumerate(prompts):
        caches = m.make_kv_caches(1, 32)
        m.forward_step(torch.tensor([p]), caches)
        single = m.forward_step(toks[i:i + 1], caches)
        assert torch.allclose(batched[i], single[0], atol=1e-5)


def test_generate_contract():
    m = make_model(seed=4)
    out = m.generate([1, 5, 9, 3], GenerateConfig(max_new_tokens=6))
    assert len(out) == 10 and out[:4] == [1, 5, 9, 3]
    assert m.generate([1, 5, 9, 3], GenerateConfig(max_new_tokens=6)) == out
    eos = out[5]
    stopped = m.generate([1, 5, 9, 3], GenerateConfig(max_new_tokens=6, eos_token_id=eos))
    assert stopped[-1] == eos and len(stopped) <= len(out)
    with pytest.raises(ValueError):
        m.generate([1, 999], GenerateConfig(max_new_tokens=1))
    with pytest.raises(ValueError):
        m.generate([1], GenerateConfig(max_new_tokens=-1))
    assert m.generate([1, 2], GenerateConfig(max_new_tokens=0)) == [1, 2]
    s1 = m.generate([1, 5], GenerateConfig(max_new_tokens=8, do_sample=True, seed=7, sampling=SamplingParams(temperature=0.9, top_k=20, top_p=0.95)))
    s2 = m.generate([1, 5], GenerateConfig(max_new_tokens=8, do_sample=True, seed=7, sampling=SamplingParams(temperature=0.9, top_k=20, top_p=0.95)))
    assert s1 == s2


@pytest.mark.parametrize("kv_int8", [False, True])
def test_scheduler_equals_standalone_generate(kv_int8):
    m = make_model(seed=5)
    prompts = [[1, 2, 3], [4, 5, 6, 7, 8, 9], [10], [11, 12, 13, 14], [3, 3, 3]]
    gens = [GenerateConfig(max_new_tokens=5, kv_int8=kv_int8),
            GenerateConfig(max_new_tokens=9, kv_int8=kv_int8, do_sample=True, seed=11, sampling=SamplingParams(temperature=0.8, top_k=10)),
            GenerateConfig(max_new_tokens=3, kv_int8=kv_int8),
            GenerateConfig(max_new_tokens=7, kv_int8=kv_int8, do_sample=True, seed=3, sampling=SamplingParams(top_p=0.9)),
            GenerateConfig(max_new_tokens=0, kv_int8=kv_int8)]
    sched = ContinuousBatchingScheduler(m, EngineConfig(block_size=4, num_blocks=16, max_seq_len=32, max_batch_size=3, kv_int8=kv_int8))
    ids = [sched.add_request(p, g) for p, g in zip(prompts, gens)]
    sched.run()
    assert sched.free_blocks() == 16 and sched.allocated_blocks() == 0
    for rid, p, g in zip(ids, prompts, gens):
        assert sched.is_finished(rid)
        assert sched.result(rid) == m.generate(p, g)


def test_scheduler_tiny_pool_head_of_line():
    m = make_model(seed=6)
    sched = ContinuousBatchingScheduler(m, EngineConfig(block_size=4, num_blocks=3, max_seq_len=12, max_batch_size=4))
    a = sched.add_request([1] * 8, GenerateConfig(max_new_tokens=4))
    b = sched.add_request([2] * 8, GenerateConfig(max_new_tokens=4))
    sched.step()
    assert sched.num_running() == 1 and sched.num_waiting() == 1
    sched.run()
    assert sched.result(a) == m.generate([1] * 8, GenerateConfig(max_new_tokens=4))
    assert sched.result(b) == m.generate([2] * 8, GenerateConfig(max_new_tokens=4))
    with pytest.raises(ValueError):
        sched.add_request([1] * 20, GenerateConfig(max_new_tokens=4))


def test_speculative_equals_target_greedy():
    target = make_model(seed=8, layers=2)
    draft = make_model(seed=9, layers=1)
    want = target.generate([5, 6, 7], GenerateConfig(max_new_tokens=12))
    for gamma in (1, 3, 5):
        res = SpeculativeDecoder(target, draft, gamma).generate([5, 6, 7], 12)
        assert res.tokens == want
        assert res.proposed >= res.accepted and res.rounds > 0 and res.target_forwards >= res.rounds
    same = SpeculativeDecoder(target, target, 4).generate([5, 6, 7], 12)
    assert same.tokens == want and same.accepted > 0


def test_disaggregated_equals_monolithic():
    m = make_model(seed=10)
    eng = DisaggregatedEngine(m, m)
    assert eng.generate([4, 3, 2, 1], 9) == m.generate([4, 3, 2, 1], GenerateConfig(max_new_tokens=9))
    kv = eng.prefill([4, 3, 2, 1])
    assert kv.prompt_len == 4 and kv.nbytes() > 0


def test_sampler_rules():
    logits = np.array([1.0, 3.0, 3.0, -2.0, 0.5], dtype=np.float32)
    s = Sampler(SamplingParams(temperature=0.0))
    assert s.sample(logits) == 1                      # lowest index on ties, RNG untouched
    assert Sampler(SamplingParams(temperature=1.0, top_k=1), seed=3).sample(np.array([0.0, 5.0, 1.0], np.float32)) == 1
    draws = [Sampler(SamplingParams(temperature=1.0, top_p=0.5), seed=i).sample(np.array([5.0, 4.9, -9.0], np.float32)) for i in range(20)]
    assert set(draws) <= {0, 1}
    pen = Sampler(SamplingParams(temperature=0.0, repetition_penalty=2.0))
    assert pen.sample(np.array([2.0, 1.5, -1.0], np.float32), [0]) == 1
    a = [Sampler(SamplingParams(temperature=1.0), seed=42).sample(logits) for _ in range(3)]
    assert a[0] == a[1] == a[2]


def test_mt19937_64_known_values():
    from tesseract_b200.models import MT19937_64
    g = MT19937_64(5489)
    first = [g.next_u64() for _ in range(3)]
    assert first == [14514284786278117030, 4620546740167642908, 13109570281517897720]
    for _ in range(9996):
        g.next_u64()
    assert g.next_u64() == 9981545732273789042   # 10000th draw of a default-seeded std::mt19937_64


def test_vocab_shard_rows_cover_the_vocabulary_in_whole_scale_blocks():
    """Vocabulary-parallel LM head: shards of a multiple of 128 rows (fp8 block scales stay whole), every rank holds
    some rows, together they cover the vocabulary; too small a vocabulary keeps the head replicated (0)."""
    from tesseract_b200.serving.engine import vocab_shard_rows
    for vocab in (2048, 32000, 128256, 151936, 1000, 257):
        for world in (2, 4, 8):
            shard = vocab_shard_rows(vocab, world)
            if shard == 0:
                assert (world - 1) * ((vocab + world * 128 - 1) // (world * 128) * 128) >= vocab
                continue
            assert shard % 128 == 0 and (world - 1) * shard < vocab <= world * shard
            sizes = [min(vocab, (r + 1) * shard) - r * shard for r in range(world)]
            assert all(s > 0 for s in sizes) and sum(sizes) == vocab
    assert vocab_shard_rows(128, 2) == 0 and vocab_shard_rows(128256, 8) == 16128


def test_paged_prefill_every_new_token_is_a_decode_query_with_its_own_length():
    """The formulation the GPU path of ``paged_prefill_attention`` uses -- new token s of a request attends the first
    len - S + s + 1 pooled keys through the same block table -- equals the chunked-prefill reference."""
    from tesseract_b200 import ops
    torch.manual_seed(3)
    A, S, H, Hkv, D, bs = 2, 5, 4, 2, 16, 4
    lens = torch.tensor([13, 5])
    nb = 12
    k_pool, v_pool = torch.randn(nb, Hkv, bs, D), torch.randn(nb, Hkv, bs, D)
    tables = torch.tensor([[0, 1, 2, 3], [4, 5, 0, 0]])
    q = torch.randn(A, S, H, D)
    ref = ops.paged_attention_ref(q, k_pool, v_pool, tables, lens)
    steps = torch.arange(S)
    q_lens = (lens[:, None] - (S - 1) + steps[None, :]).clamp_min(0).reshape(-1)
    q_tables = tables.repeat_interleave(S, dim=0)
    one = ops.paged_attention_ref(q.reshape(A * S, 1, H, D), k_pool, v_pool, q_tables, q_lens).view(A, S, H, D)
    assert torch.allclose(one, ref, atol=1e-5)
    assert torch.allclose(ops.paged_prefill_attention(q, k_pool, v_pool, tables, lens), ref, atol=1e-5)
