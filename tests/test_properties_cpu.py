"""Property tests (hypothesis) of the host-side pieces whose contracts are "lossless" or "twin-identical": byte-level BPE,
safetensors files, the KV block allocator (the reference tests these with fixed cases, tests/io/test_bpe_tokenizer.cpp,
tests/io/test_safetensors.cpp, tests/nn/test_paged_kv_cache.cpp)."""
import os

import numpy as np
import pytest
import torch
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

FIX = os.path.join(os.path.dirname(__file__), "fixtures", "hf_bpe", "tokenizer.json")
# derandomised: every run draws the same examples (explore with --hypothesis-seed=N and derandomize off)
_SETTINGS = dict(max_examples=60, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow])


@settings(**_SETTINGS)
@given(st.text(max_size=80))
def test_byte_level_bpe_is_lossless_and_the_twins_agree(text):
    from tesseract_b200.io.tokenizer import BpeTokenizer
    native = BpeTokenizer.from_file(FIX)
    os.environ["TESSERACT_HOST"] = "python"
    try:
        twin = BpeTokenizer.from_file(FIX)
        ids_twin = twin.encode(text, add_special_tokens=False)
    finally:
        os.environ.pop("TESSERACT_HOST", None)
    ids = native.encode(text, add_special_tokens=False)
    assert ids == ids_twin
    assert all(0 <= i < native.vocab_size() for i in ids)
    try:
        text.encode("utf-8")
    except UnicodeEncodeError:            # lone surrogates cannot be bytes in the first place
        return
    assert native.decode(ids) == text


_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.int8, torch.uint8, torch.bool]


@settings(**_SETTINGS)
@given(st.lists(st.tuples(st.sampled_from(range(len(_DTYPES))), st.lists(st.integers(0, 5), min_size=0, max_size=3)),
                min_size=1, max_size=5), st.integers(0, 2 ** 31 - 1))
def test_safetensors_round_trip_any_dtype_and_shape(tmp_path_factory, specs, seed):
    from tesseract_b200.io import safetensors as sft
    g = torch.Generator().manual_seed(seed)
    tensors = {}
    for k, (di, shape) in enumerate(specs):
        dt = _DTYPES[di]
        if dt.is_floating_point:
            t = torch.randn(shape, generator=g).to(dt)
        elif dt == torch.bool:
            t = torch.randint(0, 2, shape, generator=g).bool()
        else:
            t = torch.randint(0, 100, shape, generator=g).to(dt)
        tensors[f"t{k}.weight"] = t
    path = str(tmp_path_factory.mktemp("st") / "x.safetensors")
    sft.save_file(tensors, path, metadata={"note": "round trip"})
    for loader in (sft.load_file, sft.load_file_parallel):
        back = loader(path)
        assert set(back) == set(tensors)
        for name, t in tensors.items():
            assert back[name].dtype == t.dtype and tuple(back[name].shape) == tuple(t.shape)
            assert torch.equal(back[name].cpu(), t)


@settings(**_SETTINGS)
@given(st.integers(1, 40), st.lists(st.integers(0, 99), max_size=120))
def test_block_allocator_twins_hand_out_the_same_blocks(num_blocks, script):
    """A random script of allocate / free calls: the native allocator and its Python twin return the same block ids,
    raise at the same points, and never hand out a block twice."""
    from tesseract_b200 import _native
    from tesseract_b200.nn.kv_cache import BlockAllocator
    host = _native.host()
    if host is None:
        pytest.skip("native host runtime not built")
    os.environ["TESSERACT_HOST"] = "python"
    try:
        twin = BlockAllocator(num_blocks)
    finally:
        os.environ.pop("TESSERACT_HOST", None)
    nat = BlockAllocator(num_blocks)
    held = []
    for step in script:
        if step % 3 and len(held) < num_blocks:                       # allocate
            a, b = nat.allocate(), twin.allocate()
            assert a == b and a not in held and 0 <= a < num_blocks
            held.append(a)
        elif held:                                                    # free one of the held blocks
            blk = held.pop(step % len(held))
            nat.free(blk)
            twin.free(blk)
        else:                                                         # nothing held: an allocation, or a refusal
            try:
                a = nat.allocate()
            except RuntimeError:
                with pytest.raises(RuntimeError):
                    twin.allocate()
                continue
            assert a == twin.allocate()
            held.append(a)
        assert nat.num_free() == twin.num_free() == num_blocks - len(held)
        assert nat.num_used() == twin.num_used() == len(held)
    if len(held) == num_blocks:
        with pytest.raises(RuntimeError):
            nat.allocate()


@settings(**_SETTINGS)
@given(st.integers(2, 400), st.floats(0.05, 3.0), st.sampled_from([0, 1, 5, 50]), st.sampled_from([1.0, 0.95, 0.5, 0.05]),
       st.sampled_from([1.0, 1.3]), st.floats(0.01, 6.0), st.integers(0, 2 ** 31 - 1))
def test_sampler_twins_draw_the_same_tokens(V, temperature, top_k, top_p, penalty, spread, seed):
    from tesseract_b200 import _native
    from tesseract_b200.models.sampler import Sampler, SamplingParams
    if _native.host() is None:
        pytest.skip("native host runtime not built")
    rng = np.random.default_rng(seed)
    logits = torch.from_numpy((rng.standard_normal(V) * spread).astype(np.float32))
    if seed % 3 == 0:
        logits = torch.round(logits * 2) / 2                     # ties
    sp = SamplingParams(temperature=temperature, top_k=top_k, top_p=top_p, repetition_penalty=penalty)
    a, b = Sampler(sp, seed=seed, native=True), Sampler(sp, seed=seed, native=False)
    prev = rng.integers(0, V, size=5).tolist()
    for _ in range(3):
        ta, tb = a.sample(logits, prev), b.sample(logits, prev)
        assert ta == tb and 0 <= ta < V
        prev.append(ta)


@settings(**_SETTINGS)
@given(st.integers(1, 6), st.integers(1, 4), st.sampled_from([32, 64, 128]), st.integers(0, 2 ** 31 - 1))
def test_int4_and_int8_packing_round_trip(rows, groups, group, seed):
    from tesseract_b200 import quant
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, groups * group, generator=g) * 3
    q8, s8 = quant.pack_int8_symmetric(w)
    assert q8.dtype == torch.int8 and int(q8.abs().max()) <= 127
    assert (q8.float() * s8[:, None] - w).abs().max() <= s8.max() * 0.5 + 1e-6          # half a quantisation step
    q4, s4 = quant.pack_int4_group(w, group)
    back = quant.unpack_int4_group(q4, s4, group)
    step = s4.repeat_interleave(group, dim=1)
    assert back.shape == w.shape and ((back - w).abs() <= step * 0.5 + 1e-6).all()
    q4b, s4b = quant.pack_int4_group(back, group)                                       # its own values re-pack exactly
    assert torch.allclose(quant.unpack_int4_group(q4b, s4b, group), back, atol=1e-5)


@settings(**_SETTINGS)
@given(st.integers(1, 300), st.sampled_from([128, 256, 512]), st.integers(0, 2 ** 31 - 1))
def test_mx_scale_layouts_are_inverse_and_quantisation_error_is_bounded(M, K, seed):
    """The two scale-factor layouts of the MX activation quantiser carry the same exponents; dequantised values are
    within one E4M3 step of the input; every scale is a power of two that keeps its block inside the E4M3 range."""
    from tesseract_b200.ops import fp8
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(M, K, generator=g) * (10.0 ** float(torch.randint(-3, 3, (1,), generator=g)))).bfloat16()
    q, sf = fp8.quantize_act_mx_ref(x)
    qa, atoms = fp8.quantize_act_mx_ref(x, atoms=True)
    assert torch.equal(q, qa) and atoms.dim() == 3
    assert torch.equal(fp8._atoms_to_words(atoms)[:, :M], sf[:, :M])
    assert torch.equal(fp8._atoms_to_words(fp8._words_to_atoms(sf)), sf)
    back = fp8.dequantize_act_mx(q, sf).float()
    blocks = x.float().view(M, K // 32, 32).abs().amax(-1)
    tol = (blocks / 448.0 * 2 * 32).clamp_min(2.0 ** -20).repeat_interleave(32, dim=1)   # <= 2^-3 relative (3 mantissa bits) of the scaled block, with slack
    assert ((back - x.float()).abs() <= tol).all()
    assert torch.equal(fp8.dequantize_act_mx(qa, atoms).float(), back)


@settings(**_SETTINGS)
@given(st.sampled_from([1, 3, 4, 16]), st.lists(st.tuples(st.sampled_from(["append", "rewind", "reset"]), st.integers(1, 9)),
                                                  min_size=1, max_size=14), st.booleans(), st.integers(0, 2 ** 31 - 1))
def test_paged_cache_behaves_like_the_contiguous_cache(block_size, script, int8, seed):
    """A random script of appends (1 .. 9 tokens), rewinds (``set_current_len``) and resets: a paged view holds what the
    contiguous cache of the same kind holds, uses ceil(len / block) blocks, and gives every block back on reset."""
    from tesseract_b200.nn.kv_cache import (KVCache, PagedKVCache, PagedKVPool, QuantizedKVCache,
                                            QuantizedPagedKVCache, QuantizedPagedKVPool)
    H, D, max_len = 2, 8, 64
    g = torch.Generator().manual_seed(seed)
    if int8:
        pool = QuantizedPagedKVPool(40, H, block_size, D)
        paged, flat = QuantizedPagedKVCache(pool, max_len), QuantizedKVCache(1, H, max_len, D)
    else:
        pool = PagedKVPool(40, H, block_size, D)
        paged, flat = PagedKVCache(pool, max_len), KVCache(1, H, max_len, D)
    free0 = pool.allocator.num_free()
    for action, n in script:
        if action == "append":
            if flat.current_len() + n > max_len:
                continue
            k, v = torch.randn(1, H, n, D, generator=g), torch.randn(1, H, n, D, generator=g)
            paged.append(k, v)
            flat.append(k, v)
        elif action == "rewind":
            keep = flat.current_len() * n // 10
            paged.set_current_len(keep)
            flat.set_current_len(keep)
        else:
            paged.reset()
            flat.reset()
            assert pool.allocator.num_free() == free0
        L = flat.current_len()
        assert paged.current_len() == L
        assert paged.num_blocks_held() >= (L + block_size - 1) // block_size
        assert torch.equal(paged.keys_view(), flat.keys_view()) and torch.equal(paged.values_view(), flat.values_view())
    paged.reset()
    assert pool.allocator.num_free() == free0


_UNARY = ["relu", "sigmoid", "tanh", "exp", "neg"]
_BINARY = ["add", "sub", "mul"]


@settings(**_SETTINGS)
@given(st.lists(st.tuples(st.sampled_from(_UNARY + _BINARY + ["matmul", "softmax", "transpose"]), st.integers(0, 7)),
                min_size=1, max_size=8), st.integers(0, 2 ** 31 - 1))
def test_recorded_graphs_replay_and_differentiate_like_eager(ops_script, seed):
    """Random chains of recorded ops over two 4 x 4 inputs and a 4 x 4 parameter: the interpreter returns the eager
    result, the text form parses back to a graph that runs the same, and the backward transform gives autograd's
    gradient of the result with respect to the parameter (dead ops, fused patterns and all)."""
    from tesseract_b200.graph import GraphScope, build_backward, emit_mlir, parse_mlir, run
    g = torch.Generator().manual_seed(seed)
    a, b = torch.randn(4, 4, generator=g) * 0.5, torch.randn(4, 4, generator=g) * 0.5
    w = torch.randn(4, 4, generator=g) * 0.5

    def program(x, y, p):
        vals = [x, y, p]
        for kind, pick in ops_script:
            u, v = vals[pick % len(vals)], vals[(pick // 2) % len(vals)]
            if kind in _UNARY:
                r = -u if kind == "neg" else getattr(torch, kind)(u)
            elif kind in _BINARY:
                r = {"add": u + v, "sub": u - v, "mul": u * v}[kind]
            elif kind == "matmul":
                r = u @ v
            elif kind == "softmax":
                r = torch.softmax(u, dim=-1)
            else:
                r = u.transpose(0, 1)
            vals.append(r)
        return (vals[-1] * p).sum()

    wg = w.clone().requires_grad_()
    ref = program(a, b, wg)
    (gw,) = torch.autograd.grad(ref, wg)
    with GraphScope() as scope:
        ia, ib, iw = scope.bind_input(a, "a"), scope.bind_input(b, "b"), scope.bind_param(w, "w")
        scope.mark_output(program(a, b, w))
    graph = scope.graph
    bind = {ia: a, ib: b, iw: w}
    assert torch.allclose(run(graph, bind)[0], ref.detach(), atol=1e-5, rtol=1e-5)
    again = parse_mlir(emit_mlir(graph))
    rebind = dict(zip(list(again.inputs) + list(again.params), [a, b, w]))
    assert torch.allclose(run(again, rebind)[0], ref.detach(), atol=1e-5, rtol=1e-5)
    res = build_backward(graph)
    bind[res.cotangents[0]] = torch.ones(())
    outs = run(graph, bind)
    assert len(outs) == 2 and torch.allclose(outs[1], gw, atol=1e-4, rtol=1e-4)


_MODEL = {}


def _tiny_model():
    if "m" not in _MODEL:
        from tesseract_b200.models import LlamaConfig, LlamaModel
        torch.manual_seed(21)
        _MODEL["m"] = LlamaModel(LlamaConfig(vocab_size=48, hidden_size=32, num_hidden_layers=2, num_attention_heads=4,
                                             num_key_value_heads=2, intermediate_size=64, max_position_embeddings=64,
                                             dtype=torch.float32))
    return _MODEL["m"]


@settings(max_examples=25, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow])
@given(st.lists(st.tuples(st.integers(1, 9), st.integers(0, 6), st.booleans(), st.integers(0, 47)), min_size=1, max_size=6),
       st.sampled_from([2, 4]), st.integers(1, 4), st.booleans(), st.integers(0, 2 ** 31 - 1))
def test_scheduler_results_equal_standalone_generation(requests, block_size, max_batch, kv_int8, seed):
    """Random mixes of requests (prompt length, budget, greedy or seeded sampling, an EOS id that may or may not come
    up) through the continuous-batching scheduler with a small pool and batch: every result equals a standalone
    ``generate`` of the same request, and the pool is whole again at the end."""
    from tesseract_b200.models import GenerateConfig
    from tesseract_b200.models.sampler import SamplingParams
    from tesseract_b200.models.scheduler import ContinuousBatchingScheduler, EngineConfig
    m = _tiny_model()
    rng = np.random.default_rng(seed)
    sched = ContinuousBatchingScheduler(m, EngineConfig(block_size=block_size, num_blocks=24, max_seq_len=24,
                                                        max_batch_size=max_batch, kv_int8=kv_int8))
    jobs = []
    for plen, budget, sample, eos in requests:
        prompt = rng.integers(0, 48, size=plen).tolist()
        gen = GenerateConfig(max_new_tokens=budget, kv_int8=kv_int8, eos_token_id=eos if eos % 3 == 0 else -1,
                             do_sample=sample, seed=int(rng.integers(0, 1000)),
                             sampling=SamplingParams(temperature=0.9, top_k=12, top_p=0.9))
        jobs.append((sched.add_request(prompt, gen), prompt, gen))
    sched.run()
    assert sched.free_blocks() == 24 and not sched.has_pending()
    for rid, prompt, gen in jobs:
        assert sched.result(rid) == m.generate(prompt, gen)


@settings(max_examples=25, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow])
@given(st.integers(1, 8), st.integers(1, 7), st.integers(0, 14), st.integers(0, 2 ** 31 - 1))
def test_speculative_and_disaggregated_generation_equal_plain_greedy(plen, gamma, budget, seed):
    """Whatever the draft length, the prompt and the budget: speculative decoding returns the target's greedy tokens
    (with a draft model that disagrees and with the target as its own draft), and a prefill engine handing its KV to
    a decode engine returns the monolithic result."""
    from tesseract_b200.models import GenerateConfig, LlamaConfig, LlamaModel
    from tesseract_b200.models.disaggregated import DisaggregatedEngine
    from tesseract_b200.models.speculative import SpeculativeDecoder
    target = _tiny_model()
    if "draft" not in _MODEL:
        torch.manual_seed(22)
        _MODEL["draft"] = LlamaModel(LlamaConfig(vocab_size=48, hidden_size=32, num_hidden_layers=1, num_attention_heads=4,
                                                 num_key_value_heads=2, intermediate_size=64, max_position_embeddings=64,
                                                 dtype=torch.float32))
    prompt = np.random.default_rng(seed).integers(0, 48, size=plen).tolist()
    want = target.generate(prompt, GenerateConfig(max_new_tokens=budget))
    for draft in (_MODEL["draft"], target):
        res = SpeculativeDecoder(target, draft, gamma).generate(prompt, budget)
        assert res.tokens == want and res.proposed >= res.accepted
    assert DisaggregatedEngine(target, target).generate(prompt, budget) == want


@settings(max_examples=30, deadline=None, derandomize=True, suppress_health_check=[HealthCheck.too_slow])
@given(st.sampled_from([1, 2, 3, 4, 6]), st.integers(1, 5), st.integers(1, 4), st.integers(1, 6), st.booleans(),
       st.integers(0, 2 ** 31 - 1))
def test_simulated_tensor_parallel_mlp_equals_dense(world, rows, in_mult, hid_mult, bias, seed):
    """Column-parallel up projection, row-parallel down projection over the in-process communication backend, any
    shard count that divides the hidden width: forward values and every gradient equal the dense layers'."""
    from tesseract_b200.nn import Linear
    from tesseract_b200.parallel import ColumnParallelLinear, RowParallelLinear, SimCommBackend
    torch.manual_seed(seed % 1000)
    d_in, d_hid = 4 * in_mult, world * hid_mult
    up, down = Linear(d_in, d_hid, bias=bias), Linear(d_hid, d_in, bias=bias)
    comm = SimCommBackend(world)
    col, row = ColumnParallelLinear.from_dense(up, comm), RowParallelLinear.from_dense(down, comm)
    x = torch.randn(rows, d_in)
    xa, xb = x.clone().requires_grad_(), x.clone().requires_grad_()
    ya = down(torch.relu(up(xa)))
    yb = row(torch.relu(col(xb)))
    assert torch.allclose(ya, yb, atol=1e-5)
    ya.square().sum().backward()
    yb.square().sum().backward()
    assert torch.allclose(xa.grad, xb.grad, atol=1e-4)
    gw = torch.cat([p.grad for n, p in col.named_parameters() if n.endswith("weight")], dim=0)
    assert torch.allclose(gw, up.weight.grad, atol=1e-4)


@settings(**_SETTINGS)
@given(st.lists(st.integers(1, 4), min_size=1, max_size=3), st.sampled_from(["add", "sub", "mul", "div"]),
       st.integers(0, 2 ** 31 - 1))
def test_frontend_elementwise_ops_follow_numpy_and_their_gradients_sum_to_shape(shape, op, seed):
    """``tesseract.ops`` binary ops on fp32 tensors: values equal numpy's, a broadcast operand receives a gradient of
    its own shape (the sum over the broadcast axes), mismatched dtypes are refused."""
    import tesseract as ts
    rng = np.random.default_rng(seed)
    a_np = rng.standard_normal(shape).astype(np.float32)
    b_shape = [s if rng.integers(0, 2) else 1 for s in shape]
    b_np = (rng.standard_normal(b_shape) + 3.0).astype(np.float32)            # away from zero for div
    a, b = ts.Tensor(a_np), ts.Tensor(b_np)
    a.requires_grad = True
    b.requires_grad = True
    y = getattr(ts.ops, op)(a, b)
    want = {"add": a_np + b_np, "sub": a_np - b_np, "mul": a_np * b_np, "div": a_np / b_np}[op]
    assert y.shape == list(want.shape) and np.allclose(y.numpy(), want, rtol=1e-5, atol=1e-6)
    y.t.sum().backward()
    assert a.grad().shape == list(a_np.shape) and b.grad().shape == list(b_np.shape)
    if op == "add":
        assert np.allclose(b.grad().numpy(), np.full(b_shape, a_np.size / b_np.size, dtype=np.float32))
    with pytest.raises(TypeError):
        getattr(ts.ops, op)(a, ts.Tensor(b_np.astype(np.float64)))


@settings(**_SETTINGS)
@given(st.integers(1, 300), st.sampled_from([128, 256, 384]), st.booleans(), st.integers(-6, 4), st.integers(0, 2 ** 31 - 1))
def test_block_scaled_weight_quantisation_bounds(N, K, pow2, decade, seed):
    """128 x 128 block scales of an E4M3 weight: positive, powers of two when asked (never smaller than the exact
    scale, less than twice it), zero blocks get scale 1, dequantised weights within one E4M3 step of the input, and the
    scale atoms of the MX GEMM carry the exponent byte of every block."""
    from tesseract_b200.ops import fp8
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(N, K, generator=g) * (10.0 ** decade)
    if N > 130:
        w[:128, :128] = 0                                          # an all-zero block
    q, s = fp8.quantize_weight(w, pow2=pow2)
    q0, s0 = fp8.quantize_weight_ref(w)
    assert q.shape == (N, K) and q.dtype == torch.uint8 and s.shape == ((N + 127) // 128, K // 128)
    assert (s > 0).all()
    if pow2:
        assert fp8.scales_are_pow2(s) and (s >= s0 * (1 - 1e-6)).all() and (s < 2 * s0 * (1 + 1e-6)).all()
        atoms = fp8.weight_scale_atoms(s)
        assert atoms.shape == (s.shape[0], s.shape[1], 128)
        expo = (s.contiguous().view(torch.int32) >> 23) & 0xFF
        assert torch.equal(atoms[:, :, 0] & 0xFF, expo) and torch.equal((atoms[:, :, 77] >> 24) & 0xFF, expo)
    else:
        assert torch.allclose(s, s0)
    if N > 130:
        assert s[0, 0] == 1.0
    back = fp8.dequantize_weight(q, s)
    rows = torch.arange(N) // 128
    step = (s[rows].repeat_interleave(128, dim=1)[:, :K] * 32.0)         # the largest E4M3 step (at 448) is 32
    assert ((back - w).abs() <= step * 0.5 + 1e-30).all()


@settings(**_SETTINGS)
@given(st.integers(1, 3), st.integers(1, 5), st.sampled_from([(4, 4), (4, 2), (6, 1)]), st.sampled_from([2, 4]),
       st.booleans(), st.integers(0, 2 ** 31 - 1))
def test_paged_attention_oracle_equals_dense_attention_on_gathered_keys(A, S, heads, bs, int8, seed):
    """The paged-attention restatement (the oracle of the CUDA decode / prefill kernels) against plain softmax
    attention over each request's keys gathered in order: GQA head map, per-request lengths, the last new token seeing
    every key (bottom-right causal alignment), shuffled block tables, INT8 pools with per-token scales."""
    from tesseract_b200 import ops
    from tesseract_b200.nn.kv_cache import quantize_kv_per_token
    H, Hkv = heads
    D, max_blocks = 8, 5
    rng = np.random.default_rng(seed)
    g = torch.Generator().manual_seed(seed)
    nb = A * max_blocks + 2
    k_pool, v_pool = torch.randn(nb, Hkv, bs, D, generator=g), torch.randn(nb, Hkv, bs, D, generator=g)
    perm = rng.permutation(nb)[:A * max_blocks].reshape(A, max_blocks)
    tables = torch.from_numpy(perm.astype(np.int64))
    lens = torch.from_numpy(rng.integers(S, max_blocks * bs + 1, size=A).astype(np.int64))
    ks = vs = None
    kd, vd = k_pool, v_pool
    if int8:
        kq, ks = quantize_kv_per_token(k_pool)
        vq, vs = quantize_kv_per_token(v_pool)
        kd, vd = kq.float() * ks[..., None], vq.float() * vs[..., None]
        k_pool, v_pool = kq, vq
    q = torch.randn(A, S, H, D, generator=g)
    got = ops.paged_attention_ref(q, k_pool, v_pool, tables, lens, None, ks, vs)
    for a in range(A):
        L = int(lens[a])
        keys = torch.cat([kd[tables[a, i]] for i in range(max_blocks)], dim=1)[:, :L]      # [Hkv, L, D]
        vals = torch.cat([vd[tables[a, i]] for i in range(max_blocks)], dim=1)[:, :L]
        for h in range(H):
            kv = h // (H // Hkv)
            s = (q[a, :, h] @ keys[kv].t()) / D ** 0.5                                    # [S, L]
            i = torch.arange(S)[:, None] + (L - S)
            s = s.masked_fill(torch.arange(L)[None, :] > i, float("-inf"))
            want = torch.softmax(s, dim=-1) @ vals[kv]
            assert torch.allclose(got[a, :, h], want, atol=1e-5)
