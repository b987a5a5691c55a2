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
_SETTINGS = dict(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])


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
