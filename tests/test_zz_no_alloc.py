"""The allocation-free decode entry point, called through its exported C symbol.

Some users of the library (a serving loop with a frozen memory pool, a plugin inside a host application that
owns the allocator) cannot allocate device memory when they need decode attention, so
``tsb_paged_decode_static`` keeps its split-K partials in an array inside the library image. This test checks
that it returns what ``tsb_paged_decode`` returns with caller-owned scratch, twice in a row (the array is
shared and keeps the previous call's contents), that nothing is allocated by the calls, and that an over-sized
problem is refused instead of overrunning the array. It is collected last so that a run that stops at the
first failure has already executed every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sig(lib):
    P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn = lib.tsb_paged_decode_static
    fn.argtypes = [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P]
    fn.restype = I
    cap = lib.tsb_paged_decode_static_capacity_floats
    cap.argtypes, cap.restype = [], ctypes.c_longlong
    return fn, cap


def _problem(dev, A, H, Hkv, D, bs, lens, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    nb = sum((l + bs - 1) // bs for l in lens) + 2
    k_pool = torch.randn(nb, Hkv, bs, D, device=dev, generator=g).bfloat16()
    v_pool = torch.randn(nb, Hkv, bs, D, device=dev, generator=g).bfloat16()
    max_blocks = max((l + bs - 1) // bs for l in lens)
    tables = torch.zeros(A, max_blocks, dtype=torch.int32)
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(seed))
    nxt = 0
    for a, l in enumerate(lens):
        n = (l + bs - 1) // bs
        tables[a, :n] = perm[nxt:nxt + n].to(torch.int32)
        nxt += n
    q = torch.randn(A, H, D, device=dev, generator=g).bfloat16()
    return q, k_pool, v_pool, tables.to(dev), torch.tensor(lens, dtype=torch.int32, device=dev)


def test_static_scratch_decode_matches_regular_entry_point_twice():
    from tesseract_b200 import _native, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = ctypes.CDLL(str(_native.cuda_lib_path()))
    fn, cap = _sig(lib)
    assert cap() == 2 * 1024 * 1024
    stream = torch.cuda.current_stream(dev).cuda_stream
    A, H, Hkv, D, bs = 4, 8, 2, 128, 16
    for call, lens in enumerate(([900, 33, 2048, 512], [64, 1500, 7, 1999])):
        q, k_pool, v_pool, tables, lens_t = _problem(dev, A, H, Hkv, D, bs, lens, seed=call)
        ref = ops.paged_decode_attention(q, k_pool, v_pool, tables, lens_t, max_len_hint=tables.shape[1] * bs)
        out = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(dev)
        # the driver's view as well (torch's counter would miss a raw cudaMalloc inside the library); the first
        # call may still page in the kernels, so the strict comparison starts with the second one
        free_before = torch.cuda.mem_get_info(dev)[0]
        rc = fn(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), None, None, tables.data_ptr(), lens_t.data_ptr(),
                out.data_ptr(), A, H, Hkv, D, bs, k_pool.shape[0], tables.shape[1], 1.0 / D ** 0.5,
                tables.shape[1] * bs, 1, stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before
        if call > 0:
            assert torch.cuda.mem_get_info(dev)[0] >= free_before
        assert torch.isfinite(out.float()).all()
        # same kernels, same split count, same inputs: the two entry points agree to the last bit
        assert torch.equal(out, ref)
        oracle = ops.paged_attention_ref(q.float().unsqueeze(1), k_pool, v_pool, tables, lens_t).squeeze(1)
        assert (out.float() - oracle).abs().max() < 2e-2


def test_static_scratch_decode_large_batch_fits_or_is_refused_cleanly():
    """A big batch either runs (and agrees with the regular entry point) or is refused with the documented
    code before anything is launched; it never overruns the built-in array."""
    from tesseract_b200 import _native, ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    lib = ctypes.CDLL(str(_native.cuda_lib_path()))
    fn, cap = _sig(lib)
    A, H, Hkv, D, bs = 96, 32, 8, 128, 16
    lens = [600 + 13 * i for i in range(A)]
    q, k_pool, v_pool, tables, lens_t = _problem(dev, A, H, Hkv, D, bs, lens, seed=9)
    out = torch.zeros_like(q)
    rc = fn(q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), None, None, tables.data_ptr(), lens_t.data_ptr(),
            out.data_ptr(), A, H, Hkv, D, bs, k_pool.shape[0], tables.shape[1], 1.0 / D ** 0.5,
            tables.shape[1] * bs, 1, torch.cuda.current_stream(dev).cuda_stream)
    torch.cuda.synchronize()
    assert rc in (0, -4)
    if rc == -4:
        assert float(out.abs().max()) == 0.0
    else:
        ref = ops.paged_decode_attention(q, k_pool, v_pool, tables, lens_t, max_len_hint=tables.shape[1] * bs)
        assert torch.equal(out, ref)


def test_static_scratch_need_is_below_capacity_and_refusal_rule_is_the_documented_one():
    """The host-only planning hook: what a problem needs, against what the built-in array holds. On a B200 the
    split plan never asks for more than the array has (so the refusal is a guard, not a path callers meet); a
    single key split needs nothing."""
    from tesseract_b200 import _native
    torch.cuda.set_device(0)
    lib = ctypes.CDLL(str(_native.cuda_lib_path()))
    need = lib.tsb_paged_decode_static_need_floats
    need.argtypes, need.restype = [ctypes.c_int] * 6, ctypes.c_longlong
    cap = lib.tsb_paged_decode_static_capacity_floats
    cap.restype = ctypes.c_longlong
    assert need(0, 32, 8, 128, 1024, 0) == -2
    worst = 0
    for A in (1, 4, 32, 96, 256, 1024):
        for H, Hkv in ((32, 8), (8, 2), (64, 8)):
            for max_len in (16, 512, 4096, 131072):
                for i8 in (0, 1):
                    n = need(A, H, Hkv, 128, max_len, i8)
                    assert n >= 0
                    worst = max(worst, n)
    assert need(1024, 32, 8, 128, 16, 0) == 0                  # short contexts: one split, no scratch
    assert 0 < worst <= cap()
