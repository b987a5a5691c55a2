"""Native CPU FP32 GEMM of the host runtime against a float64 product (cf. the reference's CPU matmul cases,
tests/ops/test_matmul.cpp, and its thread-cap rule, src/ops/cpu/GemmAvx2.cpp:25-55)."""
import pytest
import torch

from tesseract_b200.ops import cpu_gemm


@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (5, 7, 3), (6, 16, 256), (7, 17, 257), (97, 2049, 33), (200, 130, 600)])
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_matmul_f32_matches_float64(M, N, K, b_is_nk):
    g = torch.Generator().manual_seed(M * 31 + N)
    a = torch.randn(M, K, generator=g)
    b = torch.randn(K, N, generator=g)
    want = (a.double() @ b.double()).float()
    got = cpu_gemm.matmul_f32(a, b.t().contiguous() if b_is_nk else b, b_is_nk=b_is_nk)
    assert got.shape == (M, N)
    assert (got - want).abs().max() <= 2e-5 * max(1.0, float(want.abs().max())) * max(1, K // 64)


def test_random_shapes_thread_counts_and_both_register_tiles():
    """Edge tiles, both B layouts, every thread count, and the AVX2 tile next to the AVX-512 one (a child process:
    the tile is chosen once per process)."""
    import subprocess
    import sys
    code = """
import numpy as np
from tesseract_b200 import _native
h = _native.host()
rng = np.random.default_rng(0)
for t in range(120):
    M, N, K = [int(rng.integers(1, 200)) for _ in range(3)]
    if t % 10 == 0:
        M, N, K = int(rng.integers(200, 500)), int(rng.integers(1, 2300)), int(rng.integers(150, 450))
    a = rng.standard_normal((M, K)).astype(np.float32)
    nk = bool(rng.integers(0, 2))
    b = rng.standard_normal((N, K) if nk else (K, N)).astype(np.float32)
    got = np.asarray(h.gemm_f32(a, b, nk, int(rng.integers(0, 9))))
    ref = a @ (b.T if nk else b)
    assert got.shape == ref.shape and np.allclose(got, ref, atol=2e-3, rtol=1e-4), (M, N, K, nk)
print("ok")
"""
    if cpu_gemm._host() is None:
        pytest.skip("native host runtime not built")
    import os
    for no512 in ("0", "1"):
        env = dict(os.environ, TESSERACT_GEMM_NO_AVX512=no512)
        out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300,
                             cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        assert out.returncode == 0 and "ok" in out.stdout, out.stderr[-2000:]


def test_thread_count_grows_with_work_and_respects_the_cap(monkeypatch):
    assert cpu_gemm.gemm_num_threads(8, 8, 8) == 1                      # tiny problems stay on one thread
    big = cpu_gemm.gemm_num_threads(2048, 2048, 2048)
    assert big >= 1
    monkeypatch.setenv("TESSERACT_GEMM_MAX_THREADS", "1")
    assert cpu_gemm.gemm_num_threads(2048, 2048, 2048) == 1
    monkeypatch.setenv("TESSERACT_GEMM_MAX_THREADS", "2")
    assert cpu_gemm.gemm_num_threads(2048, 2048, 2048, requested=1) == 1
    a = torch.randn(64, 64)
    assert torch.allclose(cpu_gemm.matmul_f32(a, a, threads=1), a @ a, atol=1e-4)


def test_python_twin_and_errors(monkeypatch):
    monkeypatch.setenv("TESSERACT_HOST", "python")
    a, b = torch.randn(9, 5), torch.randn(5, 4)
    assert torch.allclose(cpu_gemm.matmul_f32(a, b), a @ b, atol=1e-6)
    with pytest.raises(ValueError):
        cpu_gemm.matmul_f32(a, torch.randn(6, 4))


def test_frontend_matmul_routes_to_the_native_gemm_with_autograd(monkeypatch):
    """TESSERACT_CPU_GEMM=native: ``tesseract.ops.matmul`` of 2-D fp32 CPU tensors runs the host runtime's GEMM in the
    forward pass and in both backward products; values and gradients equal the library path."""
    import numpy as np
    import tesseract as ts
    if cpu_gemm._host() is None:
        pytest.skip("native host runtime not built")
    rng = np.random.default_rng(5)
    a_np, b_np = rng.standard_normal((37, 50)).astype(np.float32), rng.standard_normal((50, 23)).astype(np.float32)
    results = {}
    for mode in ("torch", "native"):
        monkeypatch.setenv("TESSERACT_CPU_GEMM", mode)
        assert cpu_gemm.native_selected() == (mode == "native")
        results[mode] = ts.ops.matmul(ts.Tensor(a_np.copy()), ts.Tensor(b_np.copy())).numpy().copy()
    assert np.allclose(results["torch"], results["native"], atol=1e-4)
    # gradients: same upstream gradient through both paths
    g = torch.randn(37, 23)
    grads = {}
    for mode in ("torch", "native"):
        monkeypatch.setenv("TESSERACT_CPU_GEMM", mode)
        a, b = ts.Tensor(a_np.copy()), ts.Tensor(b_np.copy())
        a.requires_grad = True
        b.requires_grad = True
        ts.ops.matmul(a, b).t.backward(g)
        grads[mode] = (a.grad().numpy().copy(), b.grad().numpy().copy())
    assert np.allclose(grads["torch"][0], grads["native"][0], atol=1e-4)
    assert np.allclose(grads["torch"][1], grads["native"][1], atol=1e-4)
