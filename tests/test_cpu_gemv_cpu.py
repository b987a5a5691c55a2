"""CPU W8A8 decode GEMV (mirrors the reference's tests/ops/test_gemv_vnni.cpp): exact against an integer
reference over shapes that straddle the 256 / 64-byte spans and the tail, native and Python paths alike, and within
quantisation error of the fp32 product."""
import pytest
import torch

from tesseract_b200.ops import cpu_gemv


def _int_ref(W, wscale, xq, xscale):
    acc = (W.to(torch.int64) * xq.to(torch.int64)[None, :]).sum(dim=1)
    return (torch.tensor(xscale, dtype=torch.float32) * wscale) * acc.float()


@pytest.mark.parametrize("mode", ["native", "python"])
def test_w8a8_matches_integer_reference_across_shapes(mode, monkeypatch):
    if mode == "python":
        monkeypatch.setenv("TESSERACT_HOST", "python")
        assert not cpu_gemv.gemv_vnni_supported()
    g = torch.Generator().manual_seed(7)
    for N, K in ((17, 64), (32, 128), (8, 200), (64, 256), (40, 511), (96, 513), (1, 2048), (129, 4096), (3, 7)):
        W = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
        wscale = torch.rand(N, generator=g) * 0.049 + 0.001
        x = torch.rand(K, generator=g) * 6.0 - 3.0
        rowsum = cpu_gemv.compute_row_sums(W)
        assert torch.equal(rowsum.long(), W.long().sum(1))
        xq, xscale = cpu_gemv.quantize_row_int8(x)
        assert xq.dtype == torch.int8 and int(xq.abs().max()) == 127 and abs(xscale - float(x.abs().max()) / 127) < 1e-7
        y = cpu_gemv.gemv_w8a8(W, wscale, rowsum, xq, xscale)
        ref = _int_ref(W, wscale, xq, xscale)
        assert torch.all((y - ref).abs() <= 1e-4 * (ref.abs() + 1e-3)), (N, K)
        if N >= 8:
            part = cpu_gemv.gemv_w8a8_range(W, wscale, rowsum, xq, xscale, 2, N - 3)
            assert torch.equal(part[2:N - 3], y[2:N - 3]) and float(part[:2].abs().sum() + part[N - 3:].abs().sum()) == 0.0
        no_sums = cpu_gemv.gemv_w8a8(W, wscale, None, xq, xscale)          # scalar path: same integers
        assert torch.all((no_sums - ref).abs() <= 1e-4 * (ref.abs() + 1e-3))


def test_native_and_python_paths_agree_bit_for_bit(monkeypatch):
    g = torch.Generator().manual_seed(3)
    W = torch.randint(-127, 128, (300, 1000), generator=g, dtype=torch.int8)
    wscale = torch.rand(300, generator=g) * 0.05 + 0.001
    x = torch.randn(1000, generator=g)
    xq_n, xs_n = cpu_gemv.quantize_row_int8(x)
    y_n = cpu_gemv.gemv_w8a8(W, wscale, cpu_gemv.compute_row_sums(W), xq_n, xs_n, threads=4)
    monkeypatch.setenv("TESSERACT_HOST", "python")
    xq_p, xs_p = cpu_gemv.quantize_row_int8(x)
    y_p = cpu_gemv.gemv_w8a8(W, wscale, cpu_gemv.compute_row_sums(W), xq_p, xs_p)
    assert torch.equal(xq_n, xq_p) and xs_n == xs_p and torch.allclose(y_n, y_p, rtol=1e-6, atol=0)


def test_w8a8_approximates_the_fp32_product_and_zero_vector():
    g = torch.Generator().manual_seed(11)
    N, K = 256, 1024
    Wf = torch.randn(N, K, generator=g) * 0.05
    wscale = Wf.abs().amax(1) / 127.0
    W = torch.round(Wf / wscale[:, None]).to(torch.int8)
    x = torch.randn(K, generator=g)
    xq, xscale = cpu_gemv.quantize_row_int8(x)
    y = cpu_gemv.gemv_w8a8(W, wscale, cpu_gemv.compute_row_sums(W), xq, xscale)
    ref = Wf.double() @ x.double()
    assert float(((y.double() - ref) ** 2).sum().sqrt() / (ref ** 2).sum().sqrt()) < 0.03
    zq, zs = cpu_gemv.quantize_row_int8(torch.zeros(64))
    assert zs == 0.0 and int(zq.abs().sum()) == 0
    with pytest.raises(ValueError):
        cpu_gemv.gemv_w8a8(W, wscale[:5], None, xq, xscale)


def test_zero_vector_quantises_to_zeros_with_scale_zero(monkeypatch):
    """The reference returns scale 0 for an all-zero activation (src/ops/cpu/GemvVnni.cpp:126-133)."""
    for host in ("native", "python"):
        monkeypatch.setenv("TESSERACT_HOST", host)
        q, scale = cpu_gemv.quantize_row_int8(torch.zeros(96))
        assert scale == 0.0 and int(q.abs().max()) == 0 and q.dtype == torch.int8
