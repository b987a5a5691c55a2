"""MX (power-of-two block-scaled E4M3) quantisers and their layouts, torch restatement on CPU."""
import torch

from tesseract_b200.ops import fp8


def test_activation_quantiser_words_atoms_and_round_trip():
    g = torch.Generator().manual_seed(0)
    x = (torch.randn(200, 384, generator=g) * torch.exp(torch.randn(200, 1, generator=g))).bfloat16()
    x[3, 32:64] = 0
    q, sf = fp8.quantize_act_mx(x)
    assert q.shape == (200, 384) and sf.shape == (3, 256) and sf.dtype == torch.int32
    # every exponent is the smallest one that keeps its block inside +-448
    e = torch.stack([(sf[:, :200].t().to(torch.int64) >> (8 * j)) & 0xFF for j in range(4)], dim=2).reshape(200, 12)
    amax = x.float().abs().view(200, 12, 32).amax(dim=2)
    scale = torch.exp2(e.float() - 127)
    assert (amax <= 448 * scale).all() and ((amax > 224 * scale) | (amax == 0)).all()
    assert int(e[3, 1]) == 127 and (sf[:, 200:] == 0x7F7F7F7F).all()
    back = fp8.dequantize_act_mx(q, sf)
    assert ((back - x.float()).abs() <= x.float().abs() * 2 ** -4 + amax.repeat_interleave(32, dim=1) * 2 ** -9).all()
    # the atom layout holds the same words: word (m % 32) * 4 + (m % 128) / 32 of atom (m / 128, k / 128)
    qa, atoms = fp8.quantize_act_mx(x, atoms=True)
    assert torch.equal(qa, q) and atoms.shape == (2, 3, 128)
    for m, kb in [(0, 0), (37, 2), (130, 1), (199, 2)]:
        assert int(atoms[m // 128, kb, (m % 32) * 4 + (m % 128) // 32]) == int(sf[kb, m])
    assert torch.equal(fp8._atoms_to_words(atoms), sf) and torch.equal(fp8._words_to_atoms(sf), atoms)
    assert torch.equal(fp8.dequantize_act_mx(qa, atoms), back)


def test_power_of_two_weight_scales_and_mx_linear_restatement():
    g = torch.Generator().manual_seed(1)
    w = torch.randn(300, 256, generator=g) * 0.05
    wq, ws = fp8.quantize_weight(w, pow2=True)
    assert fp8.scales_are_pow2(ws) and not fp8.scales_are_pow2(fp8.quantize_weight(w)[1])
    wd = fp8.dequantize_weight(wq, ws)
    assert ((wd - w).norm() / w.norm()).item() < 0.04
    atoms = fp8.weight_scale_atoms(ws)
    assert atoms.shape == (3, 2, 128)
    expo = (ws.view(torch.int32) >> 23) & 0xFF
    assert ((atoms[:, :, 0].to(torch.int64) & 0xFF) == expo).all() and (atoms == atoms[:, :, :1]).all()
    x = torch.randn(40, 256, generator=g).bfloat16()
    for layout in (False, True):
        q, sf = fp8.quantize_act_mx(x, atoms=layout)
        y = fp8.mx_linear(q, sf, wq, ws)
        full = x.float() @ w.t()
        assert y.dtype == torch.bfloat16 and ((y.float() - full).norm() / full.norm()).item() < 0.06


def test_mx_linear_layer_small_and_large_batches():
    g = torch.Generator().manual_seed(2)
    lin = torch.nn.Linear(256, 96, bias=True)
    layer = fp8.MxLinear.from_linear(lin)
    for rows in (5, 300):
        x = torch.randn(rows, 256, generator=g)
        y, want = layer(x), lin(x)
        assert y.shape == want.shape and ((y - want).norm() / want.norm()).item() < 0.06
