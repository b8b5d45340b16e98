"""MXFP8 format statement (CPU): scale rule, chunked scale layout, round trip error, and the three linear products."""
import torch

from forge_train_harness_b200.ops import mxfp8 as mx


def test_scale_is_smallest_power_of_two_that_fits_e4m3():
    x = torch.zeros(2, 64, dtype=torch.bfloat16)
    x[0, :32] = 448.0          # amax / 448 = 1 exactly -> 2^0
    x[0, 32:] = 449.0          # (bf16 rounds to 448) -> still 2^0
    x[1, 0] = 1000.0           # 1000 / 448 = 2.23 -> 2^2
    x[1, 32] = 3.0             # 3 / 448 = 0.0067 -> 2^-7
    q, sf = mx.quantize_ref(x)
    e = [int(sf[i]) for i in (0 * 16 + 0, 0 * 16 + 1, 1 * 16 + 0, 1 * 16 + 1)]
    assert e == [127, 127, 129, 120]
    d = mx.dequantize_ref(q, sf)
    assert d[1, 0] == 1000.0 or abs(float(d[1, 0]) - 1000.0) <= 32.0
    assert float(d[1, 32]) == 3.0


def test_all_zero_block_and_round_trip_error():
    torch.manual_seed(0)
    x = (torch.randn(200, 160) * 3).to(torch.bfloat16)
    x[5, 32:64] = 0
    q, sf = mx.quantize_ref(x)
    assert sf.numel() == mx.sf_bytes(200, 160) == 2 * 2 * 512
    d = mx.dequantize_ref(q, sf)
    assert torch.all(d[5, 32:64] == 0)
    blk_amax = x.float().view(200, 5, 32).abs().amax(dim=2, keepdim=True).expand(200, 5, 32).reshape(200, 160)
    # e4m3 has 3 mantissa bits: relative step 2^-3, half of it when rounding, measured against the block maximum
    assert ((d - x.float()).abs() <= blk_amax * 2.0 ** -4 + 1e-30).all()


def test_colwise_is_rowwise_of_the_transpose():
    torch.manual_seed(1)
    x = torch.randn(96, 40).to(torch.bfloat16)
    qc, sc = mx.quantize_ref(x, colwise=True)
    qr, sr = mx.quantize_ref(x.t().contiguous(), colwise=False)
    assert torch.equal(qc, qr) and torch.equal(sc, sr) and qc.shape == (40, 96)


def test_linear_products_close_to_exact():
    torch.manual_seed(2)
    M, N, K = 64, 96, 128
    x, w, dy = (torch.randn(M, K) * 0.5).to(torch.bfloat16), (torch.randn(N, K) * 0.1).to(torch.bfloat16), torch.randn(M, N).to(torch.bfloat16)
    lin = mx.Mxfp8Linear()
    y = lin.fwd(x, w, 0.5)
    ref = 0.5 * x.float() @ w.float().t()
    assert (y.float() - ref).abs().max() <= 0.06 * ref.abs().max()
    dx = lin.dgrad(dy, w)
    refd = dy.float() @ w.float()
    assert (dx.float() - refd).abs().max() <= 0.06 * refd.abs().max()
    g = torch.ones(N, K)
    lin.wgrad(dy, x, g, 2.0)
    refw = 1.0 + 2.0 * dy.float().t() @ x.float()
    assert (g - refw).abs().max() <= 0.06 * refw.abs().max()
    # weight copies are cached until the optimizer steps
    k0 = dict(lin._w)
    lin.fwd(x, w)
    assert all(lin._w[k] is k0[k] for k in k0)
    lin.invalidate()
    lin.fwd(x, w)
    assert any(lin._w[k] is not k0[k] for k in k0)
