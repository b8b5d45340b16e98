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
    # weight copies are cached in fixed buffers and refreshed in place after an optimizer step
    k0 = {k: (v[1][0], v[1][0].clone()) for k, v in lin._w.items()}
    lin.fwd(x, w)
    assert all(lin._w[k][1][0] is k0[k][0] for k in k0)
    w.mul_(2.0)
    lin.refresh()
    assert all(lin._w[k][1][0] is k0[k][0] for k in k0)
    y2 = lin.fwd(x, w, 0.5)
    assert (y2.float() - 2 * ref).abs().max() <= 0.06 * 2 * ref.abs().max()


def test_engine_trains_with_mxfp8_linears_on_cpu():
    """`parallel.fp8 = "mxfp8"` routes the layer GEMMs through the MXFP8 products (format statement on CPU) and keeps training."""
    import math

    import forge_train_harness_b200 as fth
    cfg = fth.RunConfig(model=fth.preset("tiny"), optim=fth.OptimConfig(lr=3e-3, lr_schedule="constant"),
                        parallel=fth.ParallelConfig(fp8="mxfp8"),
                        train=fth.TrainConfig(num_steps=5, micro_batch_size=2, grad_accum_steps=1, seed=0, dtype="bf16", cuda_graph=False),
                        data=fth.DataConfig(prefetch_size=0))
    cfg = cfg.replace(model={"seq_length": 64, "padded_vocab_size": 264})
    tr = fth.Trainer(cfg, device="cpu", quiet=True)
    assert tr.ops.name.endswith("+mxfp8")
    losses = [float(tr.train_step()["loss"]) for _ in range(5)]
    assert tr.ops.mx_calls >= 5 * 2 * 4 * 3 - 8   # 4 linears x 3 products per layer and step (first layer's input grad aside)
    assert all(math.isfinite(v) for v in losses) and losses[-1] < losses[0]
    # same run in bf16: the fp8 trajectory stays close
    tr2 = fth.Trainer(cfg.replace(parallel={"fp8": "off"}), device="cpu", quiet=True)
    ref = [float(tr2.train_step()["loss"]) for _ in range(5)]
    assert max(abs(a - b) / abs(b) for a, b in zip(losses, ref)) < 0.02
    tr.close()
    tr2.close()
