"""sm_100a kernels vs the plain-PyTorch fp32 reference of the same op (small and ragged shapes)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from forge_train_harness_b200.ops.cuda_ops import Sm100Ops, check_status
    yield Sm100Ops
    torch.cuda.synchronize()
    check_status()


from forge_train_harness_b200.ops.torch_ops import TorchOps as T, rope_table  # noqa: E402


def rnd(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(dtype)


def close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert err <= atol + rtol * ref, f"max err {err} vs ref max {ref}"


@pytest.mark.parametrize("M,H", [(64, 1024), (37, 4096), (16, 256), (130, 1536), (9, 64)])
def test_rmsnorm(ops, M, H):
    x, a, w = rnd(M, H), rnd(M, H), rnd(H, scale=0.3) + 1
    y, rstd = ops.rmsnorm_fwd(x, w, 1e-6, 0.25)
    y0, rstd0 = T.rmsnorm_fwd(x.float(), w.float(), 1e-6, 0.25)
    close(y, y0)
    close(rstd, rstd0, 1e-3, 1e-4)
    r, y, rstd = ops.residual_rmsnorm_fwd(x, a, 0.3, w, 1e-6)
    r0, y0, _ = T.residual_rmsnorm_fwd(x, a, 0.3, w, 1e-6)
    close(r, r0, 1e-2, 1e-2)
    close(y, y0)
    dy, dres = rnd(M, H), rnd(M, H)
    g = torch.zeros(H, device="cuda") + 1.5
    g0 = g.clone()
    dx = ops.rmsnorm_bwd(dy, x, w, rstd0.contiguous(), g, dres, 0.5)
    dx0 = T.rmsnorm_bwd(dy.float(), x.float(), w.float(), rstd0, g0, dres.float(), 0.5)
    close(dx, dx0)
    close(g, g0, 1e-3, 1e-2)
    close(ops.residual_add(x, a, 0.7), T.residual_add(x, a, 0.7))


@pytest.mark.parametrize("nkv,g,d,S,B", [(2, 8, 64, 128, 2), (1, 4, 128, 64, 3)])
def test_rope(ops, nkv, g, d, S, B):
    tab = rope_table(S, d, 10000.0, "cuda")
    q = rnd(B * S, nkv * (g + 2) * d)
    q0 = T.rope_fwd_(q.clone().float(), tab, S, nkv, g, d)
    ops.rope_fwd_(q, tab, S, nkv, g, d)
    close(q, q0)
    ops.rope_bwd_(q, tab, S, nkv, g, d)
    T.rope_bwd_(q0, tab, S, nkv, g, d)
    close(q, q0)


def test_swiglu(ops):
    gu, d = rnd(100, 2 * 512), rnd(100, 512)
    close(ops.swiglu_fwd(gu), T.swiglu_fwd(gu.float()))
    close(ops.swiglu_bwd(d, gu), T.swiglu_bwd(d.float(), gu.float()))


def test_embedding(ops):
    V, H, M = 1000, 256, 333
    w = rnd(V, H)
    ids = torch.randint(0, V, (M,), device="cuda", dtype=torch.int32)
    close(ops.embedding_fwd(ids, w, 12.0), T.embedding_fwd(ids, w, 12.0))
    close(ops.embedding_fwd(ids, w[100:600].contiguous(), 12.0, 100, True), T.embedding_fwd(ids, w[100:600], 12.0, 100, True))
    dout = rnd(M, H)
    g, g0 = torch.zeros(500, H, device="cuda"), torch.zeros(500, H, device="cuda")
    ops.embedding_bwd(dout, ids, g, 12.0, 100)
    T.embedding_bwd(dout, ids, g0, 12.0, 100)
    close(g, g0, 1e-3, 1e-3)


@pytest.mark.parametrize("M,V", [(50, 73448), (33, 512), (20, 151936)])
def test_cross_entropy(ops, M, V):
    logits = rnd(M, V, scale=3.0)
    labels = torch.randint(0, V, (M,), device="cuda", dtype=torch.int32)
    mask = (torch.rand(M, device="cuda") > 0.2).float()
    l0 = logits.clone().float()
    nll0 = T.cross_entropy_fwd_bwd(l0, labels, mask, 0.3)
    nll = ops.cross_entropy_fwd_bwd(logits, labels, mask, 0.3)
    close(nll, nll0, 1e-3, 2e-2)
    err = (logits.float() - l0).abs().max().item()
    assert err < 4e-3, err


def test_ragged_vocab_shard_head(ops):
    """A vocabulary shard whose width is not a multiple of 8 (73448 / 4 = 18362): row-padded logits through the head GEMM,
    the fused cross-entropy statistics / gradient and the two backward GEMMs."""
    M, H, V = 384, 256, 18362
    x, w = rnd(M, H), rnd(V, H, scale=0.05)
    labels = torch.randint(-V, 2 * V, (M,), device="cuda", dtype=torch.int32)   # some targets live on other shards
    mask = (torch.rand(M, device="cuda") > 0.2).float()
    logits = ops.linear_fwd(x, w, 0.5)
    assert logits.shape == (M, V) and logits.stride(0) % 8 == 0
    ref = 0.5 * (x.float() @ w.float().t())
    close(logits.float(), ref, 2e-2, 2e-2)
    from forge_train_harness_b200.ops.cuda_ops import _C
    mx, sm, tg = _C.ce_stats(logits, labels, mask, 0)
    lf = logits.float()
    close(mx, lf.max(dim=1).values, 1e-6, 1e-6)
    close(sm, torch.exp(lf - mx[:, None]).sum(dim=1), 1e-3, 1e-3)
    has = (labels >= 0) & (labels < V)
    tg0 = torch.where(has, lf.gather(1, labels.clamp(0, V - 1).long()[:, None])[:, 0], torch.zeros_like(mx))
    close(tg, tg0, 1e-6, 1e-6)
    lse = mx + torch.log(sm)
    g0 = torch.exp(lf - lse[:, None])
    g0[has, labels[has].long()] -= 1.0
    g0 = g0 * (mask * 0.3)[:, None]
    _C.ce_grad(logits, labels, mask, lse, 0.3, 0)
    assert (logits.float() - g0).abs().max().item() < 4e-3
    # single-rank fused path on a padded view
    logits2 = ops.linear_fwd(x, w, 0.5)
    lab2 = labels.clamp(0, V - 1)
    l0 = logits2.float().clone()
    nll0 = T.cross_entropy_fwd_bwd(l0, lab2, mask, 0.3)
    nll = ops.cross_entropy_fwd_bwd(logits2, lab2, mask, 0.3)
    close(nll, nll0, 1e-3, 2e-2)
    assert (logits2.float() - l0).abs().max().item() < 4e-3
    # backward GEMMs read the padded view through its row stride
    dx = ops.linear_dgrad(logits2, w, 2.0)
    close(dx.float(), 2.0 * (logits2.float() @ w.float()), 2e-2, 2e-2)
    gw = torch.zeros(V, H, device="cuda")
    ops.linear_wgrad(logits2, x, gw, 2.0)
    close(gw, 2.0 * (logits2.float().t() @ x.float()), 2e-2, 2e-2)


def test_adamw_and_sumsq(ops):
    n = 50000
    master = torch.randn(n, device="cuda")
    m, v = torch.randn(n, device="cuda") * 0.1, torch.rand(n, device="cuda") * 0.01
    grad = torch.randn(2 * n, device="cuda")
    param = torch.zeros(2 * n, device="cuda", dtype=torch.bfloat16)
    segs = [(0, 256, 20000, 0.25, True), (20000, 30000 + 256, 29999, 1.0, False)]
    ref = [t.clone() for t in (master, m, v)]
    pref = torch.zeros(2 * n, device="cuda", dtype=torch.bfloat16)
    gs = torch.tensor(0.5, device="cuda")
    T.adamw_segments(*ref, grad, pref, segs, 1e-2, 0.9, 0.95, 1e-8, 0.1, 3, gs)
    ops.adamw_segments(master, m, v, grad, param, segs, 1e-2, 0.9, 0.95, 1e-8, 0.1, 3, gs)
    close(master, ref[0], 1e-5, 1e-5)
    close(m, ref[1], 1e-5, 1e-5)
    close(v, ref[2], 1e-5, 1e-6)
    assert torch.equal(param, pref) or (param.float() - pref.float()).abs().max() < 1e-2
    x = torch.randn(1234567, device="cuda")
    close(ops.sumsq(x), T.sumsq(x), 1e-5, 1e-3)


GEMM_SHAPES = [(128, 256, 64), (256, 512, 128), (384, 1280, 1024), (200, 264, 72), (4096, 1024, 4096), (130, 9184, 320), (300, 200, 136)]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("bn", [128, 256, -128, -256, 0])  # one-CTA tiles, CTA-pair (cta_group::2) tiles, automatic choice
def test_gemm_variants(ops, M, N, K, bn):
    from forge_train_harness_b200.ops.cuda_ops import _C, check_status
    K8 = (K + 7) // 8 * 8
    x, w = rnd(M, K8, scale=0.5), rnd(N, K8, scale=0.5)
    y = _C.gemm(x, False, w, False, None, 0.5, 0, bn, 0)
    torch.cuda.synchronize()
    check_status()
    close(y, 0.5 * (x.float() @ w.float().t()), 1e-2, 1e-2 * math.sqrt(K8) * 0.25)
    if N % 8 == 0 and M % 8 == 0:
        dy = rnd(M, N, scale=0.5)
        dx = _C.gemm(dy, False, w, True, None, 1.0, 0, bn, 0)
        close(dx, dy.float() @ w.float(), 1e-2, 1e-2 * math.sqrt(N) * 0.25)
        g = torch.ones(N, K8, device="cuda")
        _C.gemm(dy, True, x, True, g, 2.0, 1, bn, 0)
        close(g, 1.0 + 2.0 * (dy.float().t() @ x.float()), 1e-2, 1e-2 * math.sqrt(M) * 0.25)
        torch.cuda.synchronize()
        check_status()


@pytest.mark.parametrize("B,S,nkv,g,d", [(1, 128, 1, 1, 64), (2, 256, 2, 2, 64), (1, 384, 1, 2, 128), (2, 512, 2, 8, 64), (1, 1024, 1, 4, 128)])
def test_flash_fwd(ops, B, S, nkv, g, d):
    from forge_train_harness_b200.ops.cuda_ops import check_status
    qkv = rnd(B * S, nkv * (g + 2) * d, scale=1.0)
    out, lse = ops.attention_fwd(qkv, S, nkv, g, d)
    torch.cuda.synchronize()
    check_status()
    out0, lse0 = T.attention_fwd(qkv.float(), S, nkv, g, d)
    close(lse, lse0, 1e-3, 2e-2)
    close(out, out0, 2e-2, 2e-2)


@pytest.mark.parametrize("B,S,nkv,g,d", [(1, 128, 1, 1, 64), (2, 256, 2, 2, 64), (1, 384, 1, 2, 128), (2, 512, 2, 8, 64), (1, 1024, 1, 4, 128)])
def test_flash_bwd(ops, B, S, nkv, g, d):
    from forge_train_harness_b200.ops.cuda_ops import check_status
    qkv = rnd(B * S, nkv * (g + 2) * d, scale=1.0)
    out, lse = ops.attention_fwd(qkv, S, nkv, g, d)
    dout = rnd(B * S, nkv * g * d, scale=1.0)
    dqkv = ops.attention_bwd(dout, qkv, out, lse, S, nkv, g, d)
    torch.cuda.synchronize()
    check_status()
    out0, lse0 = T.attention_fwd(qkv.float(), S, nkv, g, d)
    dqkv0 = T.attention_bwd(dout.float(), qkv.float(), out0, lse0, S, nkv, g, d)
    v = dqkv.view(B * S, nkv, g + 2, d).float()
    v0 = dqkv0.view(B * S, nkv, g + 2, d)
    close(v[:, :, :g], v0[:, :, :g], 3e-2, 3e-2)       # dQ
    close(v[:, :, g], v0[:, :, g], 3e-2, 3e-2)         # dK
    close(v[:, :, g + 1], v0[:, :, g + 1], 3e-2, 3e-2)  # dV
    tab = rope_table(S, d, 10000.0, "cuda")
    fused = ops.attention_rope_bwd(dout, qkv, out, lse, tab, S, nkv, g, d)
    close(fused, T.rope_bwd_(dqkv0.clone(), tab, S, nkv, g, d), 3e-2, 3e-2)


def test_gemm_repeated_calls_and_views(ops):
    """Operands that are strided row views (unit inner stride) and repeated in-place updates."""
    big = rnd(512, 2048, scale=0.5)
    x = big[:, 256:256 + 512]
    w = rnd(384, 512, scale=0.5)
    for _ in range(3):
        y = ops.linear_fwd(x, w)
        close(y, x.float() @ w.float().t(), 1e-2, 0.1)
        w.mul_(0.9)


# ---- MXFP8 ----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("R,C", [(128, 128), (256, 1024), (200, 160), (4096, 4096), (96, 320), (33, 32), (64, 584)])
@pytest.mark.parametrize("colwise", [False, True])
def test_mxfp8_quant_matches_format_statement(ops, R, C, colwise):
    if not colwise and C % 32:
        C = (C + 31) // 32 * 32          # row orientation: blocks of 32 along the columns
    from forge_train_harness_b200.ops import mxfp8 as mx
    if colwise and R % 32:
        R = (R + 31) // 32 * 32
    x = rnd(R, C, scale=2.0)
    x[3, :] = 0
    q, sf = mx.quantize(x, colwise)
    q0, sf0 = mx.quantize_ref(x, colwise)
    assert q.shape == q0.shape and torch.equal(sf.cpu(), sf0.cpu())
    assert torch.equal(q.cpu(), q0.cpu())
    # a strided source (a column slice of a wider tensor) gives the same bits
    wide = torch.zeros(R, C + 64, device="cuda", dtype=torch.bfloat16)
    wide[:, 32:32 + C] = x
    q2, sf2 = mx.quantize(wide[:, 32:32 + C], colwise)
    assert torch.equal(q2, q) and torch.equal(sf2, sf)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (200, 264, 160), (1024, 4096, 4096), (130, 96, 32)])
def test_mxfp8_gemm_matches_dequantised_matmul(ops, M, N, K):
    from forge_train_harness_b200.ops import mxfp8 as mx
    a, b = rnd(M, K), rnd(N, K, scale=0.3)
    aq, asf = mx.quantize(a)
    bq, bsf = mx.quantize(b)
    ref = mx.dequantize_ref(aq, asf) @ mx.dequantize_ref(bq, bsf).t()
    y = mx.gemm(aq, asf, bq, bsf, None, 0.5, 0)
    close(y.float(), 0.5 * ref, 1e-2, 1e-2)
    y32 = mx.gemm(aq, asf, bq, bsf, None, 1.0, 2)
    close(y32, ref, 1e-4, 1e-3)
    acc = torch.ones(M, N, device="cuda")
    mx.gemm(aq, asf, bq, bsf, acc, 2.0, 1)
    close(acc, 1.0 + 2.0 * ref, 1e-4, 1e-3)


def test_mxfp8_linear_products_close_to_bf16(ops):
    from forge_train_harness_b200.ops import mxfp8 as mx
    M, N, K = 512, 768, 1024
    x, w, dy = rnd(M, K, scale=0.5), rnd(N, K, scale=0.05), rnd(M, N)
    lin = mx.Mxfp8Linear()
    ref = x.float() @ w.float().t()
    assert (lin.fwd(x, w).float() - ref).abs().max() <= 0.05 * ref.abs().max()
    refd = dy.float() @ w.float()
    assert (lin.dgrad(dy, w).float() - refd).abs().max() <= 0.05 * refd.abs().max()
    g = torch.zeros(N, K, device="cuda")
    lin.wgrad(dy, x, g)
    refw = dy.float().t() @ x.float()
    assert (g - refw).abs().max() <= 0.05 * refw.abs().max()


def test_bounded_peer_wait_runs_out_and_reports_status(ops):
    """Failure detection on the device side: a flag wait whose peer never arrives gives up after its limit, the kernel
    returns, the host reads the status code, and the context keeps working (no trap, no endless spin)."""
    from forge_train_harness_b200.ops.cuda_ops import _C, check_status
    _C.read_status(True)
    pads = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(2)]
    # rank 0 of a 2-rank barrier whose rank 1 does not exist: slot 1 of the own pad is never written
    _C.peer_barrier([p.data_ptr() for p in pads], 0, 1, 0, 0.05, None)
    torch.cuda.synchronize()
    assert int(pads[1][0]) == 1 and int(pads[0][0]) == 1      # the release stores went out
    with pytest.raises(RuntimeError, match="peer flag never set"):
        check_status()
    check_status()                                             # the read cleared it
    # the same barrier completes once the missing flag is there, and ordinary kernels still run
    pads[0][1] = 2
    _C.peer_barrier([p.data_ptr() for p in pads], 0, 2, 0, 0.05, None)
    x, w = rnd(64, 256), rnd(256)
    y, _ = ops.rmsnorm_fwd(x, w, 1e-6)
    torch.cuda.synchronize()
    check_status()
    assert torch.isfinite(y.float()).all()


def test_debug_input_check_reports_a_bad_id_through_the_status_word(ops):
    """An id outside the vocabulary is recorded (status 7 + first bad position) without touching memory; in-range ids, and an
    id that is merely outside the LOCAL shard range, are not errors; the context keeps working."""
    from forge_train_harness_b200.ops.cuda_ops import _C, Sm100Ops, check_status
    _C.read_status(True)
    Sm100Ops.bad_index_position()
    ids = torch.randint(0, 1000, (4096,), device="cuda", dtype=torch.int32)
    Sm100Ops.check_ids(ids, 0, 1000)
    torch.cuda.synchronize()
    check_status()
    assert Sm100Ops.bad_index_position() == -1
    ids[1234] = 1000
    ids[3000] = -5
    Sm100Ops.check_ids(ids, 0, 1000)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="outside its valid range"):
        check_status()
    assert Sm100Ops.bad_index_position() == 1234 and Sm100Ops.bad_index_position() == -1   # first bad position; read resets
    # the kernels themselves stay safe on such input: the embedding writes zeros for it and reads nothing out of range
    w = rnd(1000, 256)
    e = ops.embedding_fwd(ids, w, 1.0, 0, False)
    torch.cuda.synchronize()
    check_status()
    assert float(e[1234].abs().max()) == 0.0 and float(e[3000].abs().max()) == 0.0 and torch.isfinite(e.float()).all()


@pytest.mark.parametrize("nkv,g,d,M", [(8, 2, 128, 1000), (2, 8, 64, 777), (1, 1, 64, 5)])
def test_qk_norm(ops, nkv, g, d, M):
    """Per-head q/k RMSNorm on the packed QKV layout (Qwen3 variant) against the fp32 PyTorch op: forward, rstd, backward in
    place, both weight gradients (accumulated), v heads untouched, and bitwise repeatable (no atomics)."""
    torch.manual_seed(0)
    qkv, dq = rnd(M, nkv * (g + 2) * d, scale=2.0), rnd(M, nkv * (g + 2) * d)
    wq, wk = (1.0 + 0.3 * torch.randn(d, device="cuda")).bfloat16(), (1.0 + 0.3 * torch.randn(d, device="cuda")).bfloat16()
    out, rstd = ops.qk_norm_fwd(qkv, wq, wk, 1e-6, nkv, g, d)
    ref_out, ref_rstd = T.qk_norm_fwd(qkv.float(), wq.float(), wk.float(), 1e-6, nkv, g, d)
    assert out.data_ptr() != qkv.data_ptr() and tuple(rstd.shape) == (M, nkv, g + 1)
    assert (rstd - ref_rstd).abs().max() <= 1e-5 * ref_rstd.abs().max()
    rel = (out.float() - ref_out).norm() / ref_out.norm()
    assert rel < 3e-3, float(rel)                                   # one bf16 rounding of the output
    v_in = qkv.view(M, nkv, g + 2, d)[:, :, g + 1]
    assert torch.equal(out.view(M, nkv, g + 2, d)[:, :, g + 1], v_in)  # v heads pass through bit for bit
    gq0, gk0 = torch.randn(d, device="cuda"), torch.randn(d, device="cuda")
    gq, gk = gq0.clone(), gk0.clone()
    rq, rk = gq0.clone(), gk0.clone()
    ref_dx = T.qk_norm_bwd(dq.float(), qkv.float(), ref_rstd, wq.float(), wk.float(), rq, rk, nkv, g, d)
    d_in = dq.clone()
    got = ops.qk_norm_bwd(d_in, qkv, rstd, wq, wk, gq, gk, nkv, g, d)
    assert got.data_ptr() == d_in.data_ptr()                        # in place
    rel = (got.float() - ref_dx).norm() / ref_dx.norm()
    assert rel < 3e-3, float(rel)
    assert torch.equal(got.view(M, nkv, g + 2, d)[:, :, g + 1], dq.view(M, nkv, g + 2, d)[:, :, g + 1])
    for a, b, start in ((gq, rq, gq0), (gk, rk, gk0)):
        assert ((a - start) - (b - start)).norm() <= 2e-3 * (b - start).norm() + 1e-4, float(((a - start) - (b - start)).norm())
    # run twice: identical bits
    d2, gq2, gk2 = dq.clone(), gq0.clone(), gk0.clone()
    ops.qk_norm_bwd(d2, qkv, rstd, wq, wk, gq2, gk2, nkv, g, d)
    out2, rstd2 = ops.qk_norm_fwd(qkv, wq, wk, 1e-6, nkv, g, d)
    assert torch.equal(d2, got) and torch.equal(gq2, gq) and torch.equal(gk2, gk) and torch.equal(out2, out) and torch.equal(rstd2, rstd)
