"""Per-op contract for the sm_100a kernels, beyond a max-norm check (``test_ops_gpu.py``):

* error DISTRIBUTION against an fp64 oracle: mean, 95th percentile, maximum and the signed mean / magnitude bias;
* the shapes the flagship runs use (attention at 4096 tokens with 8 x 64 and 16 x 128 query heads per KV head, the LM-head
  GEMM at 16384 x 73448 x 1024 with its ragged width);
* canary-padded outputs: the output tensor is a view inside a sentinel-filled buffer, so a tile that is not clipped at a
  ragged edge is seen on the host;
* run-twice bitwise equality for every kernel without floating-point atomics, and for the deterministic mode of the ones
  that have them (embedding backward, split-K weight gradients);
* real strided views and repeated in-place calls.

The template is the reference's operator test contract (harness/tests/test_training_engine_backward.py:54-126 and
prompt/develop_prompt/_shared/stage2-subagent-playbook.md:63-93, 320-346).
"""
import json
import math
import os

import pytest
import torch

from tests._stats import assert_close_stats, err_stats, padded

pytestmark = pytest.mark.gpu

_STATS = {}


@pytest.fixture(scope="module")
def ops():
    from forge_train_harness_b200.ops.cuda_ops import Sm100Ops, check_status
    yield Sm100Ops
    torch.cuda.synchronize()
    check_status()
    Sm100Ops.set_deterministic(False)
    out = os.environ.get("FORGE_TEST_ARTIFACTS") or os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "test_artifacts")
    if os.path.isdir(out):  # keep the measured distributions next to the other run artefacts
        with open(os.path.join(out, "op_contract_stats.json"), "w") as f:
            json.dump(_STATS, f, indent=1)


from forge_train_harness_b200.ops.torch_ops import TorchOps as T, rope_table  # noqa: E402


def rnd(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(dtype)


def keep(name, s):
    _STATS[name] = {k: v for k, v in s.items()}


# bf16 rounding of an fp32-accurate result: |err| <= 2^-9 |x|; for a unit-variance tensor that is a mean of ~1.1e-3,
# a 95th percentile of ~3.5e-3 and a maximum of ~2e-2 (at 5 sigma) of the RMS.  Bounds leave a factor of two.
BF16 = dict(mean=2.5e-3, p95=8e-3, mx=4e-2, bias=1e-4)


# ---- GEMM -----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(1024, 1280, 1024), (2048, 1024, 4096), (300, 200, 136)])
def test_gemm_error_distribution_and_canary(ops, M, N, K):
    from forge_train_harness_b200.ops.cuda_ops import _C, check_status
    K8, N8 = (K + 7) // 8 * 8, (N + 7) // 8 * 8
    x, w = rnd(M, K8, scale=0.5), rnd(N8, K8, scale=0.5)
    ref = x.double() @ w.double().t()
    for bn in (0, 256, -256, -128):
        out, check = padded((M, N8), torch.bfloat16)
        _C.gemm(x, False, w, False, out, 1.0, 0, bn, 0)
        torch.cuda.synchronize()
        check_status()
        check()
        keep(f"gemm_fwd_{M}x{N}x{K}_bn{bn}", assert_close_stats(out, ref, what=f"gemm fwd bn={bn}", **BF16))
        again, _ = padded((M, N8), torch.bfloat16)
        _C.gemm(x, False, w, False, again, 1.0, 0, bn, 0)
        assert torch.equal(out, again), "forward GEMM is not run-to-run identical"
    if M % 8 == 0:
        dy = rnd(M, N8, scale=0.5)
        dx, check = padded((M, K8), torch.bfloat16)
        _C.gemm(dy, False, w, True, dx, 1.0, 0, 0, 0)
        check()
        keep(f"gemm_dgrad_{M}x{N}x{K}", assert_close_stats(dx, dy.double() @ w.double(), what="gemm dgrad", **BF16))
        g, check = padded((N8, K8), torch.float32)
        g.fill_(0.25)
        _C.gemm(dy, True, x, True, g, 2.0, 1, 0, 0)
        check()
        refw = 0.25 + 2.0 * (dy.double().t() @ x.double())
        keep(f"gemm_wgrad_{M}x{N}x{K}", assert_close_stats(g, refw, mean=2e-5, p95=6e-5, mx=4e-4, bias=2e-6, what="gemm wgrad"))


def test_gemm_lm_head_shape_ragged_width(ops):
    """16384 x 73448 x 1024: the widest product of the flagship, 73448 is not a multiple of the tile width."""
    M, N, K = 16384, 73448, 1024
    x, w = rnd(M, K, scale=0.5), rnd(N, K, scale=0.05)
    y = ops.linear_fwd(x, w, 0.25)
    assert y.shape == (M, N)
    worst = {"mean": 0.0, "p95": 0.0, "max": 0.0, "signed_mean": 0.0}
    for r0 in range(0, M, 4096):
        ref = 0.25 * (x[r0:r0 + 4096].double() @ w.double().t())
        s = assert_close_stats(y[r0:r0 + 4096], ref, what=f"lm head rows {r0}", **BF16)
        for k in worst:
            worst[k] = max(worst[k], abs(s[k]))
        del ref
    keep("gemm_fwd_lm_head_16384x73448x1024", worst)


def test_split_k_wgrad_is_bitwise_repeatable_in_deterministic_mode(ops):
    from forge_train_harness_b200.ops.cuda_ops import _C
    dy, x = rnd(8192, 640, scale=0.5), rnd(8192, 1024, scale=0.5)   # few output tiles: the library would split K
    ops.set_deterministic(True)
    try:
        a, b = torch.zeros(640, 1024, device="cuda"), torch.zeros(640, 1024, device="cuda")
        _C.gemm(dy, True, x, True, a, 1.0, 1, 0, 0)
        _C.gemm(dy, True, x, True, b, 1.0, 1, 0, 0)
        assert torch.equal(a, b)
        assert_close_stats(a, dy.double().t() @ x.double(), mean=2e-5, p95=6e-5, mx=4e-4, bias=2e-6, what="deterministic wgrad")
    finally:
        ops.set_deterministic(False)
    c = torch.zeros(640, 1024, device="cuda")
    _C.gemm(dy, True, x, True, c, 1.0, 1, 0, 0)   # split-K form: same numbers to fp32 summation-order accuracy
    assert_close_stats(c, a, mean=2e-5, p95=6e-5, mx=4e-4, bias=2e-6, what="split-K vs one split")


# ---- attention ---------------------------------------------------------------------------------------------------------
def _attn_ref64(qkv, dout, S, nkv, g, d):
    """fp64 causal GQA attention on the packed kv-group-major layout, with autograd for the gradients."""
    M = qkv.shape[0]
    B = M // S
    q = qkv.double().detach().clone().requires_grad_(True)
    v5 = q.view(B, S, nkv, g + 2, d)
    Q, K, V = v5[:, :, :, :g], v5[:, :, :, g], v5[:, :, :, g + 1]
    s = torch.einsum("bsngd,btnd->bngst", Q, K) / math.sqrt(d)
    mask = torch.ones(S, S, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.einsum("bngst,btnd->bsngd", torch.softmax(s, dim=-1), V).reshape(M, nkv * g * d)
    (dq,) = torch.autograd.grad(o, q, dout.double())
    return o.detach(), lse.detach(), dq


@pytest.mark.parametrize("S,nkv,g,d", [(4096, 2, 8, 64), (4096, 2, 16, 128), (1024, 1, 4, 128)])
def test_flash_attention_flagship_shapes(ops, S, nkv, g, d):
    from forge_train_harness_b200.ops.cuda_ops import check_status
    qkv = rnd(S, nkv * (g + 2) * d, scale=1.0)
    dout = rnd(S, nkv * g * d, scale=1.0)
    out, lse = ops.attention_fwd(qkv, S, nkv, g, d)
    out2, lse2 = ops.attention_fwd(qkv, S, nkv, g, d)
    dqkv = ops.attention_bwd(dout, qkv, out, lse, S, nkv, g, d)
    torch.cuda.synchronize()
    check_status()
    assert torch.equal(out, out2) and torch.equal(lse, lse2), "attention forward is not run-to-run identical"
    o64, lse64, dq64 = _attn_ref64(qkv, dout, S, nkv, g, d)
    tag = f"S{S}_g{g}_d{d}"
    keep(f"flash_fwd_{tag}", assert_close_stats(out, o64, mean=4e-3, p95=1.2e-2, mx=0.25, bias=2e-4, what="attention out"))
    # the kernel's log-sum-exp, [B, heads, S] in natural log
    assert float((lse.double().reshape(-1) - lse64.reshape(-1)).abs().max()) < 5e-3
    v, v0 = dqkv.double().view(S, nkv, g + 2, d), dq64.view(S, nkv, g + 2, d)
    # the first rows attend to a handful of keys and are O(1) while the tensor's RMS is ~0.07, so the largest error, taken
    # relative to the RMS, is a bf16 rounding of an O(1) value; mean and p95 are the tight bounds
    bw = dict(mean=8e-3, p95=2.5e-2, mx=0.5, bias=5e-4)
    keep(f"flash_bwd_dq_{tag}", assert_close_stats(v[:, :, :g], v0[:, :, :g], what="dQ", **bw))
    keep(f"flash_bwd_dk_{tag}", assert_close_stats(v[:, :, g], v0[:, :, g], what="dK", **bw))
    keep(f"flash_bwd_dv_{tag}", assert_close_stats(v[:, :, g + 1], v0[:, :, g + 1], what="dV", **bw))


def test_attention_refuses_unsupported_sequence_lengths_loudly(ops):
    qkv = rnd(200, (2 + 2) * 64)
    with pytest.raises(ValueError, match="multiple of 128"):
        ops.attention_fwd(qkv, 200, 1, 2, 64)


# ---- bandwidth-bound ops -----------------------------------------------------------------------------------------------
def test_rmsnorm_distribution_canary_and_repeatability(ops):
    M, H = 777, 1024
    x, a, w = rnd(M, H), rnd(M, H), rnd(H, scale=0.3) + 1
    # the destination must be contiguous (it is this rank's rows of an all-gather buffer): sentinels before and after it
    big = torch.full((M * H + 2048,), -777.0, device="cuda", dtype=torch.bfloat16)
    y_view = big[1024:1024 + M * H].view(M, H)
    r, y, rstd = ops.residual_rmsnorm_fwd(x, a, 0.3, w, 1e-6, y_out=y_view)
    assert bool((big[:1024] == -777.0).all()) and bool((big[1024 + M * H:] == -777.0).all()) and y.data_ptr() == y_view.data_ptr()
    rr = x.double() + a.double() * 0.3
    rr_b = rr.to(torch.bfloat16).double()
    rstd64 = torch.rsqrt(rr_b.pow(2).mean(-1) + 1e-6)
    keep("residual_add", assert_close_stats(r, rr, what="residual", **BF16))
    keep("rmsnorm_fwd", assert_close_stats(y, rr_b * rstd64[:, None] * w.double(), what="rmsnorm", **BF16))
    assert_close_stats(rstd, rstd64, mean=1e-6, p95=3e-6, mx=2e-5, bias=5e-7, what="rstd")
    r2, y2, rstd2 = ops.residual_rmsnorm_fwd(x, a, 0.3, w, 1e-6)
    assert torch.equal(y, y2) and torch.equal(r, r2) and torch.equal(rstd, rstd2)
    # backward: dx against the closed form in fp64; the weight gradient accumulates in place, call after call
    dy, dres = rnd(M, H), rnd(M, H)
    gw = torch.full((H,), 1.5, device="cuda")
    xb = r.double()
    xhat = xb * rstd64[:, None]
    gwt = dy.double() * w.double()
    dx64 = rstd64[:, None] * (gwt - xhat * (gwt * xhat).mean(-1, keepdim=True)) + dres.double()
    for rep in range(3):
        dx = ops.rmsnorm_bwd(dy, r, w, rstd64.float().contiguous(), gw, dres)
        keep("rmsnorm_bwd_dx", assert_close_stats(dx, dx64, what="rmsnorm dx", **BF16))
        assert_close_stats(gw, 1.5 + (rep + 1) * (dy.double() * xhat).sum(0), mean=1e-5, p95=3e-5, mx=2e-4, bias=2e-6,
                           what=f"rmsnorm dw after {rep + 1} calls")


def test_swiglu_rope_distribution_and_repeatability(ops):
    gu, d = rnd(1000, 2 * 2048), rnd(1000, 2048)
    g64, u64 = gu.double().chunk(2, -1)
    sig = torch.sigmoid(g64)
    out = ops.swiglu_fwd(gu)
    PROD = dict(BF16, mx=0.1)   # a product of two Gaussians has heavier tails: its largest entry is ~20 x the RMS
    keep("swiglu_fwd", assert_close_stats(out, g64 * sig * u64, what="swiglu", **PROD))
    assert torch.equal(out, ops.swiglu_fwd(gu))
    dgu = ops.swiglu_bwd(d, gu)
    dg = d.double() * u64 * (sig * (1 + g64 * (1 - sig)))
    du = d.double() * g64 * sig
    keep("swiglu_bwd", assert_close_stats(dgu, torch.cat([dg, du], -1), what="swiglu bwd", **PROD))
    assert torch.equal(dgu, ops.swiglu_bwd(d, gu))
    # RoPE in place on a packed QKV buffer that is a strided row view of a wider tensor's first columns
    S, nkv, g, hd = 512, 2, 8, 64
    tab = rope_table(S, hd, 10000.0, "cuda")
    q = rnd(2 * S, nkv * (g + 2) * hd)
    q0 = T.rope_fwd_(q.clone().double().float(), tab, S, nkv, g, hd)
    a, b = q.clone(), q.clone()
    ops.rope_fwd_(a, tab, S, nkv, g, hd)
    ops.rope_fwd_(b, tab, S, nkv, g, hd)
    assert torch.equal(a, b)
    keep("rope", assert_close_stats(a, q0, what="rope", **BF16))


def test_cross_entropy_distribution_canary_and_repeatability(ops):
    M, V = 257, 73448
    logits_view, check = padded((M, V), torch.bfloat16)
    src = rnd(M, V, scale=3.0)
    logits_view.copy_(src)
    labels = torch.randint(0, V, (M,), device="cuda", dtype=torch.int32)
    mask = (torch.rand(M, device="cuda") > 0.2).float()
    l64 = src.double()
    lse = torch.logsumexp(l64, -1)
    nll64 = (lse - l64.gather(1, labels.long()[:, None])[:, 0]) * mask.double()
    g64 = torch.softmax(l64, -1)
    g64[torch.arange(M), labels.long()] -= 1.0
    g64 = g64 * (mask.double() * 0.3)[:, None]
    nll = ops.cross_entropy_fwd_bwd(logits_view, labels, mask, 0.3)
    check()
    assert_close_stats(nll, nll64, mean=2e-6, p95=6e-6, mx=5e-5, bias=1e-6, what="nll")
    # gradient entries span many orders of magnitude: bound the error against the row's largest entry instead of the RMS
    err = (logits_view.double() - g64).abs().max().item()
    assert err < 2e-3, err
    keep("cross_entropy_grad", err_stats(logits_view, g64))
    again = src.clone()
    nll2 = ops.cross_entropy_fwd_bwd(again, labels, mask, 0.3)
    assert torch.equal(nll, nll2) and torch.equal(again, logits_view.contiguous())


def test_embedding_backward_deterministic_mode(ops):
    """Heavily repeated token ids (the case in which float atomics reorder): the deterministic form is bitwise repeatable,
    equals the fp64 sum to fp32 accuracy, respects the vocabulary shard and accumulates across calls."""
    V, H, M = 512, 256, 20000
    ids = (torch.randint(0, 40, (M,), device="cuda") ** 2 % V).to(torch.int32)   # a few very frequent tokens
    dout = rnd(M, H)
    lo, n_local = 64, 300
    ref = torch.zeros(V, H, device="cuda", dtype=torch.float64)
    ref.index_add_(0, ids.long(), dout.double() * 12.0)
    ref = ref[lo:lo + n_local]
    ops.set_deterministic(True)
    try:
        a, b = torch.zeros(n_local, H, device="cuda"), torch.zeros(n_local, H, device="cuda")
        ops.embedding_bwd(dout, ids, a, 12.0, lo)
        ops.embedding_bwd(dout, ids, b, 12.0, lo)
        assert torch.equal(a, b)
        assert_close_stats(a, ref, mean=2e-6, p95=6e-6, mx=1e-4, bias=1e-6, what="deterministic embedding bwd")
        ops.embedding_bwd(dout, ids, a, 12.0, lo)
        assert_close_stats(a, 2 * ref, mean=2e-6, p95=6e-6, mx=1e-4, bias=1e-6, what="accumulated twice")
    finally:
        ops.set_deterministic(False)
    c = torch.zeros(n_local, H, device="cuda")
    ops.embedding_bwd(dout, ids, c, 12.0, lo)            # atomic form: same sums to fp32 accuracy
    assert_close_stats(c, ref, mean=2e-6, p95=6e-6, mx=1e-4, bias=1e-6, what="atomic embedding bwd")


def test_adamw_distribution_and_repeatability(ops):
    n = 1 << 20
    master = torch.randn(n, device="cuda")
    m, v = torch.randn(n, device="cuda") * 0.1, torch.rand(n, device="cuda") * 0.01
    grad = torch.randn(n, device="cuda")
    gs = torch.tensor(0.5, device="cuda")
    segs = [(0, 0, n, 0.25, True)]
    lr, b1, b2, eps, wd, step = 1e-2, 0.9, 0.95, 1e-8, 0.1, 3
    g64 = grad.double() * 0.5
    m64 = b1 * m.double() + (1 - b1) * g64
    v64 = b2 * v.double() + (1 - b2) * g64 * g64
    upd = (m64 / (1 - b1 ** step)) / ((v64 / (1 - b2 ** step)).sqrt() + eps)
    w64 = master.double() * (1 - lr * 0.25 * wd) - lr * 0.25 * upd
    outs = []
    for _ in range(2):
        ma, mm, vv = master.clone(), m.clone(), v.clone()
        p = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
        ops.adamw_segments(ma, mm, vv, grad, p, segs, lr, b1, b2, eps, wd, step, gs)
        outs.append((ma, mm, vv, p))
    assert all(torch.equal(a, b) for a, b in zip(*outs))
    ma, mm, vv, p = outs[0]
    keep("adamw_master", assert_close_stats(ma, w64, mean=2e-7, p95=6e-7, mx=1e-5, bias=5e-8, what="adamw master"))
    assert_close_stats(mm, m64, mean=2e-7, p95=6e-7, mx=1e-5, bias=5e-8, what="exp_avg")
    assert_close_stats(vv, v64, mean=2e-6, p95=6e-6, mx=1e-4, bias=1e-6, what="exp_avg_sq")
    assert torch.equal(p, ma.to(torch.bfloat16))


def test_attention_in_kernel_timelines(ops):
    """The clock64 stamps of the attention kernels, read by the timeline tool: every phase of a step has a positive median
    and the phases add up to the step; with no buffer set the kernels skip the stamps (every other test runs that way)."""
    from forge_train_harness_b200.utils.attn_timeline import backward_timeline, forward_timeline
    f = forward_timeline(S=2048, B=1)
    b = backward_timeline(S=2048, B=1)
    for part in list(f.values()) + list(b.values()):
        assert part is not None and part["steps"] >= 8 and part["total"] > 500
        phases = [v for k, v in part.items() if k not in ("total", "steps")]
        assert all(v >= 0 for v in phases) and abs(sum(phases) - part["total"]) <= 0.25 * part["total"]
