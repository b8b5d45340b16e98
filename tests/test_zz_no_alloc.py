"""The allocation-free RMSNorm backward, called through its exported C symbol, against the regular entry point.

Collected last on purpose (file name): a run that stops at the first failure has then already run every other test.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import forge_train_harness_b200.ops.cuda_ops as co  # makes sure the extension and its dependencies are loaded
    lib = ctypes.CDLL(co._SO)
    fn = lib.fth_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    return co, fn


def _call(fn, dy, x, w, rstd, dres, dw, out_scale):
    dx = torch.empty_like(x)
    err = ctypes.create_string_buffer(256)
    rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dres.data_ptr() if dres is not None else None,
            dx.data_ptr(), dw.data_ptr(), x.shape[0], x.shape[1], out_scale,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), err, 256)
    return rc, dx, err.value.decode()


def test_no_alloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    co, fn = _lib()
    torch.manual_seed(0)
    # two calls in a row with different shapes: the second must not be disturbed by what the first left in the scratch
    for (M, H, use_res) in [(4096, 1024, True), (777, 4096, False)]:
        x = torch.randn(M, H, device="cuda").to(torch.bfloat16)
        dy = torch.randn(M, H, device="cuda").to(torch.bfloat16)
        dres = torch.randn(M, H, device="cuda").to(torch.bfloat16) if use_res else None
        w = (torch.randn(H, device="cuda") * 0.2 + 1).to(torch.bfloat16)
        _, rstd = co.Sm100Ops.rmsnorm_fwd(x, w, 1e-6)
        dw_ref = torch.full((H,), 0.5, device="cuda")
        dw_new = dw_ref.clone()
        dx_ref = co.Sm100Ops.rmsnorm_bwd(dy, x, w, rstd, dw_ref, dres, 0.5)
        rc, dx_new, msg = _call(fn, dy, x, w, rstd, dres, dw_new, 0.5)
        torch.cuda.synchronize()
        assert rc == 0, msg
        assert torch.equal(dx_new, dx_ref)  # per-row math is identical
        err = (dw_new - dw_ref).abs().max().item()
        assert err <= 2e-2 + 2e-2 * dw_ref.abs().max().item(), err  # different partial-sum grouping only


def test_no_alloc_rejects_rows_wider_than_the_scratch():
    co, fn = _lib()
    M, H = 8, 8192
    x = torch.randn(M, H, device="cuda").to(torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(M, device="cuda")
    dw = torch.zeros(H, device="cuda")
    rc, _, msg = _call(fn, x, x, w, rstd, None, dw, 1.0)
    assert rc != 0 and "4096" in msg
    assert float(dw.abs().sum()) == 0.0
