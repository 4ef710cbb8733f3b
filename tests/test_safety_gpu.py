"""GPU tests of the library's safety nets, all through the C ABI:

* the give-up path of the kernels' bounded waits (a wait that nothing completes runs out by itself after a few
  thousand cycles, the status word reports it, the convolution entry points refuse work until it is cleared);
* guard bands: outputs and workspaces sit between poisoned bands that must come back untouched, on shapes
  whose tiles are ragged in every direction (the substitute for a memory checker on the kernels' stores).
"""
import ctypes as C

import numpy as np
import pytest

from oracle import aether_oracle as O

pytestmark = pytest.mark.gpu
POISON = 0x7FA5A5A5          # a NaN bit pattern no kernel produces
BAND = 4096                  # floats before and after every buffer


@pytest.fixture(scope="module")
def env():
    import torch
    from aether_ml_b200 import _lib
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    return torch, _lib


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def test_bounded_wait_runs_out_and_is_reported(env):
    torch, _lib = env
    L = _lib.lib()
    torch.cuda.synchronize()
    assert L.aether_device_status() == 0
    assert L.aether_selftest_bounded_wait(0, None) == -1                       # limit out of range: nothing launched
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert L.aether_selftest_bounded_wait(20000, stream) == 0, L.aether_last_error()
    torch.cuda.synchronize()                                                    # the kernel ends by itself
    assert L.aether_device_status() == 5
    # while the code is pending the convolution entry points refuse to launch
    d = _lib.AetherConvDesc(2, 8, 8, 64, 64, 3, 3, 1, 1, 1, 1, _lib.MATH_BF16)
    x = torch.zeros((2, 8, 8, 64), device="cuda"); w = torch.zeros((3, 3, 64, 64), device="cuda")
    y = torch.empty((2, 8, 8, 64), device="cuda")
    ws = torch.empty(L.aether_conv2d_workspace_bytes(C.byref(d)), dtype=torch.uint8, device="cuda")
    n0 = _lib.launch_count()
    rc = L.aether_conv2d_fwd(C.byref(d), _ptr(x), _ptr(w), None, _ptr(y), _ptr(ws), ws.numel(), stream)
    assert rc == -4 and b"abandoned a bounded wait" in L.aether_last_error()
    assert _lib.launch_count() == n0
    L.aether_device_status_clear()
    assert L.aether_device_status() == 0
    rc = L.aether_conv2d_fwd(C.byref(d), _ptr(x), _ptr(w), None, _ptr(y), _ptr(ws), ws.numel(), stream)
    assert rc == 0, L.aether_last_error()
    torch.cuda.synchronize()
    assert L.aether_device_status() == 0 and float(y.abs().max()) == 0.0


class Banded:
    """A device array with a poisoned band on either side."""

    def __init__(self, torch, numel, dtype, fill=None):
        self.torch = torch
        self.item = 4 if dtype == torch.float32 else 1
        band = BAND * 4 // self.item
        self.raw = torch.empty(numel + 2 * band, dtype=dtype, device="cuda")
        self.band = band
        as_i32 = self.raw.view(torch.int32) if dtype != torch.int32 else self.raw
        as_i32[:BAND] = POISON
        as_i32[-BAND:] = POISON
        self.t = self.raw[band:band + numel]
        if fill is not None:
            self.t.copy_(fill.reshape(-1))
        elif dtype == torch.float32:
            self.t.view(torch.int32).fill_(POISON)

    def intact(self):
        i32 = self.raw.view(self.torch.int32)
        return bool((i32[:BAND] == POISON).all()) and bool((i32[-BAND:] == POISON).all())


# ragged in rows, columns, images and channels; halo, per-tap, first-layer and CUDA-core kernels
GUARD_SHAPES = [(3, 56, 56, 64, 128, 3, "same", "bf16"), (2, 33, 17, 16, 20, 3, "same", "bf16"),
                (5, 9, 7, 64, 64, 3, "valid", "bf16"), (2, 20, 150, 32, 32, 3, "same", "bf16"),
                (3, 30, 30, 128, 64, 3, "same", "bf16"), (2, 33, 17, 16, 20, 3, "same", "tf32"),
                (5, 17, 13, 3, 128, 3, "same", "bf16"), (3, 11, 9, 5, 7, 3, "same", "fp32")]


@pytest.mark.parametrize("shape", GUARD_SHAPES)
def test_guard_bands_around_outputs_and_workspace(env, shape):
    torch, _lib = env
    L = _lib.lib()
    S, H, W, Cin, Cout, f, pad, mode = shape
    P = (f - 1) // 2 if pad == "same" else 0
    Ho, Wo = H + 2 * P - f + 1, W + 2 * P - f + 1
    rng = np.random.default_rng(S * 1000 + H)
    xh = rng.standard_normal((S, H, W, Cin)).astype(np.float32)
    wh = (rng.standard_normal((f, f, Cin, Cout)) * np.sqrt(2.0 / (f * f * Cin))).astype(np.float32)
    bh = rng.standard_normal(Cout).astype(np.float32)
    dyh = rng.standard_normal((S, Ho, Wo, Cout)).astype(np.float32)
    d = _lib.AetherConvDesc(S, H, W, Cin, Cout, f, f, 1, 1, P, P, _lib.MATH_MODES[mode])
    x = Banded(torch, xh.size, torch.float32, torch.from_numpy(xh).cuda())
    w = Banded(torch, wh.size, torch.float32, torch.from_numpy(wh).cuda())
    b = Banded(torch, bh.size, torch.float32, torch.from_numpy(bh).cuda())
    dy = Banded(torch, dyh.size, torch.float32, torch.from_numpy(dyh).cuda())
    y = Banded(torch, S * Ho * Wo * Cout, torch.float32)
    dx = Banded(torch, xh.size, torch.float32)
    dw = Banded(torch, wh.size, torch.float32)
    db = Banded(torch, Cout, torch.float32)
    ws = Banded(torch, int(L.aether_conv2d_workspace_bytes(C.byref(d))), torch.uint8)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.aether_conv2d_fwd(C.byref(d), _ptr(x.t), _ptr(w.t), _ptr(b.t), _ptr(y.t), _ptr(ws.t), ws.t.numel(), stream)
    assert rc == 0, L.aether_last_error()
    torch.cuda.synchronize()
    everything = (x, w, b, dy, y, dx, dw, db, ws)
    assert all(a.intact() for a in everything), "forward wrote outside its arrays"
    rc = L.aether_conv2d_bwd(C.byref(d), _ptr(x.t), _ptr(dy.t), _ptr(w.t), _ptr(dx.t), _ptr(dw.t), _ptr(db.t), _ptr(ws.t),
                             ws.t.numel(), 1, stream)
    assert rc == 0, L.aether_last_error()
    torch.cuda.synchronize()
    assert L.aether_device_status() == 0
    assert all(a.intact() for a in everything), "backward wrote outside its arrays"
    # every output element was written (no poison left) and the inputs are unchanged
    for a in (y, dx, dw, db):
        assert not bool((a.t.view(torch.int32) == POISON).any())
    assert np.array_equal(x.t.cpu().numpy(), xh.reshape(-1)) and np.array_equal(dy.t.cpu().numpy(), dyh.reshape(-1))
    tol = {"bf16": 1e-2, "tf32": 1e-3, "fp32": 1e-5}[mode]
    yo = O.conv_forward_blas(xh, wh, bh, (1, 1), pad, dtype=np.float64)
    dxo, dwo, dbo = O.conv_backward_blas(xh, wh, dyh, (1, 1), pad, dtype=np.float64)
    assert O.rel_l2(y.t.cpu().numpy().reshape(yo.shape), yo) <= tol
    assert O.rel_l2(dx.t.cpu().numpy().reshape(dxo.shape), dxo) <= tol
    assert O.rel_l2(dw.t.cpu().numpy().reshape(dwo.shape), dwo) <= tol
    assert O.rel_l2(db.t.cpu().numpy(), dbo) <= 1e-5


def test_guard_bands_around_block_tail(env):
    """The fused Batch_Norm + ReLU + pooling passes, forward and backward, between poisoned bands."""
    torch, _lib = env
    L = _lib.lib()
    S, H, W, Cc = 3, 10, 6, 20
    rng = np.random.default_rng(5)
    xh = rng.standard_normal((S, H, W, Cc)).astype(np.float32)
    x = Banded(torch, xh.size, torch.float32, torch.from_numpy(xh).cuda())
    vec = lambda v: Banded(torch, Cc, torch.float32, torch.from_numpy(np.asarray(v, np.float32)).cuda())
    gamma, beta = vec(rng.random(Cc) + 0.5), vec(rng.standard_normal(Cc))
    rm, rv, bm, bv = vec(np.zeros(Cc)), vec(np.ones(Cc)), vec(np.zeros(Cc)), vec(np.zeros(Cc))
    dgamma, dbeta = vec(np.zeros(Cc)), vec(np.zeros(Cc))
    n_pool = S * (H // 2) * (W // 2) * Cc
    pooled = Banded(torch, n_pool, torch.float32)
    arg = Banded(torch, n_pool, torch.uint8)
    dyp = Banded(torch, n_pool, torch.float32, torch.from_numpy(rng.standard_normal(n_pool).astype(np.float32)).cuda())
    dx = Banded(torch, xh.size, torch.float32)
    ws = Banded(torch, int(L.aether_bn_workspace_bytes(S * H * W, Cc)), torch.uint8)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.aether_bn_act_pool_fwd(_ptr(x.t), None, 0, _ptr(gamma.t), _ptr(beta.t), _ptr(rm.t), _ptr(rv.t), _ptr(bm.t),
                                  _ptr(bv.t), _ptr(pooled.t), _ptr(arg.t), S, H, W, Cc, 2, 2, 1e-5, 0.9, 0.0, None, 1,
                                  _ptr(ws.t), ws.t.numel(), stream)
    assert rc == 0, L.aether_last_error()
    rc = L.aether_bn_act_pool_bwd(_ptr(x.t), _ptr(dyp.t), _ptr(arg.t), _ptr(gamma.t), _ptr(beta.t), _ptr(bm.t), _ptr(bv.t),
                                  _ptr(dx.t), _ptr(dgamma.t), _ptr(dbeta.t), S, H, W, Cc, 2, 2, 1e-5, 0.0, None, _ptr(ws.t),
                                  ws.t.numel(), stream)
    assert rc == 0, L.aether_last_error()
    torch.cuda.synchronize()
    for a in (x, gamma, beta, rm, rv, bm, bv, dgamma, dbeta, pooled, arg, dyp, dx, ws):
        assert a.intact()
    assert not bool((pooled.t.view(torch.int32) == POISON).any()) and not bool((dx.t.view(torch.int32) == POISON).any())


def test_guard_bands_around_block_tail_with_operand_copies(env):
    """The same passes in their hand-off form: bf16 operand copies (rows padded from 32 to 64 channels),
    column sums, the selected-cell values, and the fp32 results left out (NULL) -- every buffer between poisoned bands."""
    torch, _lib = env
    L = _lib.lib()
    S, H, W, Cc, ld = 3, 10, 6, 32, 64
    rng = np.random.default_rng(6)
    xh = rng.standard_normal((S, H, W, Cc)).astype(np.float32)
    x = Banded(torch, xh.size, torch.float32, torch.from_numpy(xh).cuda())
    vec = lambda v: Banded(torch, Cc, torch.float32, torch.from_numpy(np.asarray(v, np.float32)).cuda())
    gamma, beta = vec(rng.random(Cc) + 0.5), vec(rng.standard_normal(Cc))
    rm, rv, bm, bv = vec(np.zeros(Cc)), vec(np.ones(Cc)), vec(np.zeros(Cc)), vec(np.zeros(Cc))
    dgamma, dbeta = vec(np.zeros(Cc)), vec(np.zeros(Cc))
    n_win = S * (H // 2) * (W // 2)
    arg = Banded(torch, n_win * Cc, torch.uint8)
    xsel = Banded(torch, n_win * Cc, torch.float32)
    copy_f = Banded(torch, n_win * ld * 2, torch.uint8)               # bf16 [windows][ld]
    copy_b = Banded(torch, S * H * W * ld * 2, torch.uint8)           # bf16 [pixels][ld]
    rows_max = 8
    colsum = Banded(torch, rows_max * Cc, torch.float32)
    dyp = Banded(torch, n_win * Cc, torch.float32, torch.from_numpy(rng.standard_normal(n_win * Cc).astype(np.float32)).cuda())
    ws = Banded(torch, int(L.aether_bn_workspace_bytes(S * H * W, Cc)), torch.uint8)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    rc = L.aether_bn_act_pool_fwd_copy(_ptr(x.t), None, 0, _ptr(gamma.t), _ptr(beta.t), _ptr(rm.t), _ptr(rv.t), _ptr(bm.t),
                                       _ptr(bv.t), None, _ptr(arg.t), S, H, W, Cc, 2, 2, 1e-5, 0.9, 0.0, None, 1,
                                       _ptr(copy_f.t), ld, _ptr(xsel.t), _ptr(ws.t), ws.t.numel(), stream)
    assert rc == 0, L.aether_last_error()
    rows = C.c_int(0)
    rc = L.aether_bn_act_pool_bwd_copy(_ptr(x.t), _ptr(dyp.t), _ptr(arg.t), _ptr(gamma.t), _ptr(beta.t), _ptr(bm.t), _ptr(bv.t),
                                       None, _ptr(dgamma.t), _ptr(dbeta.t), S, H, W, Cc, 2, 2, 1e-5, 0.0, None, _ptr(copy_b.t), ld,
                                       _ptr(colsum.t), rows_max, C.byref(rows), _ptr(xsel.t), _ptr(ws.t), ws.t.numel(), stream)
    assert rc == 0, L.aether_last_error()
    torch.cuda.synchronize()
    assert 1 <= rows.value <= rows_max
    for a in (x, gamma, beta, rm, rv, bm, bv, dgamma, dbeta, arg, xsel, copy_f, copy_b, colsum, dyp, ws):
        assert a.intact()
    # the copies: values in the first Cc channels of every row, zeros in the padding
    cf = copy_f.t.view(torch.bfloat16).view(n_win, ld).float()
    cb = copy_b.t.view(torch.bfloat16).view(S * H * W, ld).float()
    assert float(cf[:, Cc:].abs().max()) == 0.0 and float(cb[:, Cc:].abs().max()) == 0.0
    assert float(cf[:, :Cc].abs().max()) > 0.0 and float(cb[:, :Cc].abs().max()) > 0.0
    # column sums of the dx that was never written as fp32: compare with the copy's own column sums (bf16 rounding)
    got = colsum.t.view(rows_max, Cc)[:rows.value].sum(dim=0)
    want = cb[:, :Cc].sum(dim=0)
    assert float((got - want).abs().max()) <= 2e-2 * float(cb.abs().sum(dim=0).max())
