"""GPU parity tests of Conv_Layer (through the C ABI) against the NumPy oracle and the golden vectors
made by the reference's own classes.  Tolerances are relative L2: 1e-2 for bf16, 1e-3 for tf32,
1e-5 for the fp32 CUDA-core path."""
import zlib

import numpy as np
import pytest

from oracle import aether_oracle as O

pytestmark = pytest.mark.gpu
TOL = {"bf16": 1e-2, "tf32": 1e-3, "fp32": 1e-5}


@pytest.fixture(scope="module")
def env():
    import torch
    from aether_ml_b200 import _lib, layers
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    return torch, _lib, layers


def first_layer_tc(mode, w):
    """bf16 mode runs first layers (1-4 input channels, K <= 64, 16..256 filters) on the tensor cores with
    thread-built bf16 operands: forward always, dW when the filter count is a power of two (dB is summed in fp32
    either way and dX, which a first layer rarely needs, stays on the CUDA cores)."""
    fH, fW, Cin, Cout = w.shape
    return mode == "bf16" and Cin <= 4 and fH * fW * Cin <= 64 and Cout % 4 == 0 and 16 <= Cout <= 256


def first_layer_tc_dw(mode, w):
    Cout = w.shape[3]
    return first_layer_tc(mode, w) and Cout & (Cout - 1) == 0


def run_layer(env, mode, x, w, b, dy, f, st, pad):
    torch, _lib, layers = env
    np.random.seed(0)
    layer = layers.Conv_Layer(x.shape[1:], w.shape[3], tuple(f), tuple(st), pad, math_mode=mode)
    layer.set_parameters(w, b)
    assert layer.weights is layer.filter_weights
    y = layer.forward(x, True)
    dx = layer.backward(dy)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    return (y.cpu().numpy(), dx.cpu().numpy(), layer.dweights.cpu().numpy(), layer.dbiases.cpu().numpy())


GOLDEN = ["conv_same_3x3", "conv_valid_3x3", "conv_same_5x5", "conv_stride2_valid", "conv_tensor_path_small",
          "conv_cfg1_tiny"]


@pytest.mark.parametrize("mode", ["bf16", "tf32", "fp32"])
@pytest.mark.parametrize("name", GOLDEN)
def test_golden_vectors(env, golden, name, mode):
    g = golden(name)
    st = tuple(int(v) for v in g["strides"]); f = tuple(int(v) for v in g["filter_size"]); pad = str(g["padding"])
    y, dx, dw, db = run_layer(env, mode, g["x"], g["w"], g["b"], g["dy"], f, st, pad)
    # shapes outside the tensor-core path run in fp32 whatever the requested mode
    tensor_path = name == "conv_tensor_path_small" and mode != "fp32"
    tol = TOL[mode] if tensor_path else TOL["fp32"]
    assert y.shape == g["y"].shape and dx.shape == g["x"].shape and dw.shape == g["w"].shape
    assert O.rel_l2(y, g["y"]) <= (TOL["bf16"] if first_layer_tc(mode, g["w"]) else tol)
    assert O.rel_l2(dx, g["dx"]) <= tol
    assert O.rel_l2(dw, g["dw"]) <= (TOL["bf16"] if first_layer_tc_dw(mode, g["w"]) else tol)
    assert O.rel_l2(db, g["db"]) <= tol


def test_notebook_known_answers(env, golden):
    g = golden("notebook_kat")
    zeros = np.zeros(1, np.float32)
    y, _, _, _ = run_layer(env, "fp32", g["image"][None, :, :, None], g["kernel"][:, :, None, None], zeros,
                           np.zeros((1, 4, 4, 1), np.float32), (3, 3), (1, 1), "same")
    assert np.array_equal(y[0, :, :, 0], g["expected"])
    ones = np.ones((1, 5, 5, 3), np.float32)
    y, _, _, _ = run_layer(env, "fp32", ones, np.ones((3, 3, 3, 1), np.float32), zeros,
                           np.zeros((1, 3, 3, 1), np.float32), (3, 3), (1, 1), "valid")
    assert y.shape == (1, 3, 3, 1) and np.all(y == 27)


# (S, H, W, Cin, Cout, f, pad): tensor-core shapes incl. ragged tiles, padded channel counts, 1x1, 5x5
SHAPES = [
    (2, 8, 8, 64, 64, 3, "same"), (8, 16, 16, 128, 128, 3, "same"), (3, 56, 56, 64, 128, 3, "same"),
    (16, 8, 8, 256, 256, 3, "same"), (4, 14, 14, 32, 64, 3, "same"), (5, 9, 7, 64, 64, 3, "valid"),
    (3, 10, 10, 48, 80, 5, "same"), (200, 1, 1, 512, 128, 1, "valid"), (2, 33, 17, 16, 20, 3, "same"),
    (1, 3, 3, 64, 192, 3, "same"), (130, 4, 4, 64, 64, 3, "same"), (2, 20, 150, 32, 32, 3, "same"),
    # enough 256-wide work for CTA pairs: an odd number of pixel tiles (forward), dX at 256 input channels, two column tiles
    (61, 24, 24, 128, 256, 3, "same"), (150, 16, 16, 256, 128, 3, "same"), (300, 8, 8, 128, 512, 3, "same"),
    # 27 strips per image x 11: in TF32 the 295 KB filter only fits the window kernel as two halves on a CTA pair
    (11, 54, 56, 64, 128, 3, "same"),
]


@pytest.mark.parametrize("mode", ["bf16", "tf32"])
@pytest.mark.parametrize("shape", SHAPES)
def test_tensor_core_shapes(env, shape, mode):
    S, H, W, Cin, Cout, f, pad = shape
    rng = np.random.default_rng(zlib.crc32(repr(shape).encode()))       # the same inputs in every run
    x = rng.standard_normal((S, H, W, Cin)).astype(np.float32)
    w = (rng.standard_normal((f, f, Cin, Cout)) * np.sqrt(2.0 / (f * f * Cin))).astype(np.float32)
    b = (rng.standard_normal(Cout) * 0.1).astype(np.float32)
    Ho, Wo = O.conv_out_hw(H, W, (f, f), (1, 1), pad)
    dy = rng.standard_normal((S, Ho, Wo, Cout)).astype(np.float32)
    y, dx, dw, db = run_layer(env, mode, x, w, b, dy, (f, f), (1, 1), pad)
    yo = O.conv_forward_blas(x, w, b, (1, 1), pad, dtype=np.float64)
    dxo, dwo, dbo = O.conv_backward_blas(x, w, dy, (1, 1), pad, dtype=np.float64)
    tol = TOL[mode]
    assert O.rel_l2(y, yo) <= tol and O.rel_l2(dx, dxo) <= tol
    assert O.rel_l2(dw, dwo) <= tol and O.rel_l2(db, dbo) <= 1e-5


@pytest.mark.parametrize("shape", [(4, 20, 24, 64, 128, (3, 4), "same"), (3, 16, 30, 64, 128, (3, 2), "valid"),
                                   (2, 14, 40, 128, 256, (3, 3), "same"), (5, 13, 19, 64, 128, (3, 3), "valid"),
                                   (2, 15, 15, 64, 128, (5, 3), "same")])
def test_filter_row_dw_shapes(env, shape):
    """Three-row filters of width 2..4 on >= 12-pixel-wide images with 128-multiple output channels take the
    dW kernel that stacks a filter row's taps along N (two CTA classes); rectangular filters, ragged strips,
    several channel blocks.  The (5, 3) filter is a neighbour that must fall back to the other dW kernels."""
    S, H, W, Cin, Cout, f, pad = shape
    rng = np.random.default_rng(11)
    x = rng.standard_normal((S, H, W, Cin)).astype(np.float32)
    w = (rng.standard_normal((f[0], f[1], Cin, Cout)) * np.sqrt(2.0 / (f[0] * f[1] * Cin))).astype(np.float32)
    b = (rng.standard_normal(Cout) * 0.1).astype(np.float32)
    Ho, Wo = O.conv_out_hw(H, W, f, (1, 1), pad)
    dy = rng.standard_normal((S, Ho, Wo, Cout)).astype(np.float32)
    y, dx, dw, db = run_layer(env, "bf16", x, w, b, dy, f, (1, 1), pad)
    yo = O.conv_forward_blas(x, w, b, (1, 1), pad, dtype=np.float64)
    dxo, dwo, dbo = O.conv_backward_blas(x, w, dy, (1, 1), pad, dtype=np.float64)
    tol = TOL["bf16"]
    assert O.rel_l2(y, yo) <= tol and O.rel_l2(dx, dxo) <= tol
    assert O.rel_l2(dw, dwo) <= tol and O.rel_l2(db, dbo) <= 1e-5
    # every tap's gradient on its own (a tap dropped or doubled by a kernel barely moves the global norm)
    for i in range(f[0]):
        for j in range(f[1]):
            assert O.rel_l2(dw[i, j], dwo[i, j]) <= 2 * tol, (i, j)


@pytest.mark.parametrize("shape", [(3, 9, 9, 3, 8, 3, (2, 2), "valid"), (2, 12, 10, 5, 7, 3, (1, 1), "same"),
                                   (4, 28, 28, 1, 32, 3, (1, 1), "same"), (2, 11, 11, 4, 6, 5, (2, 1), "same"),
                                   # first-layer kernels (1..4 input channels, power-of-two filter count 16..256)
                                   (5, 17, 13, 3, 128, 3, (1, 1), "same"), (3, 20, 20, 1, 64, 5, (2, 2), "valid"),
                                   (2, 9, 9, 3, 256, 3, (1, 2), "same"), (6, 14, 14, 2, 16, 3, (1, 1), "same"),
                                   (70, 32, 32, 3, 128, 3, (1, 1), "same"),
                                   # several tiles per CTA with two operand stages (256 filters) / four (64)
                                   (300, 16, 16, 3, 256, 3, (1, 1), "same"), (500, 16, 16, 4, 64, 3, (1, 1), "same")])
def test_cuda_core_shapes(env, shape):
    S, H, W, Cin, Cout, f, st, pad = shape
    rng = np.random.default_rng(3)
    x = rng.random((S, H, W, Cin)).astype(np.float32)
    w = rng.standard_normal((f, f, Cin, Cout)).astype(np.float32)
    b = rng.standard_normal(Cout).astype(np.float32)
    Ho, Wo = O.conv_out_hw(H, W, (f, f), st, pad)
    dy = rng.standard_normal((S, Ho, Wo, Cout)).astype(np.float32)
    yo = O.conv_forward(x, w, b, st, pad)
    dxo, dwo, dbo = O.conv_backward(x, w, dy, st, pad)
    y, dx, dw, db = run_layer(env, "fp32", x, w, b, dy, (f, f), st, pad)
    for a, o in ((y, yo), (dx, dxo), (dw, dwo), (db, dbo)):
        assert O.rel_l2(a, o) <= 1e-5
    # the same layer in bf16 mode: first layers run forward on the tensor cores, everything else is unchanged
    y, dx, dw, db = run_layer(env, "bf16", x, w, b, dy, (f, f), st, pad)
    assert O.rel_l2(y, yo) <= (TOL["bf16"] if first_layer_tc("bf16", w) else 1e-5)
    assert O.rel_l2(dw, dwo) <= (TOL["bf16"] if first_layer_tc_dw("bf16", w) else 1e-5)
    for a, o in ((dx, dxo), (db, dbo)):
        assert O.rel_l2(a, o) <= 1e-5


def test_config1_full_size(env):
    """First BASELINE config: (128,32,32,3) -> 32 filters, U[0,1) inputs, He-normal filters, zero bias."""
    rng = np.random.default_rng(1235)
    x = rng.random((128, 32, 32, 3)).astype(np.float32)
    w = (rng.standard_normal((3, 3, 3, 32)) * np.sqrt(2.0 / 27)).astype(np.float32)
    b = np.zeros(32, np.float32)
    dy = rng.standard_normal((128, 32, 32, 32)).astype(np.float32)
    y, dx, dw, db = run_layer(env, "bf16", x, w, b, dy, (3, 3), (1, 1), "same")
    yo = O.conv_forward_blas(x, w, b, dtype=np.float64)
    dxo, dwo, dbo = O.conv_backward_blas(x, w, dy, dtype=np.float64)
    assert O.rel_l2(y, yo) <= TOL["bf16"]                  # forward and dW: thread-built bf16 operands, tensor cores
    assert O.rel_l2(dw, dwo) <= TOL["bf16"]
    for a, o in ((dx, dxo), (db, dbo)):
        assert O.rel_l2(a, o) <= 1e-5
    y32 = run_layer(env, "fp32", x, w, b, dy, (3, 3), (1, 1), "same")[0]
    assert O.rel_l2(y32, yo) <= 1e-5


@pytest.mark.parametrize("mode", ["bf16", "tf32"])
@pytest.mark.parametrize("shape", [(256, 32, 32, 64, 64), (256, 16, 16, 128, 128), (256, 8, 8, 256, 256),
                                   (256, 56, 56, 64, 128)])
def test_sweep_shapes_full_size_properties(env, shape, mode):
    """Full-size sweep shapes: size-independent checks instead of a full CPU recomputation.
    (1) adjoint identities <conv(x;b=0), dy> = <x, dX> = <W, dW>; (2) a random sample of output
    pixels, input pixels and filter taps recomputed exactly on the CPU; (3) dB = column sums;
    (4) bit-identical results when run twice (fixed-order reductions)."""
    torch, _lib, layers = env
    S, H, W, Cin, Cout = shape
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn((S, H, W, Cin), generator=g, device="cuda")
    dy = torch.randn((S, H, W, Cout), generator=g, device="cuda")
    np.random.seed(5)
    layer = layers.Conv_Layer((H, W, Cin), Cout, (3, 3), (1, 1), "same", math_mode=mode)
    y = layer.forward(x, True).clone()
    dx = layer.backward(dy).clone()
    dw = layer.dweights.clone(); db = layer.dbiases.clone()
    y2 = layer.forward(x, True)
    dx2 = layer.backward(dy)
    torch.cuda.synchronize()
    assert _lib.device_status() == 0
    assert torch.equal(y, y2) and torch.equal(dx, dx2) and torch.equal(dw, layer.dweights) and torch.equal(db, layer.dbiases)
    tol = TOL[mode]
    a = float((y.double() * dy.double()).sum())            # bias is zero at construction
    bx = float((x.double() * dx.double()).sum())
    bw = float((layer.filter_weights.double() * dw.double()).sum())
    scale = float(y.double().norm() * dy.double().norm())
    assert abs(a - bx) <= tol * scale and abs(a - bw) <= tol * scale
    assert O.rel_l2(db.cpu().numpy(), dy.double().sum(dim=(0, 1, 2)).cpu().numpy()) <= 1e-5
    # sampled exact recomputation
    rng = np.random.default_rng(11)
    w = layer.filter_weights.cpu().numpy().astype(np.float64)
    xs = x.cpu().numpy(); dys = dy.cpu().numpy()
    ref, got = [], []
    for _ in range(48):
        s, h, ww = rng.integers(S), rng.integers(H), rng.integers(W)
        acc = np.zeros(Cout); accx = np.zeros(Cin)
        for i in range(3):
            for j in range(3):
                hi, wi = h + i - 1, ww + j - 1
                if 0 <= hi < H and 0 <= wi < W:
                    acc += xs[s, hi, wi].astype(np.float64) @ w[i, j]
                ho, wo = h + 1 - i, ww + 1 - j
                if 0 <= ho < H and 0 <= wo < W:
                    accx += w[i, j] @ dys[s, ho, wo].astype(np.float64)
        ref.append(np.concatenate([acc, accx])); got.append(np.concatenate([y[s, h, ww].cpu().numpy(), dx[s, h, ww].cpu().numpy()]))
    assert O.rel_l2(np.stack(got), np.stack(ref)) <= tol
    # a few filter taps of dW over the full reduction
    for (i, j) in ((0, 0), (1, 1), (2, 1)):
        xp = torch.nn.functional.pad(x, (0, 0, 1, 1, 1, 1))[:, i:i + H, j:j + W, :]
        ref_tap = (xp.reshape(-1, Cin).double().T @ dy.reshape(-1, Cout).double()).cpu().numpy()
        assert O.rel_l2(dw[i, j].cpu().numpy(), ref_tap) <= tol


def test_edge_cases_and_errors(env):
    torch, _lib, layers = env
    layer = layers.Conv_Layer((8, 8, 64), 64, math_mode="bf16")
    with pytest.raises(ValueError):
        layer.forward(np.zeros((2, 8, 8), np.float32), True)                 # not 4-D
    with pytest.raises(ValueError):
        layer.forward(np.zeros((2, 8, 8, 32), np.float32), True)             # wrong channel count
    with pytest.raises(RuntimeError):
        layers.Conv_Layer((8, 8, 64), 64).backward(np.zeros((2, 8, 8, 64), np.float32))
    layer.forward(np.zeros((2, 8, 8, 64), np.float32), True)
    with pytest.raises(ValueError):
        layer.backward(np.zeros((2, 8, 8, 32), np.float32))                  # wrong dvalues shape
    small = layers.Conv_Layer((2, 2, 4), 4, filter_size=(5, 5), padding="valid")
    with pytest.raises(ValueError):
        small.forward(np.zeros((1, 2, 2, 4), np.float32), True)              # filter larger than input
    # batch of one, single pixel
    one = layers.Conv_Layer((1, 1, 64), 64, math_mode="bf16")
    x = np.ones((1, 1, 1, 64), np.float32)
    y = one.forward(x, True).cpu().numpy()
    assert O.rel_l2(y, O.conv_forward(x, one.filter_weights.cpu().numpy(), np.zeros(64))) <= 1e-2


def test_operand_copies_are_rebuilt_when_their_source_changes(env):
    """The backward pass reuses the bf16 copies of x and of the filter that the forward pass left in the workspace
    only while they still describe the arrays: after an in-place change of the weights (dX must use the NEW
    weights, as the reference's backward reads filter_weights when it runs, CNN_classes_cupy.py:138) or of the
    stored input (dW must use the new values) the copies are rebuilt; untouched arrays take the short path."""
    torch, _lib, layers = env
    rng = np.random.default_rng(8)
    S, H, W, Cin, Cout = 3, 12, 12, 64, 64
    x = rng.standard_normal((S, H, W, Cin)).astype(np.float32)
    dy = rng.standard_normal((S, H, W, Cout)).astype(np.float32)
    np.random.seed(3)
    layer = layers.Conv_Layer((H, W, Cin), Cout, (3, 3), (1, 1), "same", math_mode="bf16")
    xt = torch.from_numpy(x).cuda()
    layer.forward(xt, True)
    n0 = _lib.launch_count()
    layer.backward(dy)
    short = _lib.launch_count() - n0                          # nothing changed: both copies reused
    layer.forward(xt, True)
    layer.filter_weights.mul_(-0.5)                           # in-place change between the passes
    xt.add_(1.0)
    n0 = _lib.launch_count()
    dx = layer.backward(dy)
    assert _lib.launch_count() - n0 == short + 2              # one more cast pass (x) and one more filter pass
    torch.cuda.synchronize()
    w_new = layer.filter_weights.cpu().numpy()
    dxo, dwo, dbo = O.conv_backward_blas(x + 1.0, w_new, dy, dtype=np.float64)
    assert O.rel_l2(dx.cpu().numpy(), dxo) <= TOL["bf16"]
    assert O.rel_l2(layer.dweights.cpu().numpy(), dwo) <= TOL["bf16"]
