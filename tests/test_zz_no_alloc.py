"""GPU test of aether_bn_fwd_train_static, the Batch_Norm training forward that keeps its scratch inside the
library instead of taking a workspace (for hosts that cannot allocate device memory around the call).
Called straight through the C ABI and compared with aether_bn_fwd_train on the same inputs, twice in a row
with different shapes so that the second call runs on top of the first call's leftovers.
This file sorts last on purpose: a run that stops at the first failure has then already run every other test."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _run_both(torch, L, shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(shape, generator=g, device="cuda") * 2.0 + 3.0
    Cc = shape[-1]
    rows = x.numel() // Cc
    gamma = torch.rand(Cc, generator=g, device="cuda") + 0.5
    beta = torch.randn(Cc, generator=g, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = {}
    for name in ("workspace", "static"):
        rm = torch.zeros(Cc, device="cuda"); rv = torch.ones(Cc, device="cuda")
        bm = torch.empty(Cc, device="cuda"); bv = torch.empty(Cc, device="cuda")
        y = torch.empty_like(x)
        if name == "workspace":
            ws = torch.empty(L.aether_bn_workspace_bytes(rows, Cc), dtype=torch.uint8, device="cuda")
            rc = L.aether_bn_fwd_train(_ptr(x), _ptr(gamma), _ptr(beta), _ptr(rm), _ptr(rv), _ptr(bm), _ptr(bv), _ptr(y),
                                       rows, Cc, 1e-5, 0.9, _ptr(ws), ws.numel(), stream)
        else:
            rc = L.aether_bn_fwd_train_static(_ptr(x), _ptr(gamma), _ptr(beta), _ptr(rm), _ptr(rv), _ptr(bm), _ptr(bv),
                                              _ptr(y), rows, Cc, 1e-5, 0.9, stream)
        assert rc == 0, L.aether_last_error()
        torch.cuda.synchronize()
        out[name] = [t.double().cpu().numpy() for t in (y, bm, bv, rm, rv)]
    return out


def test_static_scratch_matches_workspace_variant_twice():
    import torch
    from aether_ml_b200 import _lib
    if not torch.cuda.is_available():
        pytest.fail("CUDA device required for -m gpu tests")
    L = _lib.lib()
    # first a large call (fills much of the built-in scratch), then a smaller one on top of its leftovers
    for shape, seed in (((128, 32, 32, 64), 1), ((37, 5, 3, 12), 2), ((64, 1000), 3)):
        res = _run_both(torch, L, shape, seed)
        for a, b in zip(res["static"], res["workspace"]):
            err = np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)
            assert err <= 1e-5, (shape, err)
    # beyond the stated limit the call is refused, with a message, before anything is launched
    launches = _lib.launch_count()
    x = torch.zeros((4, 2048), device="cuda"); v = torch.zeros(2048, device="cuda")
    rc = L.aether_bn_fwd_train_static(_ptr(x), _ptr(v), _ptr(v), _ptr(v), _ptr(v), _ptr(v), _ptr(v), _ptr(x), 4, 2048,
                                      1e-5, 0.9, None)
    assert rc == -2 and b"exceeds the built-in scratch" in L.aether_last_error()
    assert _lib.launch_count() == launches
