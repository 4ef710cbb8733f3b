"""ctypes binding of libaether_b200.so (declared in include/aether_b200.h).

The library is the only compute path: there is no CPU or eager fallback.  ``lib()`` raises if the
shared object is missing, and every wrapper raises on a non-zero return code.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("AETHER_LIB", os.path.join(_HERE, "libaether_b200.so"))

MATH_BF16, MATH_TF32, MATH_FP32 = 0, 1, 2
MATH_MODES = {"bf16": MATH_BF16, "tf32": MATH_TF32, "fp32": MATH_FP32}
POOL_MAX, POOL_AVG = 0, 1


class AetherConvDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("S", "H", "W", "Cin", "Cout", "fH", "fW", "sH", "sW", "padH", "padW", "math_mode")]


class AetherOperandLayout(C.Structure):
    _fields_ = [("x_copy_offset", C.c_size_t), ("x_copy_ld", C.c_int32), ("dy_copy_offset", C.c_size_t),
                ("dy_copy_ld", C.c_int32), ("dy_colsum_offset", C.c_size_t), ("dy_colsum_rows_max", C.c_int32)]


CONV_X_COPY_READY, CONV_W_COPY_READY, CONV_DY_COPY_READY = 1, 2, 4


class AetherError(RuntimeError):
    pass


_P = C.c_void_p
_F = C.c_float
_I = C.c_int
_I64 = C.c_int64
_U64 = C.c_uint64
_SZ = C.c_size_t
_D = C.POINTER(AetherConvDesc)

# name -> (restype, argtypes); kept in one table so a test can check it against the header.
SIGNATURES = {
    "aether_version": (_I, []),
    "aether_last_error": (C.c_char_p, []),
    "aether_launch_count": (_U64, []),
    "aether_device_status": (_I, []),
    "aether_device_status_clear": (None, []),
    "aether_selftest_bounded_wait": (_I, [_I64, _P]),
    "aether_profile_enable": (_I, [_I]),
    "aether_profile_read": (_I, [_I, C.POINTER(C.c_double), C.POINTER(C.c_int)]),
    "aether_profile_reset": (None, []),
    "aether_conv2d_workspace_bytes": (_SZ, [_D]),
    "aether_conv2d_fwd": (_I, [_D, _P, _P, _P, _P, _P, _SZ, _P]),
    "aether_conv2d_bnstats_blocks": (_I64, [_D]),
    "aether_conv2d_fwd_bnstats": (_I, [_D, _P, _P, _P, _P, _P, _SZ, _P, _SZ, _P]),
    "aether_conv2d_bwd": (_I, [_D, _P, _P, _P, _P, _P, _P, _P, _SZ, _I, _P]),
    "aether_conv2d_operand_layout": (_I, [_D, C.POINTER(AetherOperandLayout)]),
    "aether_conv2d_fwd_ex": (_I, [_D, _P, _P, _P, _P, _P, _SZ, _P, _SZ, _I, _P]),
    "aether_conv2d_bwd_ex": (_I, [_D, _P, _P, _P, _P, _P, _P, _P, _SZ, _I, _I, _P]),
    "aether_bn_act_pool_fwd_copy": (_I, [_P, _P, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _F, _P,
                                         _I, _P, _I, _P, _P, _SZ, _P]),
    "aether_bn_act_pool_bwd_copy": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _P, _P, _I,
                                         _P, _I, C.POINTER(C.c_int), _P, _P, _SZ, _P]),
    "aether_bn_act_fwd_train": (_I, [_P, _P, _I64, _P, _P, _P, _P, _P, _P, _P, _I64, _I, _F, _F, _F, _P, _P, _SZ, _P]),
    "aether_bn_act_fwd_eval": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I, _F, _F, _P, _SZ, _P]),
    "aether_bn_act_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I64, _I, _F, _F, _P, _P, _SZ, _P]),
    "aether_bn_act_pool_fwd": (_I, [_P, _P, _I64, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _F, _P, _I,
                                    _P, _SZ, _P]),
    "aether_bn_act_pool_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _F, _P, _P, _SZ, _P]),
    "aether_bn_fwd_train_partials": (_I, [_P, _P, _I64, _P, _P, _P, _P, _P, _P, _P, _I64, _I, _F, _F, _P, _SZ, _P]),
    "aether_bn_workspace_bytes": (_SZ, [_I64, _I]),
    "aether_bn_fwd_train": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I64, _I, _F, _F, _P, _SZ, _P]),
    "aether_bn_fwd_train_static": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I64, _I, _F, _F, _P]),
    "aether_bn_fwd_eval": (_I, [_P, _P, _P, _P, _P, _P, _I64, _I, _F, _P, _SZ, _P]),
    "aether_bn_bwd": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I64, _I, _F, _P, _SZ, _P]),
    "aether_pool_fwd": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P]),
    "aether_pool_bwd": (_I, [_P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P]),
    "aether_leaky_relu_fwd": (_I, [_P, _P, _I64, _F, _P]),
    "aether_leaky_relu_bwd": (_I, [_P, _P, _P, _I64, _F, _P]),
    "aether_channel_scale": (_I, [_P, _P, _P, _I64, _I, _P]),
    "aether_dropout_fwd": (_I, [_P, _P, _P, _I64, _F, _U64, _U64, _P]),
    "aether_mul": (_I, [_P, _P, _P, _I64, _P]),
    "aether_adam_step": (_I, [_P, _P, _P, _P, _I64, _F, _F, _F, _F, _F, _F, _F, _P]),
    "aether_adam_step_dev": (_I, [_P, _P, _P, _P, _I64, _F, _F, _F, _F, _F, _F, _P, _P]),
    "aether_dropout_fwd_dev": (_I, [_P, _P, _P, _I64, _F, _U64, _U64, _P, _P]),
    "aether_channel_mask_dev": (_I, [_P, _I, _F, _U64, _P, _P]),
    "aether_regularizer_grad": (_I, [_P, _P, _I64, _F, _F, _P]),
    "aether_regularizer_loss": (_I, [_P, _I64, _F, _F, _P, _P]),
    "aether_softmax_cce": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _P]),
    "aether_softmax_bwd": (_I, [_P, _P, _P, _I, _I, _P]),
    "aether_softmax_cce_targets": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _F, _F, _I, _P]),
}

_lib = None


def lib():
    """Load (once) and return the ctypes handle; raises if the library has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise AetherError(
                "libaether_b200.so not found at %s -- build it with `python -m aether_ml_b200.build` "
                "(there is no fallback path)" % LIB_PATH)
        h = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            try:
                fn = getattr(h, name)
            except AttributeError:
                raise AetherError("%s does not export %s: it was built from older sources -- rebuild it with "
                                  "`python -m aether_ml_b200.build`" % (LIB_PATH, name)) from None
            fn.restype = res
            fn.argtypes = args
        _lib = h
    return _lib


def check(rc, what=""):
    if rc != 0:
        msg = lib().aether_last_error().decode("utf-8", "replace")
        if rc == -1:
            raise ValueError("%s: %s" % (what, msg))
        raise AetherError("%s failed (%d): %s" % (what, rc, msg))


def launch_count():
    return int(lib().aether_launch_count())


def device_status():
    return int(lib().aether_device_status())
