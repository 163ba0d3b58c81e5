"""ctypes binding of libferrox_b200.so — the same symbols a Ferrox build would bind from Rust.

The library is built in-tree by ``python -m ferrox_b200.build``.  Importing this module never
falls back to another implementation: a missing library or symbol raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_double, c_float, c_int, c_int64, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libferrox_b200.so")

FXB_OK = 0
ERR_INVALID_ARGUMENT, ERR_UNSUPPORTED, ERR_LAUNCH_FAILED, ERR_DEVICE_TIMEOUT, ERR_CUDA, ERR_WORKSPACE = 1, 2, 3, 4, 5, 6
ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_TANH = 0, 1, 2, 3
MATH_3XTF32, MATH_TF32 = 0, 1


class Conv2dDesc(Structure):
    _fields_ = [(n, c_int64) for n in ("N", "C", "H", "W", "K", "R", "S", "stride_h", "stride_w", "pad_h", "pad_w")]


class LayerDesc(Structure):
    _fields_ = [("kind", ctypes.c_int32), ("act", ctypes.c_int32), ("out_channels", c_int64), ("kernel", c_int64),
                ("stride", c_int64), ("pad", c_int64)]


LAYER_CONV, LAYER_FLATTEN, LAYER_LINEAR = 0, 1, 2


class FerroxB200Error(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


_P = c_void_p
_DP = POINTER(Conv2dDesc)


def _sigs(real):
    """name -> (restype, argtypes) for one dtype; `real` is c_float or c_double."""
    H, S, I64, I, SZ = c_void_p, c_void_p, c_int64, c_int, c_size_t
    return {
        "matmul": (I, [H, _P, _P, _P, I64, I64, I64, S]),
        "gemm": (I, [H, I, I, I64, I64, I64, _P, I64, _P, I64, _P, I64, _P, I, _P, SZ, S]),
        "linear_fwd": (I, [H, _P, _P, _P, _P, I64, I64, I64, I, S]),
        "linear_fwd_ws": (I, [H, _P, _P, _P, _P, I64, I64, I64, I, _P, SZ, S]),
        "linear_bwd": (I, [H, _P, _P, _P, _P, _P, _P, _P, I64, I64, I64, I, _P, SZ, S]),
        "conv2d_forward": (I, [H, _P, _P, _P, _DP, _P, SZ, S]),
        "conv2d_bias_act_fwd": (I, [H, _P, _P, _P, _P, _DP, I, _P, SZ, S]),
        "deconv2d": (I, [H, _P, _P, _P, _DP, _P, SZ, S]),
        "conv2d_dgrad_act": (I, [H, _P, _P, _P, _P, _DP, I, _P, SZ, S]),
        "cross_correlation2d": (I, [H, _P, _P, _P, _DP, _P, SZ, S]),
        "conv2d_wgrad_bias_act": (I, [H, _P, _P, _P, _P, _P, _DP, I, _P, SZ, S]),
        "conv2d_backward": (I, [H, _P, _P, _P, _P, _P, _P, _P, _DP, I, _P, SZ, _P, S]),
        "act_fwd": (I, [H, _P, _P, I64, I, S]),
        "act_bwd": (I, [H, _P, _P, _P, I64, I, S]),
        "add": (I, [H, _P, _P, _P, I64, S]),
        "mul": (I, [H, _P, _P, _P, I64, S]),
        "axpby": (I, [H, real, _P, real, _P, _P, I64, S]),
        "greater_scalar": (I, [H, _P, real, _P, I64, S]),
        "bias_add": (I, [H, _P, _P, I64, I64, I64, S]),
        "sum_axes": (I, [H, _P, POINTER(c_int64), I, POINTER(c_int), I, _P, _P, SZ, S]),
        "sum_all": (I, [H, _P, I64, _P, _P, SZ, S]),
        "softmax_ce": (I, [H, _P, _P, _P, _P, I64, I64, real, S]),
        "sgd_step": (I, [H, _P, _P, _P, I64, real, real, real, I, real, S]),
        "adam_step": (I, [H, _P, _P, _P, _P, I64, real, real, real, real, real, I64, real, S]),
        "adam_step_devcount": (I, [H, _P, _P, _P, _P, I64, real, real, real, real, real, _P, real, S]),
        "materialize": (I, [H, _P, _P, POINTER(c_int64), POINTER(c_int64), I, S]),
        "transpose": (I, [H, _P, _P, POINTER(c_int64), I, POINTER(c_int), S]),
        "broadcast_to": (I, [H, _P, POINTER(c_int64), I, _P, POINTER(c_int64), I, S]),
        "batch_norm_fwd": (I, [H, _P, _P, _P, _P, _P, _P, _P, _P, I64, I64, I64, c_double, c_double, I, I, _P, SZ, S]),
        "batch_norm_bwd": (I, [H, _P, _P, _P, _P, _P, _P, _P, _P, _P, I64, I64, I64, c_double, I, _P, SZ, S]),
        "global_avg_pool_fwd": (I, [H, _P, _P, I64, I64, I64, I64, S]),
        "global_avg_pool_bwd": (I, [H, _P, _P, I64, I64, I64, I64, S]),
    }


_COMMON = {
    "fxb_create": (c_int, [c_int, POINTER(c_void_p)]),
    "fxb_destroy": (c_int, [c_void_p]),
    "fxb_last_error": (c_char_p, [c_void_p]),
    "fxb_status_string": (c_char_p, [c_int]),
    "fxb_set_math_mode": (c_int, [c_void_p, c_int]),
    "fxb_set_operand_path": (c_int, [c_void_p, c_int]),
    "fxb_set_accumulate_stages": (c_int, [c_void_p, c_int]),
    "fxb_set_sigmoid_grad_mode": (c_int, [c_void_p, c_int]),
    "fxb_check_device_status": (c_int, [c_void_p, c_void_p]),
    "fxb_selftest_bounded_wait": (c_int, [c_void_p, c_int64, c_void_p]),
    "fxb_version": (c_int, []),
    "fxb_launch_count": (ctypes.c_uint64, [c_void_p]),
    "fxb_gemm_workspace_bytes": (c_size_t, [c_void_p, c_int64, c_int64, c_int64, c_size_t]),
    "fxb_linear_bwd_workspace_bytes": (c_size_t, [c_void_p, c_int64, c_int64, c_int64, c_size_t]),
    "fxb_linear_fwd_workspace_bytes": (c_size_t, [c_void_p, c_int64, c_int64, c_int64, c_size_t]),
    "fxb_conv2d_wgrad_workspace_bytes": (c_size_t, [c_void_p, _DP, c_size_t]),
    "fxb_conv2d_fprop_workspace_bytes": (c_size_t, [c_void_p, _DP, c_size_t]),
    "fxb_conv2d_fprop_prepass_f32": (c_int, [c_void_p, c_void_p, c_void_p, _DP, c_void_p, c_size_t, c_void_p]),
    "fxb_conv2d_fprop_main_f32": (c_int, [c_void_p, c_void_p, c_void_p, _DP, c_int, c_void_p, c_size_t, c_void_p]),
    "fxb_conv2d_dgrad_workspace_bytes": (c_size_t, [c_void_p, _DP, c_size_t]),
    "fxb_conv2d_backward_workspace_bytes": (c_size_t, [c_void_p, _DP, c_size_t]),
    "fxb_conv2d_packed_input_bytes": (c_size_t, [c_void_p, _DP, c_size_t]),
    "fxb_conv2d_bias_act_fwd_packing_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, _DP, c_int, c_void_p, c_size_t,
                                                    c_void_p, c_size_t, POINTER(c_int), c_void_p]),
    "fxb_conv2d_bias_act_fwd_chain_f32": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, _DP, c_int, c_void_p, c_size_t,
                                                  c_void_p, c_size_t, POINTER(c_int), c_void_p, _DP, c_void_p, c_size_t,
                                                  POINTER(c_int), c_void_p]),
    "fxb_conv2d_input_slab_bytes": (c_size_t, [c_void_p, _DP, c_size_t]),
    "fxb_batch_norm_workspace_bytes": (c_size_t, [c_void_p, c_int64, c_int64, c_int64, c_size_t]),
    "fxb_sum_axes_workspace_bytes": (c_size_t, [c_void_p, POINTER(c_int64), c_int, POINTER(c_int), c_int, c_size_t]),
    "fxb_sum_axes_static_scratch_f32": (c_int, [c_void_p, c_void_p, POINTER(c_int64), c_int, POINTER(c_int), c_int, c_void_p,
                                                c_void_p]),
    "fxb_net_create": (c_int, [c_void_p, c_size_t, POINTER(LayerDesc), c_int, c_int64, c_int64, c_int64, c_int64,
                               POINTER(c_void_p)]),
    "fxb_net_destroy": (c_int, [c_void_p]),
    "fxb_net_param_count": (c_int64, [c_void_p]),
    "fxb_net_param_layers": (c_int, [c_void_p]),
    "fxb_net_param_offsets": (c_int, [c_void_p, c_int, POINTER(c_int64), POINTER(c_int64), POINTER(c_int64)]),
    "fxb_net_arena_bytes": (c_size_t, [c_void_p]),
    "fxb_net_num_classes": (c_int64, [c_void_p]),
    "fxb_net_bind": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_size_t]),
    "fxb_net_forward": (c_int, [c_void_p, c_void_p, POINTER(c_void_p), c_void_p]),
    "fxb_net_loss": (c_int, [c_void_p, c_void_p, c_void_p, c_double, c_void_p]),
    "fxb_net_backward_range": (c_int, [c_void_p, c_void_p, c_int, c_int, c_void_p]),
}


def exported_symbols():
    """Every symbol include/ferrox_b200.h declares."""
    names = list(_COMMON)
    for suf, real in (("f32", c_float), ("f64", c_double)):
        names += [f"fxb_{n}_{suf}" for n in _sigs(real)]
    return names


_lib = None


def load():
    """Loads the shared library and declares every prototype.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FerroxB200Error(ERR_UNSUPPORTED,
                              f"{LIB_PATH} is missing: build it with `python -m ferrox_b200.build` "
                              "(there is no fallback implementation)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in _COMMON.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    for suf, real in (("f32", c_float), ("f64", c_double)):
        for n, (res, args) in _sigs(real).items():
            fn = getattr(lib, f"fxb_{n}_{suf}")
            fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib
