"""CPU ORACLE bindings — TEST INFRASTRUCTURE ONLY.

ctypes/numpy front end of ``libferrox_cpu_oracle.so`` (built from ``ferrox_cpu_oracle.cpp`` by
``make -C oracle``).  Only the test-suite, the smoke check and the CPU-baseline leg of the
benchmark may import this module; the CUDA library never does.

Besides the per-op wrappers it composes the reference's training step for a sequential
conv/linear network exactly as the reference's graph would run it (forward, softmax
cross-entropy with mean reduction, backward, optimizer step):
examples/common/training.rs:33-81, src/nn/layers/conv2d.rs:168-214,
src/nn/layers/linear.rs:183-279, src/ops/batched.rs:194-217.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from ctypes import c_int, c_int64, c_void_p

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libferrox_cpu_oracle.so")
_lib = None

ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_TANH = 0, 1, 2, 3


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file (g++, single-threaded code)."""
    src = os.path.join(_HERE, "ferrox_cpu_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libferrox_cpu_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
    return _lib


def _suf(dtype) -> str:
    dtype = np.dtype(dtype)
    if dtype == np.float32:
        return "f32"
    if dtype == np.float64:
        return "f64"
    raise TypeError(f"oracle supports float32/float64, got {dtype}")


def _p(a):
    return None if a is None else c_void_p(a.ctypes.data)


def _c(a, dtype=None):
    return np.ascontiguousarray(a, dtype=dtype)


def _scalar(dtype, v):
    return ctypes.c_float(v) if np.dtype(dtype) == np.float32 else ctypes.c_double(v)


def conv_out_hw(H, W, kh, kw, stride, pad):
    return (H + 2 * pad[0] - kh) // stride[0] + 1, (W + 2 * pad[1] - kw) // stride[1] + 1


def matmul(a, b):
    a, b = _c(a), _c(b, a.dtype)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    c = np.empty((M, N), a.dtype)
    getattr(lib(), f"orc_matmul_{_suf(a.dtype)}")(_p(a), _p(b), _p(c), c_int64(M), c_int64(N), c_int64(K))
    return c


def conv2d(x, w, stride=(1, 1), pad=(0, 0)):
    x, w = _c(x), _c(w, x.dtype)
    B, C, H, W = x.shape
    OC, C2, kh, kw = w.shape
    assert C == C2
    oh, ow = conv_out_hw(H, W, kh, kw, stride, pad)
    y = np.empty((B, OC, oh, ow), x.dtype)
    getattr(lib(), f"orc_conv2d_fwd_{_suf(x.dtype)}")(
        _p(x), _p(w), _p(y), *map(c_int64, (B, C, H, W, OC, kh, kw, stride[0], stride[1], pad[0], pad[1])))
    return y


def deconv2d(dy, w, x_shape, stride=(1, 1), pad=(0, 0), mode=1):
    """dX.  mode 1 = per-sample contract, mode 0 = the reference's literal batch>1 code."""
    dy, w = _c(dy), _c(w, dy.dtype)
    B, C, H, W = x_shape
    OC, _, kh, kw = w.shape
    dx = np.empty(tuple(x_shape), dy.dtype)
    getattr(lib(), f"orc_deconv2d_{_suf(dy.dtype)}")(
        _p(dy), _p(w), _p(dx), *map(c_int64, (B, C, H, W, OC, kh, kw, stride[0], stride[1], pad[0], pad[1])),
        c_int(mode))
    return dx


def cross_correlation2d(x, dy, w_shape, stride=(1, 1), pad=(0, 0), mode=1):
    """dW.  mode 1 = per-sample contract, mode 0 = the reference's literal batch>1 code."""
    x, dy = _c(x), _c(dy, x.dtype)
    B, C, H, W = x.shape
    OC, _, kh, kw = w_shape
    dw = np.empty(tuple(w_shape), x.dtype)
    getattr(lib(), f"orc_cross_correlation2d_{_suf(x.dtype)}")(
        _p(x), _p(dy), _p(dw), *map(c_int64, (B, C, H, W, OC, kh, kw, stride[0], stride[1], pad[0], pad[1])),
        c_int(mode))
    return dw


def act_fwd(x, act):
    x = _c(x)
    y = np.empty_like(x)
    getattr(lib(), f"orc_act_fwd_{_suf(x.dtype)}")(_p(x), _p(y), c_int64(x.size), c_int(act))
    return y


def act_bwd(dy, aux, act, sigmoid_math=False):
    """aux = op input for relu, cached op output for sigmoid/tanh (src/ops/unary.rs)."""
    dy, aux = _c(dy), _c(aux, dy.dtype)
    dx = np.empty_like(dy)
    getattr(lib(), f"orc_act_bwd_{_suf(dy.dtype)}")(_p(dy), _p(aux), _p(dx), c_int64(dy.size), c_int(act),
                                                    c_int(1 if sigmoid_math else 0))
    return dx


def sum_axes(x, axes, keep_dims=False):
    x = _c(x)
    axes = sorted({a % x.ndim for a in axes})
    shape = (c_int64 * x.ndim)(*x.shape)
    red = (c_int * x.ndim)(*[1 if i in axes else 0 for i in range(x.ndim)])
    kept = [s for i, s in enumerate(x.shape) if i not in axes]
    out = np.empty(int(np.prod(kept)) if kept else 1, x.dtype)
    getattr(lib(), f"orc_sum_axes_{_suf(x.dtype)}")(_p(x), shape, c_int(x.ndim), red, _p(out))
    if keep_dims:
        return out.reshape([1 if i in axes else s for i, s in enumerate(x.shape)])
    return out.reshape(kept)


def linear_fwd(x, w, b=None):
    x, w = _c(x), _c(w, x.dtype)
    b = None if b is None else _c(b, x.dtype)
    B, i = x.shape
    o = w.shape[0]
    y = np.empty((B, o), x.dtype)
    getattr(lib(), f"orc_linear_fwd_{_suf(x.dtype)}")(_p(x), _p(w), _p(b), _p(y), c_int64(B), c_int64(i), c_int64(o))
    return y


def linear_bwd(x, w, dz, need_dx=True):
    x, w, dz = _c(x), _c(w, x.dtype), _c(dz, x.dtype)
    B, i = x.shape
    o = w.shape[0]
    dx = np.empty((B, i), x.dtype) if need_dx else None
    dw = np.empty((o, i), x.dtype)
    db = np.empty((o,), x.dtype)
    getattr(lib(), f"orc_linear_bwd_{_suf(x.dtype)}")(_p(x), _p(w), _p(dz), _p(dx), _p(dw), _p(db),
                                                     c_int64(B), c_int64(i), c_int64(o))
    return dx, dw, db


def conv_bias_add(y, bias):
    y = _c(y).copy()
    B, K = y.shape[:2]
    P = int(np.prod(y.shape[2:]))
    getattr(lib(), f"orc_conv_bias_add_{_suf(y.dtype)}")(_p(y), _p(_c(bias, y.dtype)), c_int64(B), c_int64(K), c_int64(P))
    return y


def softmax_ce(logits, targets_onehot, need_grad=True):
    z, t = _c(logits), _c(targets_onehot, logits.dtype)
    B, C = z.shape
    g = np.empty_like(z) if need_grad else None
    fn = getattr(lib(), f"orc_softmax_ce_{_suf(z.dtype)}")
    fn.restype = ctypes.c_float if z.dtype == np.float32 else ctypes.c_double
    loss = fn(_p(z), _p(t), _p(g), c_int64(B), c_int64(C))
    return z.dtype.type(loss), g


def sgd_step(p, g, mom=None, lr=0.01, momentum=0.0, wd=0.0, nesterov=False):
    """In place on p (and mom)."""
    assert p.flags.c_contiguous
    dt = p.dtype
    getattr(lib(), f"orc_sgd_step_{_suf(dt)}")(_p(p), _p(_c(g, dt)), _p(mom), c_int64(p.size), _scalar(dt, lr),
                                              _scalar(dt, momentum), _scalar(dt, wd), c_int(int(nesterov)))


def adam_step(p, g, m, v, step, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, wd=0.0):
    """In place on p, m, v.  step is 1-based."""
    assert p.flags.c_contiguous and m.flags.c_contiguous and v.flags.c_contiguous
    dt = p.dtype
    getattr(lib(), f"orc_adam_step_{_suf(dt)}")(_p(p), _p(_c(g, dt)), _p(m), _p(v), c_int64(p.size),
                                               _scalar(dt, lr), _scalar(dt, b1), _scalar(dt, b2),
                                               _scalar(dt, eps), _scalar(dt, wd), c_int64(step))


# ----------------------------------------------------------------------------------------------
# Layout ops, batch normalisation and global average pooling: numpy restatements (pure data
# movement, or the reference's graph ops applied one after the other in the tensor's own dtype).
def materialize(data, shape, strides):
    """Contiguous copy of the view (shape, element strides; 0 = broadcast) of the flat array `data`:
    kernels/materialize.cu:25-46 (output index -> coordinates -> strided input index)."""
    data = np.asarray(data).ravel()
    idx = np.zeros(tuple(shape), np.int64)
    for ax, (n, st) in enumerate(zip(shape, strides)):
        sh = [1] * len(shape)
        sh[ax] = n
        idx = idx + (np.arange(n, dtype=np.int64) * st).reshape(sh)
    return data[idx]


def transpose(x, axes=None):
    """CPUStorage::transpose (src/backend/storage/cpu.rs:543-562): permuted axes, owned copy;
    axes=None reverses all axes."""
    return np.ascontiguousarray(np.transpose(np.asarray(x), axes))


def broadcast_to(x, shape):
    """CPUStorage::broadcast_to (src/backend/storage/cpu.rs:510-541): shapes aligned at the last axis,
    an extent must equal the target's or be 1."""
    x = np.asarray(x)
    if len(shape) < x.ndim:
        raise ValueError("Cannot broadcast to smaller number of dimensions")
    off = len(shape) - x.ndim
    for i, (c, t) in enumerate(zip(x.shape, shape[off:])):
        if c != 1 and c != t:
            raise ValueError(f"Cannot broadcast dimension {i} from size {c} to size {t}")
    return np.ascontiguousarray(np.broadcast_to(x, shape))


def _bn_axes(x):
    return [0, 2, 3] if x.ndim == 4 else [0]


def _bc(v, x):
    """reshape_and_broadcast (src/nn/layers/utils.rs:6-42): [C] -> [1, C, 1, 1] (or [1, C])."""
    return v.reshape([1, -1] + [1] * (x.ndim - 2))


def mean_axes(x, axes):
    """CPUStorage::mean (src/backend/storage/cpu.rs:1193-1221): sum, then times 1/count."""
    count = int(np.prod([x.shape[a] for a in axes]))
    return sum_axes(x, axes) * x.dtype.type(1.0 / count)


def batch_norm_fwd(x, gamma, beta, eps=1e-5, running_mean=None, running_var=None, momentum=0.1, training=True):
    """BatchNorm::apply_training_batch_norm / apply_inference_batch_norm / finish_normalization
    (src/nn/layers/norm.rs:190-331), op by op.  Training returns (y, batch_mean, batch_var) and
    updates running_mean / running_var in place (norm.rs:126-163)."""
    x = _c(x)
    dt = x.dtype.type
    axes = _bn_axes(x)
    if training:
        mean = mean_axes(x, axes)
        centered = x - _bc(mean, x)
        var = mean_axes(centered * centered, axes)
        if running_mean is not None:
            running_mean[...] = running_mean * dt(1.0 - momentum) + mean * dt(momentum)
            running_var[...] = running_var * dt(1.0 - momentum) + var * dt(momentum)
    else:
        mean, var = running_mean, running_var
        centered = x - _bc(mean, x)
    std = np.sqrt(_bc(var, x) + dt(eps))
    normalized = centered / std
    y = normalized * _bc(_c(gamma, x.dtype), x) + _bc(_c(beta, x.dtype), x)
    return (y, mean, var) if training else y


def batch_norm_bwd(x, dy, gamma, mean, var, eps=1e-5):
    """Gradients of the training-mode graph above, chained rule by rule: Add / Mul / Div
    (src/ops/basic.rs:95-115, :187-263), Sqrt (src/ops/unary.rs:123-143), AddScalar, BroadcastTo
    (src/ops/reshape.rs:82-99), Mean (src/ops/reduction.rs:170-196), Sub.  Returns (dx, dgamma, dbeta)."""
    x, dy = _c(x), _c(dy, x.dtype)
    dt = x.dtype.type
    axes = _bn_axes(x)
    m = int(np.prod([x.shape[a] for a in axes]))
    inv_m = dt(1.0 / m)
    centered = x - _bc(mean, x)
    std = np.sqrt(np.broadcast_to(_bc(var, x), x.shape) + dt(eps))
    normalized = centered / std
    gb = _bc(_c(gamma, x.dtype), x)
    dbeta = sum_axes(dy, axes)                       # Add -> BroadcastTo::gradient
    dgamma = sum_axes(dy * normalized, axes)         # Mul
    d_norm = dy * gb
    d_centered = d_norm / std                        # Div, first input
    d_std = d_norm * (-(normalized / std))           # Div, second input: grad * -(out / b)
    d_vpe = d_std / (std * dt(2.0))                  # Sqrt: grad / (2 * out)
    d_var = sum_axes(_c(d_vpe), axes)                # BroadcastTo::gradient of the variance
    d_sq = np.broadcast_to(_bc(d_var * inv_m, x), x.shape)  # Mean::gradient
    d_centered = d_centered + d_sq * centered        # Mul(centered, centered): both inputs accumulate
    d_centered = d_centered + d_sq * centered
    d_mean = sum_axes(_c(-d_centered), axes)         # Sub, second input -> BroadcastTo::gradient
    dx = d_centered + np.broadcast_to(_bc(d_mean * inv_m, x), x.shape)
    return _c(dx), dgamma, dbeta


def global_avg_pool_fwd(x, flatten=True):
    """GlobalAvgPool2d::forward (src/nn/layers/pooling.rs:604-619): Mean over axes [2, 3]."""
    x = _c(x)
    y = mean_axes(x, [2, 3])
    return y if flatten else y.reshape(x.shape[0], x.shape[1], 1, 1)


def global_avg_pool_bwd(dy, x_shape):
    """Mean::gradient (src/ops/reduction.rs:170-196): grad * (1/count), broadcast to the input shape."""
    dy = _c(dy)
    n, c, h, w = x_shape
    scaled = dy.reshape(n, c) * dy.dtype.type(1.0 / (h * w))
    return np.ascontiguousarray(np.broadcast_to(scaled.reshape(n, c, 1, 1), x_shape))


# ----------------------------------------------------------------------------------------------
# Sequential network train step, composed like the reference graph.
# layers: list of dicts
#   {"kind": "conv", "stride": s, "pad": p, "act": ACT_*}   params W [K,C,R,S], b [K]
#   {"kind": "flatten"}
#   {"kind": "linear", "act": ACT_*}                        params W [out,in], b [out]
def net_forward_backward(layers, params, x, targets_onehot):
    """Returns (loss, grads) with grads in the same order/shape as params (list of (W, b))."""
    acts = [x]
    pre = []
    pi = 0
    for L in layers:
        h = acts[-1]
        if L["kind"] == "conv":
            W, b = params[pi]; pi += 1
            z = conv2d(h, W, (L["stride"],) * 2, (L["pad"],) * 2)
            z = conv_bias_add(z, b)
            pre.append(z)
            acts.append(act_fwd(z, L["act"]) if L["act"] else z)
        elif L["kind"] == "linear":
            W, b = params[pi]; pi += 1
            z = linear_fwd(h, W, b)
            pre.append(z)
            acts.append(act_fwd(z, L["act"]) if L["act"] else z)
        else:
            pre.append(None)
            acts.append(h.reshape(h.shape[0], -1))
    loss, g = softmax_ce(acts[-1], targets_onehot)
    grads = [None] * len(params)
    for li in range(len(layers) - 1, -1, -1):
        L = layers[li]
        h_in, z, h_out = acts[li], pre[li], acts[li + 1]
        if L["kind"] == "flatten":
            g = g.reshape(h_in.shape)
            continue
        pi -= 1
        W, b = params[pi]
        if L["act"]:
            g = act_bwd(g, z if L["act"] == ACT_RELU else h_out, L["act"])
        first = li == 0
        if L["kind"] == "conv":
            s, p = (L["stride"],) * 2, (L["pad"],) * 2
            db = sum_axes(g, [3, 2, 0])
            dW = cross_correlation2d(h_in, g, W.shape, s, p, mode=1)
            grads[pi] = (dW, db)
            if not first:
                g = deconv2d(g, W, h_in.shape, s, p, mode=1)
        else:
            dx, dW, db = linear_bwd(h_in, W, g, need_dx=not first)
            grads[pi] = (dW, db)
            g = dx
    return loss, grads
