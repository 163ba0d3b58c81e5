"""Host-side mirror of Ferrox's `CudaOps<T>` (src/backend/cuda/ops.rs:23-38) over the C ABI.

Each method has the name, argument meaning and error behaviour of the reference method it
stands for: it validates shapes, takes the output from the pool (here torch's caching
allocator stands in for Ferrox's bucketed pool — the library itself never allocates) and makes
one C-ABI call on the current stream.  Errors come back as `FerroxB200Error(message)`, the
counterpart of the reference's `Err(String)`.

torch is used for device memory and streams only; every computation is a call into
libferrox_b200.so.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_int64, c_void_p

import torch

from . import _cabi
from ._cabi import ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_TANH, Conv2dDesc, FerroxB200Error

_ACT_NAMES = {None: ACT_NONE, "none": ACT_NONE, "relu": ACT_RELU, "sigmoid": ACT_SIGMOID, "tanh": ACT_TANH}


def act_code(act) -> int:
    if isinstance(act, int):
        return act
    return _ACT_NAMES[act]


def _ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


class CudaOps:
    """One instance per device (the reference keeps one per dtype; dtype is per call here)."""

    def __init__(self, device: int | None = None):
        if not torch.cuda.is_available():
            raise FerroxB200Error(_cabi.ERR_CUDA, "CUDA is not available: ferrox_b200 has no CPU path")
        self.lib = _cabi.load()
        self.device = torch.cuda.current_device() if device is None else int(device)
        h = c_void_p()
        rc = self.lib.fxb_create(self.device, ctypes.byref(h))
        if rc != 0:
            raise FerroxB200Error(rc, self.lib.fxb_last_error(None).decode())
        self.h = h
        self._ws = None
        # conv forward / input gradient: hand the library a workspace (pre-split cp.async path) or not
        # (operands gathered and split inside the kernel); both give the same values
        self._use_workspace = True

    def close(self):
        if getattr(self, "h", None):
            self.lib.fxb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ plumbing
    def _stream(self):
        return c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _check(self, rc):
        if rc != 0:
            raise FerroxB200Error(rc, self.lib.fxb_last_error(self.h).decode())

    def _fn(self, name, t):
        if t.dtype == torch.float32:
            return getattr(self.lib, f"fxb_{name}_f32")
        if t.dtype == torch.float64:
            return getattr(self.lib, f"fxb_{name}_f64")
        raise FerroxB200Error(_cabi.ERR_UNSUPPORTED, f"ferrox_b200 supports f32 and f64 tensors, got {t.dtype}")

    def _get_tensor(self, shape, like):
        # counterpart of CudaOps::get_tensor (ops.rs:121-133): uninitialised pool memory
        return torch.empty(tuple(shape), dtype=like.dtype, device=like.device)

    def _in(self, t):
        if not t.is_cuda:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, "tensor is not on a CUDA device")
        return t if t.is_contiguous() else t.contiguous()  # the reference materialises first

    def workspace(self, nbytes, device):
        if nbytes == 0:
            return None, 0
        if self._ws is None or self._ws.numel() < nbytes + 256 or self._ws.device != device:
            self._ws = torch.empty(max(nbytes, 1 << 20) + 256, dtype=torch.uint8, device=device)
        off = (-self._ws.data_ptr()) % 256  # the library wants 256-byte alignment
        view = self._ws[off:]
        return view, view.numel()

    @property
    def use_workspace(self):
        return self._use_workspace

    @use_workspace.setter
    def use_workspace(self, on):
        self._use_workspace = bool(on)
        self._check(self.lib.fxb_set_operand_path(self.h, 0 if on else 1))

    def set_operand_path(self, path: str):
        """'auto' (tensor-map copies where the shapes allow, else cp.async), 'cp_async', or 'gather'."""
        code = {"auto": 0, "gather": 1, "cp_async": 2}[path]
        self._use_workspace = code != 1
        self._check(self.lib.fxb_set_operand_path(self.h, code))

    def set_accumulate_stages(self, stages: int):
        """K stages (of 32) the f32 convolution kernels accumulate in TMEM between two drains: 1, 2 or 4."""
        self._check(self.lib.fxb_set_accumulate_stages(self.h, int(stages)))

    def set_math_mode(self, mode):
        self._check(self.lib.fxb_set_math_mode(self.h, mode))

    def set_sigmoid_grad_mode(self, math_mode: bool):
        self._check(self.lib.fxb_set_sigmoid_grad_mode(self.h, 1 if math_mode else 0))

    def launch_count(self) -> int:
        return int(self.lib.fxb_launch_count(self.h))

    def check_device_status(self):
        self._check(self.lib.fxb_check_device_status(self.h, self._stream()))

    def selftest_bounded_wait(self, limit_cycles=1_000_000):
        """Launches the library's bounded-wait self-test kernel (a wait that must run out)."""
        self._check(self.lib.fxb_selftest_bounded_wait(self.h, int(limit_cycles), self._stream()))

    @staticmethod
    def _desc(x_shape, w_shape, stride, padding):
        N, C, H, W = x_shape
        K, _, R, S = w_shape
        return Conv2dDesc(N, C, H, W, K, R, S, stride[0], stride[1], padding[0], padding[1])

    @staticmethod
    def conv_out_shape(x_shape, w_shape, stride, padding):
        N, _, H, W = x_shape
        K, _, R, S = w_shape
        return (N, K, (H + 2 * padding[0] - R) // stride[0] + 1, (W + 2 * padding[1] - S) // stride[1] + 1)

    # ------------------------------------------------------------------ reference op surface
    def matmul(self, a, b):
        """CudaOps::matmul (ops.rs:841-889)."""
        a, b = self._in(a), self._in(b)
        if a.dim() != 2 or b.dim() != 2:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, "Matrix multiplication requires 2D tensors")
        if a.shape[1] != b.shape[0]:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT,
                                  f"Matrix multiplication shape mismatch: ({a.shape[0]}, {a.shape[1]}) @ ({b.shape[0]}, {b.shape[1]})")
        out = self._get_tensor((a.shape[0], b.shape[1]), a)
        M, N, K = a.shape[0], b.shape[1], a.shape[1]
        nb = self.lib.fxb_gemm_workspace_bytes(self.h, M, N, K, a.element_size()) if M * N * K >= 1 << 24 else 0
        if nb:
            # large products: the general entry point with a pool workspace (split-K / tensor-map engine)
            ws, wsb = self.workspace(nb, a.device)
            self._check(self._fn("gemm", a)(self.h, 0, 0, M, N, K, _ptr(a), K, _ptr(b), N, _ptr(out), N, None, 0, _ptr(ws),
                                            wsb, self._stream()))
            return out
        self._check(self._fn("matmul", a)(self.h, _ptr(a), _ptr(b), _ptr(out), M, N, K, self._stream()))
        return out

    def gemm(self, a, b, trans_a=False, trans_b=False, bias=None, act=None):
        """op(A).op(B) with transposed views instead of materialised transposes."""
        a, b = self._in(a), self._in(b)
        M, K = (a.shape[1], a.shape[0]) if trans_a else a.shape
        K2, N = (b.shape[1], b.shape[0]) if trans_b else b.shape
        if K != K2:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, f"Matrix multiplication shape mismatch: ({M}, {K}) @ ({K2}, {N})")
        out = self._get_tensor((M, N), a)
        nb = self.lib.fxb_gemm_workspace_bytes(self.h, M, N, K, a.element_size())
        ws, wsb = self.workspace(nb, a.device)
        self._check(self._fn("gemm", a)(self.h, int(trans_a), int(trans_b), M, N, K, _ptr(a), a.shape[1], _ptr(b),
                                        b.shape[1], _ptr(out), N, _ptr(bias), act_code(act), _ptr(ws), wsb, self._stream()))
        return out

    def conv2d_forward(self, x, w, stride, padding, bias=None, act=None):
        """CudaOps::conv2d_forward (ops.rs:1202-1298); bias/act select the fused epilogue."""
        x, w = self._in(x), self._in(w)
        if x.dim() != 4 or w.dim() != 4:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, "Conv2D requires 4D tensors [batch, channels, height, width]")
        if x.shape[1] != w.shape[1]:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT,
                                  f"Input channels {x.shape[1]} don't match filter channels {w.shape[1]}")
        if x.shape[2] + 2 * padding[0] < w.shape[2] or x.shape[3] + 2 * padding[1] < w.shape[3]:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, "Conv2D filter larger than the padded input")
        d = self._desc(x.shape, w.shape, stride, padding)
        out = self._get_tensor(self.conv_out_shape(x.shape, w.shape, stride, padding), x)
        nb = self.lib.fxb_conv2d_fprop_workspace_bytes(self.h, ctypes.byref(d), x.element_size()) if self.use_workspace else 0
        ws, wsb = self.workspace(nb, x.device)
        if bias is None and act_code(act) == ACT_NONE:
            self._check(self._fn("conv2d_forward", x)(self.h, _ptr(x), _ptr(w), _ptr(out), ctypes.byref(d), _ptr(ws), wsb,
                                                      self._stream()))
        else:
            self._check(self._fn("conv2d_bias_act_fwd", x)(self.h, _ptr(x), _ptr(w), _ptr(bias), _ptr(out), ctypes.byref(d),
                                                           act_code(act), _ptr(ws), wsb, self._stream()))
        return out

    def conv2d_forward_prepass(self, x, w, stride, padding):
        """Only the operand pre-pass of the f32 conv2d_forward (for timing the two parts separately)."""
        x, w = self._in(x), self._in(w)
        d = self._desc(x.shape, w.shape, stride, padding)
        nb = self.lib.fxb_conv2d_fprop_workspace_bytes(self.h, ctypes.byref(d), x.element_size())
        ws, wsb = self.workspace(nb, x.device)
        self._check(self.lib.fxb_conv2d_fprop_prepass_f32(self.h, _ptr(x), _ptr(w), ctypes.byref(d), _ptr(ws), wsb, self._stream()))

    def conv2d_forward_main(self, x_shape, w_shape, stride, padding, bias=None, act=None, like=None):
        """Only the contraction kernel of the f32 conv2d_forward, on the operands the last
        conv2d_forward_prepass call for the same shapes left in the workspace."""
        d = self._desc(x_shape, w_shape, stride, padding)
        like = bias if like is None else like
        out = self._get_tensor(self.conv_out_shape(x_shape, w_shape, stride, padding), like)
        nb = self.lib.fxb_conv2d_fprop_workspace_bytes(self.h, ctypes.byref(d), 4)
        ws, wsb = self.workspace(nb, like.device)
        self._check(self.lib.fxb_conv2d_fprop_main_f32(self.h, _ptr(bias), _ptr(out), ctypes.byref(d), act_code(act), _ptr(ws), wsb,
                                                       self._stream()))
        return out

    def deconv2d(self, dy, w, input_shape, stride, padding, y=None, act=None):
        """CudaOps::deconv2d (ops.rs:1458-1539): gradient w.r.t. the conv input."""
        dy, w = self._in(dy), self._in(w)
        if dy.dim() != 4 or w.dim() != 4 or len(input_shape) != 4:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, "Conv2d backward requires 4D tensors")
        d = self._desc(input_shape, w.shape, stride, padding)
        out = self._get_tensor(input_shape, dy)
        nb = self.lib.fxb_conv2d_dgrad_workspace_bytes(self.h, ctypes.byref(d), dy.element_size()) if self.use_workspace else 0
        ws, wsb = self.workspace(nb, dy.device)
        if act_code(act) == ACT_NONE:
            self._check(self._fn("deconv2d", dy)(self.h, _ptr(dy), _ptr(w), _ptr(out), ctypes.byref(d), _ptr(ws), wsb,
                                                 self._stream()))
        else:
            self._check(self._fn("conv2d_dgrad_act", dy)(self.h, _ptr(dy), _ptr(self._in(y)), _ptr(w), _ptr(out),
                                                         ctypes.byref(d), act_code(act), _ptr(ws), wsb, self._stream()))
        return out

    def cross_correlation2d(self, x, dy, output_shape, stride, padding, y=None, act=None, want_bias_grad=False):
        """CudaOps::cross_correlation2d (ops.rs:1544-1622): gradient w.r.t. the filter."""
        x, dy = self._in(x), self._in(dy)
        if x.dim() != 4 or dy.dim() != 4 or len(output_shape) != 4:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, "Cross correlation requires 4D tensors")
        d = self._desc(x.shape, output_shape, stride, padding)
        out = self._get_tensor(output_shape, x)
        nb = self.lib.fxb_conv2d_wgrad_workspace_bytes(self.h, ctypes.byref(d), x.element_size())
        ws, wsb = self.workspace(nb, x.device)
        if act_code(act) == ACT_NONE and not want_bias_grad:
            self._check(self._fn("cross_correlation2d", x)(self.h, _ptr(x), _ptr(dy), _ptr(out), ctypes.byref(d), _ptr(ws),
                                                           wsb, self._stream()))
            return out
        db = self._get_tensor((output_shape[0],), x) if want_bias_grad else None
        self._check(self._fn("conv2d_wgrad_bias_act", x)(self.h, _ptr(x), _ptr(dy), _ptr(None if y is None else self._in(y)),
                                                         _ptr(out), _ptr(db), ctypes.byref(d), act_code(act), _ptr(ws), wsb,
                                                         self._stream()))
        return (out, db) if want_bias_grad else out

    def conv2d_forward_packing(self, x, w, stride, padding, bias=None, act=None):
        """conv2d_forward that also packs the layer input for the filter gradient of the same layer.
        Returns (y, packed) with packed = None when the shape has no packed form."""
        x, w = self._in(x), self._in(w)
        d = self._desc(x.shape, w.shape, stride, padding)
        out = self._get_tensor(self.conv_out_shape(x.shape, w.shape, stride, padding), x)
        nb = self.lib.fxb_conv2d_fprop_workspace_bytes(self.h, ctypes.byref(d), x.element_size())
        ws, wsb = self.workspace(nb, x.device)
        pb = self.lib.fxb_conv2d_packed_input_bytes(self.h, ctypes.byref(d), x.element_size()) if x.dtype == torch.float32 else 0
        if pb == 0:
            return self.conv2d_forward(x, w, stride, padding, bias, act), None
        packed = torch.empty(pb + 256, dtype=torch.uint8, device=x.device)
        packed = packed[(-packed.data_ptr()) % 256:]
        written = c_int(0)
        self._check(self.lib.fxb_conv2d_bias_act_fwd_packing_f32(self.h, _ptr(x), _ptr(w), _ptr(bias), _ptr(out), ctypes.byref(d),
                                                                 act_code(act), _ptr(ws), wsb, _ptr(packed), pb,
                                                                 ctypes.byref(written), self._stream()))
        return out, (packed if written.value else None)

    def conv2d_input_slabs(self, x_shape, w_shape, stride, padding, device):
        """A zeroed buffer for the class slabs of a convolution's input (None when the layer reads none): what a
        producing layer's conv2d_forward_chain writes and the consuming layer's reads."""
        d = self._desc(x_shape, w_shape, stride, padding)
        nb = self.lib.fxb_conv2d_input_slab_bytes(self.h, ctypes.byref(d), 4)
        if nb == 0:
            return None
        buf = torch.zeros(nb + 256, dtype=torch.uint8, device=device)
        return buf[(-buf.data_ptr()) % 256:]

    def conv2d_forward_chain(self, x, w, stride, padding, bias=None, act=None, in_slabs=None, next_w_shape=None,
                             next_stride=None, next_padding=None, out_slabs=None):
        """f32 conv2d_forward for consecutive convolution layers: `in_slabs` = this layer's input slabs as written
        by the previous layer's call; with the next layer's filter shape / stride / padding and `out_slabs`
        (conv2d_input_slabs of that layer) the epilogue also writes the next layer's slabs.
        Returns (y, out_slabs_written)."""
        x, w = self._in(x), self._in(w)
        d = self._desc(x.shape, w.shape, stride, padding)
        oshape = self.conv_out_shape(x.shape, w.shape, stride, padding)
        out = self._get_tensor(oshape, x)
        nb = self.lib.fxb_conv2d_fprop_workspace_bytes(self.h, ctypes.byref(d), x.element_size())
        ws, wsb = self.workspace(nb, x.device)
        nd = self._desc(oshape, next_w_shape, next_stride, next_padding) if next_w_shape is not None else None
        written = c_int(0)
        self._check(self.lib.fxb_conv2d_bias_act_fwd_chain_f32(
            self.h, _ptr(x), _ptr(w), _ptr(bias), _ptr(out), ctypes.byref(d), act_code(act), _ptr(ws), wsb, None, 0, None,
            _ptr(in_slabs), ctypes.byref(nd) if nd is not None else None, _ptr(out_slabs),
            0 if out_slabs is None else out_slabs.numel(), ctypes.byref(written), self._stream()))
        return out, bool(written.value)

    def conv2d_backward(self, x, dy, w, stride, padding, y=None, act=None, need_dx=True, need_db=True, packed=None):
        """Conv2dOp::gradient (src/ops/batched.rs:194-217) in one call: (dX, dW, db) of the fused
        conv + bias + activation layer, with one operand pass over dY."""
        x, dy, w = self._in(x), self._in(dy), self._in(w)
        d = self._desc(x.shape, w.shape, stride, padding)
        dx = self._get_tensor(x.shape, x) if need_dx else None
        dw = self._get_tensor(w.shape, x)
        db = self._get_tensor((w.shape[0],), x) if need_db else None
        nb = self.lib.fxb_conv2d_backward_workspace_bytes(self.h, ctypes.byref(d), x.element_size())
        ws, wsb = self.workspace(nb, x.device)
        self._check(self._fn("conv2d_backward", x)(self.h, _ptr(x), _ptr(dy), _ptr(None if y is None else self._in(y)), _ptr(w),
                                                   _ptr(dx), _ptr(dw), _ptr(db), ctypes.byref(d), act_code(act), _ptr(ws), wsb,
                                                   _ptr(packed), self._stream()))
        return dx, dw, db

    def _act_fwd(self, x, code):
        x = self._in(x)
        out = self._get_tensor(x.shape, x)
        self._check(self._fn("act_fwd", x)(self.h, _ptr(x), _ptr(out), x.numel(), code, self._stream()))
        return out

    def relu(self, x):
        """CudaOps::relu (ops.rs:539-547)."""
        return self._act_fwd(x, ACT_RELU)

    def sigmoid(self, x):
        """CudaOps::sigmoid (ops.rs:550-558)."""
        return self._act_fwd(x, ACT_SIGMOID)

    def tanh(self, x):
        """CudaOps::tanh (ops.rs:620-628)."""
        return self._act_fwd(x, ACT_TANH)

    def act_backward(self, dy, aux, act):
        """dY * act'(aux): the fused form of ReLU/Sigmoid/Tanh::gradient (src/ops/unary.rs:254-375)."""
        dy, aux = self._in(dy), self._in(aux)
        if dy.shape != aux.shape:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, "activation backward: shape mismatch")
        out = self._get_tensor(dy.shape, dy)
        self._check(self._fn("act_bwd", dy)(self.h, _ptr(dy), _ptr(aux), _ptr(out), dy.numel(), act_code(act), self._stream()))
        return out

    def _binary(self, name, a, b):
        a, b = self._in(a), self._in(b)
        if a.shape != b.shape:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, f"Shape mismatch: {list(a.shape)} vs {list(b.shape)}")
        out = self._get_tensor(a.shape, a)
        self._check(self._fn(name, a)(self.h, _ptr(a), _ptr(b), _ptr(out), a.numel(), self._stream()))
        return out

    def add(self, a, b):
        """CudaOps::add (ops.rs:217)."""
        return self._binary("add", a, b)

    def mul(self, a, b):
        """CudaOps::mul (ops.rs:244)."""
        return self._binary("mul", a, b)

    def axpby(self, alpha, x, beta, y):
        x = self._in(x)
        out = self._get_tensor(x.shape, x)
        self._check(self._fn("axpby", x)(self.h, alpha, _ptr(x), beta, _ptr(None if y is None else self._in(y)), _ptr(out),
                                         x.numel(), self._stream()))
        return out

    def greater_scalar(self, x, s):
        """CudaOps::greater_scalar (ops.rs:1052): 1.0 where x > s else 0.0."""
        x = self._in(x)
        out = self._get_tensor(x.shape, x)
        self._check(self._fn("greater_scalar", x)(self.h, _ptr(x), s, _ptr(out), x.numel(), self._stream()))
        return out

    def bias_add_(self, y, bias):
        """In place y[n,k,...] += bias[k] (the unfused BroadcastTo + Add)."""
        assert y.is_contiguous()
        outer, ch = y.shape[0], y.shape[1]
        plane = y.numel() // max(1, outer * ch)
        self._check(self._fn("bias_add", y)(self.h, _ptr(y), _ptr(bias), outer, ch, plane, self._stream()))
        return y

    def sum_axes(self, x, axes, keep_dims=False):
        """CudaOps::sum_axes (ops.rs:670-697)."""
        x = self._in(x)
        axes = list(axes)
        for ax in axes:
            if ax >= x.dim() or ax < 0:
                raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT,
                                      f"Axis {ax} is out of bounds for tensor with {x.dim()} dimensions")
        shape = (c_int64 * max(1, x.dim()))(*x.shape)
        ax = (c_int * max(1, len(axes)))(*axes)
        kept = [s for i, s in enumerate(x.shape) if i not in axes]
        out = self._get_tensor(kept, x)
        nb = self.lib.fxb_sum_axes_workspace_bytes(self.h, shape, x.dim(), ax, len(axes), x.element_size())
        ws, wsb = self.workspace(nb, x.device)
        self._check(self._fn("sum_axes", x)(self.h, _ptr(x), shape, x.dim(), ax, len(axes), _ptr(out), _ptr(ws), wsb,
                                            self._stream()))
        if keep_dims:
            out = out.reshape([1 if i in axes else s for i, s in enumerate(x.shape)])
        return out

    def sum_all(self, x):
        """CudaOps::sum_all (ops.rs:653-667); returns a 0-d tensor."""
        x = self._in(x)
        out = self._get_tensor((), x)
        shape = (c_int64 * 1)(x.numel())
        ax = (c_int * 1)(0)
        nb = self.lib.fxb_sum_axes_workspace_bytes(self.h, shape, 1, ax, 1, x.element_size())
        ws, wsb = self.workspace(nb, x.device)
        self._check(self._fn("sum_all", x)(self.h, _ptr(x), x.numel(), _ptr(out), _ptr(ws), wsb, self._stream()))
        return out

    # ------------------------------------------------------------------ layout ops
    def materialize(self, t):
        """CudaOps::materialize (ops.rs:175-214): a strided / broadcast view (any torch view whose strides
        are non-negative) copied into new contiguous memory by the library's layout kernels."""
        if not t.is_cuda:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, "tensor is not on a CUDA device")
        out = self._get_tensor(t.shape, t)
        nd = max(1, t.dim())
        shape = (c_int64 * nd)(*t.shape)
        strides = (c_int64 * nd)(*t.stride())
        self._check(self._fn("materialize", t)(self.h, _ptr(t), _ptr(out), shape, strides, t.dim(), self._stream()))
        return out

    def transpose(self, x, axes=None):
        """Transpose::compute (src/ops/matrix.rs:69-110) followed by the materialisation every consumer
        triggers: the permuted tensor in contiguous memory.  axes=None reverses all axes."""
        x = self._in(x)
        nd = x.dim()
        perm = list(range(nd - 1, -1, -1)) if axes is None else list(axes)
        if sorted(perm) != list(range(nd)):
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, f"transpose: axes must be a permutation of 0..{nd - 1}")
        out = self._get_tensor([x.shape[a] for a in perm], x)
        shape = (c_int64 * max(1, nd))(*x.shape)
        ax = None if axes is None else (c_int * max(1, nd))(*perm)
        self._check(self._fn("transpose", x)(self.h, _ptr(x), _ptr(out), shape, nd, ax, self._stream()))
        return out

    def broadcast_to(self, x, shape):
        """broadcast_to + materialize (src/backend/storage/cuda.rs:795-803)."""
        x = self._in(x)
        shape = list(shape)
        if x.dim() > len(shape):
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, "broadcast_to: the target must have at least as many dimensions")
        out = self._get_tensor(shape, x)
        ins = (c_int64 * max(1, x.dim()))(*x.shape)
        outs = (c_int64 * max(1, len(shape)))(*shape)
        self._check(self._fn("broadcast_to", x)(self.h, _ptr(x), ins, x.dim(), _ptr(out), outs, len(shape), self._stream()))
        return out

    # ------------------------------------------------------------------ normalisation and pooling
    @staticmethod
    def _ncp(x):
        if x.dim() < 2:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, "BatchNorm requires at least 2D input [batch_size, features]")
        n, ch = x.shape[0], x.shape[1]
        return n, ch, x.numel() // max(1, n * ch)

    def batch_norm_forward(self, x, gamma, beta, eps=1e-5, momentum=0.1, running_mean=None, running_var=None, training=True,
                           act=None):
        """BatchNorm::forward (src/nn/layers/norm.rs:214-331).  Training returns (y, batch_mean, batch_var)
        and updates the running statistics in place when given; inference returns y."""
        x = self._in(x)
        n, ch, p = self._ncp(x)
        y = self._get_tensor(x.shape, x)
        if training:
            mean, var = self._get_tensor((ch,), x), self._get_tensor((ch,), x)
            nb = self.lib.fxb_batch_norm_workspace_bytes(self.h, n, ch, p, x.element_size())
            ws, wsb = self.workspace(nb, x.device)
        else:
            mean = var = ws = None
            wsb = 0
        self._check(self._fn("batch_norm_fwd", x)(self.h, _ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), _ptr(mean), _ptr(var),
                                                  _ptr(running_mean), _ptr(running_var), n, ch, p, eps, momentum, int(training),
                                                  act_code(act), _ptr(ws), wsb, self._stream()))
        return (y, mean, var) if training else y

    def batch_norm_backward(self, x, dy, gamma, batch_mean, batch_var, eps=1e-5, y=None, act=None, need_dx=True):
        """(dX, dgamma, dbeta) of the fused batch-norm (+ activation) layer."""
        x, dy = self._in(x), self._in(dy)
        n, ch, p = self._ncp(x)
        dx = self._get_tensor(x.shape, x) if need_dx else None
        dg, db = self._get_tensor((ch,), x), self._get_tensor((ch,), x)
        nb = self.lib.fxb_batch_norm_workspace_bytes(self.h, n, ch, p, x.element_size())
        ws, wsb = self.workspace(nb, x.device)
        self._check(self._fn("batch_norm_bwd", x)(self.h, _ptr(x), _ptr(dy), _ptr(None if y is None else self._in(y)), _ptr(gamma),
                                                  _ptr(batch_mean), _ptr(batch_var), _ptr(dx), _ptr(dg), _ptr(db), n, ch, p, eps,
                                                  act_code(act), _ptr(ws), wsb, self._stream()))
        return dx, dg, db

    def global_avg_pool_forward(self, x, flatten=True):
        """GlobalAvgPool2d::forward (src/nn/layers/pooling.rs:604-619): [N,C,H,W] -> [N,C] (or [N,C,1,1])."""
        x = self._in(x)
        if x.dim() != 4:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT, "GlobalAvgPool2d requires 4D input [batch, channels, height, width]")
        n, ch, hh, ww = x.shape
        y = self._get_tensor((n, ch) if flatten else (n, ch, 1, 1), x)
        self._check(self._fn("global_avg_pool_fwd", x)(self.h, _ptr(x), _ptr(y), n, ch, hh, ww, self._stream()))
        return y

    def global_avg_pool_backward(self, dy, input_shape):
        dy = self._in(dy)
        n, ch, hh, ww = input_shape
        dx = self._get_tensor(input_shape, dy)
        self._check(self._fn("global_avg_pool_bwd", dy)(self.h, _ptr(dy), _ptr(dx), n, ch, hh, ww, self._stream()))
        return dx

    # ------------------------------------------------------------------ fused layer ops
    def linear_forward(self, x, w, bias=None, act=None):
        """Y = act(X.W^T + b): Linear::forward (src/nn/layers/linear.rs:183-279) in one kernel."""
        x, w = self._in(x), self._in(w)
        if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
            raise FerroxB200Error(_cabi.ERR_INVALID_ARGUMENT,
                                  f"Input shape {list(x.shape)} doesn't match expected last dimension {w.shape[1]}")
        out = self._get_tensor((x.shape[0], w.shape[0]), x)
        nb = self.lib.fxb_linear_fwd_workspace_bytes(self.h, x.shape[0], x.shape[1], w.shape[0], x.element_size())
        if nb:
            ws, wsb = self.workspace(nb, x.device)
            self._check(self._fn("linear_fwd_ws", x)(self.h, _ptr(x), _ptr(w), _ptr(bias), _ptr(out), x.shape[0], x.shape[1],
                                                     w.shape[0], act_code(act), _ptr(ws), wsb, self._stream()))
            return out
        self._check(self._fn("linear_fwd", x)(self.h, _ptr(x), _ptr(w), _ptr(bias), _ptr(out), x.shape[0], x.shape[1],
                                              w.shape[0], act_code(act), self._stream()))
        return out

    def linear_backward(self, x, w, dy, y=None, act=None, need_dx=True, need_db=True):
        """(dX, dW, db) of the fused linear layer; `y` is the layer output when act is set."""
        x, w, dy = self._in(x), self._in(w), self._in(dy)
        B, i = x.shape
        o = w.shape[0]
        dx = self._get_tensor((B, i), x) if need_dx else None
        dw = self._get_tensor((o, i), x)
        db = self._get_tensor((o,), x) if need_db else None
        nb = self.lib.fxb_linear_bwd_workspace_bytes(self.h, B, i, o, x.element_size())
        ws, wsb = self.workspace(nb, x.device)
        self._check(self._fn("linear_bwd", x)(self.h, _ptr(x), _ptr(w), _ptr(None if y is None else self._in(y)), _ptr(dy),
                                              _ptr(dx), _ptr(dw), _ptr(db), B, i, o, act_code(act), _ptr(ws), wsb,
                                              self._stream()))
        return dx, dw, db

    def softmax_cross_entropy(self, logits, targets, need_grad=True, grad_scale=1.0):
        """CCELoss::forward with mean reduction plus its gradient (classification.rs:191-257)."""
        logits, targets = self._in(logits), self._in(targets)
        loss = self._get_tensor((), logits)
        g = self._get_tensor(logits.shape, logits) if need_grad else None
        self._check(self._fn("softmax_ce", logits)(self.h, _ptr(logits), _ptr(targets), _ptr(loss), _ptr(g),
                                                   logits.shape[0], logits.shape[1], grad_scale, self._stream()))
        return loss, g

    def sgd_step_(self, p, g, mom=None, lr=0.01, momentum=0.0, weight_decay=0.0, nesterov=False, grad_scale=1.0):
        self._check(self._fn("sgd_step", p)(self.h, _ptr(p), _ptr(g), _ptr(mom), p.numel(), lr, momentum, weight_decay,
                                            int(nesterov), grad_scale, self._stream()))

    def adam_step_(self, p, g, m, v, step, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, grad_scale=1.0):
        self._check(self._fn("adam_step", p)(self.h, _ptr(p), _ptr(g), _ptr(m), _ptr(v), p.numel(), lr, beta1, beta2, eps,
                                             weight_decay, step, grad_scale, self._stream()))

    def adam_step_devcount_(self, p, g, m, v, step_dev, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, grad_scale=1.0):
        """Adam::step with the step count in the int64 device tensor `step_dev` (advanced by the call)."""
        self._check(self._fn("adam_step_devcount", p)(self.h, _ptr(p), _ptr(g), _ptr(m), _ptr(v), p.numel(), lr, beta1, beta2, eps,
                                                      weight_decay, _ptr(step_dev), grad_scale, self._stream()))
