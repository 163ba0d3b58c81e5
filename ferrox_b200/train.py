"""Train step of a sequential conv/linear network on the ferrox_b200 C ABI, single GPU or
batch-sharded data parallel (one process per GPU, gradients all-reduced with NCCL through
torch.distributed while the first layers are still in backward).

The step follows the reference's loop (examples/common/training.rs:33-81): forward, softmax
cross-entropy with mean reduction, backward, optimizer step (SGD src/nn/optim/sgd.rs:210-245 or
Adam src/nn/optim/adam.rs:288-358).  torch provides device memory, streams and the process
group; every kernel in the step is one of this library's.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int64, c_void_p

import numpy as np
import torch

from . import _cabi
from ._cabi import LAYER_CONV, LAYER_FLATTEN, LAYER_LINEAR, FerroxB200Error, LayerDesc
from .cuda_ops import CudaOps, act_code


def conv(out_channels, kernel=3, stride=1, pad=1, act="relu"):
    return dict(kind="conv", out_channels=out_channels, kernel=kernel, stride=stride, pad=pad, act=act)


def flatten():
    return dict(kind="flatten")


def linear(out_features, act=None):
    return dict(kind="linear", out_channels=out_features, act=act)


_KINDS = {"conv": LAYER_CONV, "flatten": LAYER_FLATTEN, "linear": LAYER_LINEAR}


def layer_param_shapes(layers, in_shape):
    """[(W shape, b shape)] for the parameter layers of a network on input [C,H,W] (or [F])."""
    if len(in_shape) == 1:
        c, h, w = in_shape[0], 1, 1
    else:
        c, h, w = in_shape
    shapes = []
    for L in layers:
        if L["kind"] == "conv":
            k, s, p = L["kernel"], L["stride"], L["pad"]
            shapes.append(((L["out_channels"], c, k, k), (L["out_channels"],)))
            c, h, w = L["out_channels"], (h + 2 * p - k) // s + 1, (w + 2 * p - k) // s + 1
        elif L["kind"] == "flatten":
            c, h, w = c * h * w, 1, 1
        else:
            shapes.append(((L["out_channels"], c * h * w), (L["out_channels"],)))
            c, h, w = L["out_channels"], 1, 1
    return shapes


def kaiming_uniform_params(layers, in_shape, rng, dtype=np.float32):
    """Seeded Kaiming-uniform weights U(-sqrt(6/fan_in), +sqrt(6/fan_in)), zero biases."""
    out = []
    for ws, bs in layer_param_shapes(layers, in_shape):
        fan_in = int(np.prod(ws[1:]))
        bound = np.sqrt(6.0 / fan_in)
        out.append((rng.uniform(-bound, bound, size=ws).astype(dtype), np.zeros(bs, dtype)))
    return out


def flat_offsets(shapes):
    """(weight_off, bias_off, end_off) per parameter layer of the flat buffer: weight then bias,
    layers in order (the layout fxb_net_param_offsets reports)."""
    out, off = [], 0
    for ws, bs in shapes:
        w = int(np.prod(ws))
        b = int(np.prod(bs))
        out.append((off, off + w, off + w + b))
        off += w + b
    return out


def plan_buckets(offsets, nparams, tail_layers=None):
    """Splits the flat gradient buffer (+1 loss slot at the end) into the two all-reduce buckets.

    Returns (split_layer, split_off): parameter layers >= split_layer (the last layers, whose
    gradients are ready first) plus the loss slot form the tail bucket [split_off, nparams+1);
    the head bucket is [0, split_off).  By default the tail bucket is the shortest run of last layers
    that holds at least half of the parameters (but never the first layer, so that two buckets remain): it goes on the wire as soon as half of the gradient
    bytes exist and overlaps with the backward pass of the layers before it (measured on 8 GPUs with
    the deep CNN: 3.8 % faster than a tail of all layers but the first)."""
    n = len(offsets)
    if tail_layers is None:
        tail = n
        for k in range(1, n + 1):
            if 2 * (nparams - offsets[n - k][0]) >= nparams:
                tail = k
                break
        tail = min(tail, max(1, n - 1))
    else:
        tail = min(n, tail_layers)
    split_layer = n - tail
    split_off = offsets[split_layer][0] if split_layer < n else nparams
    return split_layer, split_off


def plan_bucket_list(offsets, nparams, splits=None):
    """All-reduce buckets in issue order: [(first_layer, start, end)].  `splits` are the parameter layers at which a
    bucket starts, e.g. [3, 1] for five layers = buckets of layers {3,4} (+ the loss slot), {1,2}, {0}; a bucket is
    issued as soon as backward has finished its first layer.  None: the two buckets of plan_buckets."""
    n = len(offsets)
    if splits is None:
        splits = [plan_buckets(offsets, nparams)[0]]
    cuts = sorted({int(s) for s in splits if 0 < int(s) < n}, reverse=True)
    out, end = [], nparams + 1
    for first in cuts + [0]:
        start = offsets[first][0]
        if start < end:
            out.append((first, start, end))
            end = start
    return out


class SequentialNet:
    """Flat parameter / gradient buffers + activation arena bound to one fxb_net."""

    def __init__(self, ops: CudaOps, layers, batch, in_shape, dtype=torch.float32):
        self.ops, self.lib = ops, ops.lib
        self.layers, self.batch, self.dtype = layers, int(batch), dtype
        self.in_shape = tuple(in_shape) if len(in_shape) == 3 else (in_shape[0], 1, 1)
        descs = (LayerDesc * len(layers))()
        for i, L in enumerate(layers):
            descs[i] = LayerDesc(_KINDS[L["kind"]], act_code(L.get("act")), L.get("out_channels", 0), L.get("kernel", 0),
                                 L.get("stride", 1), L.get("pad", 0))
        h = c_void_p()
        es = 4 if dtype == torch.float32 else 8
        ops._check(self.lib.fxb_net_create(ops.h, es, descs, len(layers), self.batch, *self.in_shape, ctypes.byref(h)))
        self.h = h
        self.nparams = self.lib.fxb_net_param_count(h)
        self.classes = self.lib.fxb_net_num_classes(h)
        self.n_param_layers = self.lib.fxb_net_param_layers(h)
        self.offsets = []
        for i in range(self.n_param_layers):
            w, b, e = c_int64(), c_int64(), c_int64()
            ops._check(self.lib.fxb_net_param_offsets(h, i, ctypes.byref(w), ctypes.byref(b), ctypes.byref(e)))
            self.offsets.append((w.value, b.value, e.value))
        dev = torch.device("cuda", ops.device)
        self.params = torch.zeros(self.nparams, dtype=dtype, device=dev)
        # one extra slot after the gradients carries the loss, so it rides in the same all-reduce
        self.grads = torch.zeros(self.nparams + 1, dtype=dtype, device=dev)
        self.arena = torch.empty(self.lib.fxb_net_arena_bytes(h) + 256, dtype=torch.uint8, device=dev)
        base = self.arena.data_ptr()
        self._arena_ptr = (base + 255) & ~255
        ops._check(self.lib.fxb_net_bind(h, c_void_p(self.params.data_ptr()), c_void_p(self.grads.data_ptr()),
                                         c_void_p(self._arena_ptr), self.arena.numel() - (self._arena_ptr - base)))
        self.shapes = layer_param_shapes(layers, in_shape)

    def close(self):
        if getattr(self, "h", None):
            self.lib.fxb_net_destroy(self.h)
            self.h = None

    def set_params(self, params):
        flat = np.concatenate([np.concatenate([np.asarray(w).ravel(), np.asarray(b).ravel()]) for w, b in params])
        assert flat.size == self.nparams
        self.params.copy_(torch.from_numpy(flat).to(self.dtype))

    def _unflatten(self, flat):
        flat = flat.detach().cpu().numpy()
        out = []
        for (wo, bo, eo), (ws, bs) in zip(self.offsets, self.shapes):
            out.append((flat[wo:bo].reshape(ws).copy(), flat[bo:eo].reshape(bs).copy()))
        return out

    def get_params(self):
        return self._unflatten(self.params)

    def get_grads(self):
        return self._unflatten(self.grads[: self.nparams])

    @property
    def loss_slot(self):
        return self.grads[self.nparams:]

    def forward(self, x):
        out = c_void_p()
        self.ops._check(self.lib.fxb_net_forward(self.h, c_void_p(x.data_ptr()), ctypes.byref(out), self.ops._stream()))
        return out.value

    def loss(self, targets, grad_scale=1.0):
        self.ops._check(self.lib.fxb_net_loss(self.h, c_void_p(targets.data_ptr()), c_void_p(self.loss_slot.data_ptr()),
                                              float(grad_scale), self.ops._stream()))

    def backward_range(self, x, last, first):
        self.ops._check(self.lib.fxb_net_backward_range(self.h, c_void_p(x.data_ptr()), last, first, self.ops._stream()))


class Trainer:
    """One training step = forward + loss + backward (+ gradient all-reduce) + optimizer step.

    Data parallel: every rank holds the same parameters and runs the step on its slice of the
    global batch with the loss seed scaled by 1/world, so the SUM all-reduce of the flat gradient
    buffer yields the global-batch mean gradient and every rank applies the same update.  The
    gradients are reduced in buckets of consecutive layers (`bucket_splits`, see plan_bucket_list; by default the
    last `tail_layers` parameter layers and the loss slot, then the rest), each issued while the layers before it
    are still in backward.
    """

    def __init__(self, net: SequentialNet, optimizer="sgd", lr=0.01, world_size=1, process_group=None, tail_layers=None,
                 use_graph=False, bucket_splits=None, **opt_kw):
        self.net, self.ops = net, net.ops
        # use_graph: after three eager steps the whole step (kernels, all-reduces, optimizer) is captured once
        # into a CUDA graph and replayed from then on; the inputs are copied into fixed buffers first.
        self.use_graph, self._graph, self._eager_steps = bool(use_graph), None, 0
        self._x_static = self._t_static = None
        self._graph_launches = None
        self.optimizer, self.lr, self.opt_kw = optimizer, lr, opt_kw
        self.world, self.pg = int(world_size), process_group
        self.step_count = 0
        if bucket_splits is None:
            bucket_splits = [plan_buckets(net.offsets, net.nparams, tail_layers)[0]]
        self.buckets = plan_bucket_list(net.offsets, net.nparams, bucket_splits)
        if optimizer == "adam":
            self.m = torch.zeros_like(net.params)
            self.v = torch.zeros_like(net.params)
            # graph mode keeps the step count on the device (kernel arguments are frozen in a graph)
            self.step_dev = torch.zeros(1, dtype=torch.int64, device=net.params.device)
        elif optimizer == "sgd":
            self.mom = torch.zeros_like(net.params) if opt_kw.get("momentum", 0.0) else None
        else:
            raise ValueError(optimizer)

    def _allreduce(self, t):
        import torch.distributed as dist
        return dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.pg, async_op=True)

    def close(self):
        """Releases the captured CUDA graph (it holds the all-reduce kernels of the process group's communicator:
        drop it before the process group is destroyed)."""
        if self._graph is not None:
            torch.cuda.synchronize()
            self._graph.reset()
            self._graph = None

    @property
    def launches_per_step(self):
        """Kernels of this library in one step (counted while the graph was captured; None before that)."""
        return self._graph_launches

    def input_buffers(self):
        """(x, targets) buffers the captured graph reads, once it exists: a caller that fills them directly
        (e.g. with its host-to-device copy) and passes them to step() saves the device-to-device copy."""
        return self._x_static, self._t_static

    def step(self, x, targets):
        """x [B_local, ...], targets one-hot [B_local, classes], both on the device.  Returns the
        device tensor holding the (global mean) loss."""
        if not self.use_graph:
            return self._step_body(x, targets)
        if self._graph is None:
            if self._eager_steps < 3:  # sets kernel attributes, fills the tensor-map cache, creates the communicator
                self._eager_steps += 1
                return self._step_body(x, targets)
            self._x_static, self._t_static = torch.empty_like(x), torch.empty_like(targets)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            n0 = self.ops.launch_count()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                self._step_body(self._x_static, self._t_static)
            self._graph_launches = self.ops.launch_count() - n0  # every replay runs these kernels again
            self.step_count -= 1  # the capture recorded the step without running it
            self._graph = graph
        if x.data_ptr() != self._x_static.data_ptr():
            self._x_static.copy_(x, non_blocking=True)
        if targets.data_ptr() != self._t_static.data_ptr():
            self._t_static.copy_(targets, non_blocking=True)
        self._graph.replay()
        self.step_count += 1
        return self.net.loss_slot

    def _step_body(self, x, targets):
        net, ops = self.net, self.ops
        n = net.n_param_layers
        net.forward(x)
        net.loss(targets, 1.0 / self.world)
        works = []
        if self.world > 1:
            last = n - 1
            for first, start, end in self.buckets:   # the last layers' bucket (with the loss slot) goes first
                net.backward_range(x, last, first)
                works.append(self._allreduce(net.grads[start:end]))
                last = first - 1
        else:
            net.backward_range(x, n - 1, 0)
        for w in works:
            w.wait()
        self._optimizer_step()
        return net.loss_slot

    def _optimizer_step(self):
        net, ops = self.net, self.ops
        self.step_count += 1
        g = net.grads[: net.nparams]
        if self.optimizer == "adam" and self.use_graph:
            ops.adam_step_devcount_(net.params, g, self.m, self.v, self.step_dev, lr=self.lr, beta1=self.opt_kw.get("beta1", 0.9),
                                    beta2=self.opt_kw.get("beta2", 0.999), eps=self.opt_kw.get("eps", 1e-8),
                                    weight_decay=self.opt_kw.get("weight_decay", 0.0))
        elif self.optimizer == "adam":
            ops.adam_step_(net.params, g, self.m, self.v, self.step_count, lr=self.lr, beta1=self.opt_kw.get("beta1", 0.9),
                           beta2=self.opt_kw.get("beta2", 0.999), eps=self.opt_kw.get("eps", 1e-8),
                           weight_decay=self.opt_kw.get("weight_decay", 0.0))
        else:
            ops.sgd_step_(net.params, g, self.mom, lr=self.lr, momentum=self.opt_kw.get("momentum", 0.0),
                          weight_decay=self.opt_kw.get("weight_decay", 0.0), nesterov=self.opt_kw.get("nesterov", False))

    def step_with_marks(self, x, targets):
        """The same step as step(), one parameter layer per backward call, with a CUDA event and a host
        timestamp recorded at the start of every phase.  Returns [(phase name, event, host seconds)], the
        last entry marking the end; the time between two events is the phase's time on the compute stream
        (for "allreduce_wait": the part of the all-reduces that backward did not hide)."""
        import time
        net = self.net
        n = net.n_param_layers
        marks = []

        def mark(name):
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            marks.append((name, e, time.perf_counter()))

        mark("forward")
        net.forward(x)
        mark("loss")
        net.loss(targets, 1.0 / self.world)
        works = []
        starts = {first: (start, end) for first, start, end in self.buckets}
        for pi in range(n - 1, -1, -1):
            mark(f"backward_layer{pi}")
            net.backward_range(x, pi, pi)
            if self.world > 1 and pi in starts:
                mark(f"allreduce_issue_from_layer{pi}")
                works.append(self._allreduce(net.grads[starts[pi][0]:starts[pi][1]]))
        mark("allreduce_wait")
        for w in works:
            w.wait()
        mark("optimizer")
        self._optimizer_step()
        mark("end")
        return marks

    def loss_value(self):
        """Global mean loss of the last step (one device-to-host read).  This is the step's only
        synchronisation point, so the device status word is read here as well: a bounded wait that
        ran out in any kernel of the step raises FerroxB200Error instead of letting the optimizer
        go on with partly written gradients."""
        self.ops.check_device_status()
        v = float(self.net.loss_slot.item())
        return v / self.world if self.world > 1 else v


# The BASELINE network configurations.
def small_cnn_layers():      # 32x1x28x28 -> 10, SGD lr 0.01
    return [conv(16), conv(32), flatten(), linear(10)], (1, 28, 28)


def mlp_layers():            # 256x784 -> 10
    return [linear(512, "relu"), linear(512, "relu"), linear(10)], (784,)


def deep_cnn_layers():       # global batch 1024x3x32x32 -> 10, Adam lr 1e-3
    return [conv(64, stride=1), conv(128, stride=2), conv(256, stride=2), conv(256, stride=2), flatten(), linear(10)], (3, 32, 32)
