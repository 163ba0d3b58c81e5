"""GPU parity of the layout kernels (materialize, transpose, broadcast_to: bit-exact data movement)
and of batch normalisation / global average pooling against the CPU oracle."""
import numpy as np
import pytest
import torch

from test_gpu_parity import assert_parity, dev, host

pytestmark = pytest.mark.gpu

DTYPES = [np.float32, np.float64]


def test_layout_golden_vectors_through_cuda(ops, golden):
    g = golden["matrix_transpose"]
    a = np.array(g["input"], np.float32).reshape(g["rows"], g["cols"])
    assert host(ops.transpose(dev(a))).ravel().tolist() == g["expected"]
    g = golden["test_transpose_operation"]
    assert list(ops.transpose(dev(np.array(g["input"], np.float32).reshape(g["shape"]))).shape) == g["expected_shape"]
    g = golden["test_bias_broadcasting"]
    b = ops.broadcast_to(dev(np.array(g["input"], np.float32).reshape(g["in_shape"])), g["target_shape"])
    assert host(b).tolist() == np.array(g["expected"], np.float32).tolist()
    g = golden["test_broadcast_to"]
    b = ops.broadcast_to(dev(np.array(g["input"], np.float32)), g["target_shape"])
    assert host(b).tolist() == [g["input"]] * 3
    g = golden["test_global_avgpool2d_forward"]
    y = ops.global_avg_pool_forward(dev(np.array(g["input"], np.float32).reshape(g["x_shape"])), flatten=False)
    assert list(y.shape) == g["y_shape"] and abs(host(y).item() - g["expected"][0]) <= g["tol"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape,axes", [
    ((2, 3), None), ((784, 512), None), ((513, 300), None), ((1000, 7), None), ((5, 1), None), ((1,), None), ((7,), None),
    ((4, 5, 6), None), ((4, 5, 6), (0, 2, 1)), ((4, 5, 6), (1, 0, 2)), ((3, 8, 14, 12), (0, 2, 3, 1)),
    ((3, 8, 14, 12), (0, 3, 1, 2)), ((3, 8, 14, 12), (1, 0, 2, 3)), ((6, 64, 9, 11), (1, 0, 2, 3)),
    ((2, 3, 4, 5, 6), (4, 3, 2, 1, 0)), ((2, 3, 2, 3, 2, 3, 2, 3), (7, 0, 6, 1, 5, 2, 4, 3)), ((2048, 1024), None),
])
def test_transpose_bit_exact(ops, oracle, dtype, shape, axes):
    rng = np.random.default_rng(len(shape))
    x = rng.standard_normal(shape).astype(dtype)
    got = host(ops.transpose(dev(x), axes))
    ref = oracle.transpose(x, axes)
    assert got.shape == ref.shape and np.array_equal(got, ref)
    if len(shape) > 1:
        inv = np.argsort(axes if axes is not None else list(range(len(shape) - 1, -1, -1)))
        back = host(ops.transpose(ops.transpose(dev(x), axes), [int(a) for a in inv]))
        assert np.array_equal(back, x)  # the gradient of Transpose is the inverse permutation


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("in_shape,out_shape", [
    ((1,), (4,)), ((2,), (3, 2)), ((1, 16, 1, 1), (8, 16, 28, 28)), ((1, 10), (256, 10)), ((5, 1), (5, 7)),
    ((3, 1, 5), (2, 3, 4, 5)), ((64,), (17, 64)), ((1, 1), (1, 1)), ((4, 1, 1), (4, 3, 1)), ((7, 3), (7, 3)),
])
def test_broadcast_to_bit_exact(ops, oracle, dtype, in_shape, out_shape):
    rng = np.random.default_rng(sum(out_shape))
    x = rng.standard_normal(in_shape).astype(dtype)
    got = host(ops.broadcast_to(dev(x), out_shape))
    assert np.array_equal(got, oracle.broadcast_to(x, out_shape))


@pytest.mark.parametrize("dtype", DTYPES)
def test_materialize_strided_views(ops, oracle, dtype):
    rng = np.random.default_rng(5)
    base = rng.standard_normal((6, 10, 12)).astype(dtype)
    t = dev(base)
    views = [t.permute(2, 0, 1), t[:, ::2, :], t[1:5, 3:9, 2:11:3], t.permute(1, 2, 0)[2:, :, ::2], t[:, :, 5:6].expand(6, 10, 4),
             t[2], t.transpose(0, 1), t[:, 0, :].unsqueeze(1).expand(6, 3, 12)]
    for v in views:
        got = ops.materialize(v)
        assert got.is_contiguous() and torch.equal(got, v.contiguous())
        flat = host(t).ravel()
        off = v.storage_offset()
        ref = oracle.materialize(flat[off:], tuple(v.shape), tuple(v.stride()))
        assert np.array_equal(host(got), ref)


def test_layout_errors(ops):
    from ferrox_b200.cuda_ops import FerroxB200Error
    with pytest.raises(FerroxB200Error, match="permutation"):
        ops.transpose(dev(np.zeros((2, 3), np.float32)), (0, 0))
    with pytest.raises(FerroxB200Error, match="Cannot broadcast dimension"):
        ops.broadcast_to(dev(np.zeros((3,), np.float32)), (2, 2))
    with pytest.raises(FerroxB200Error, match="at least as many dimensions"):
        ops.broadcast_to(dev(np.zeros((2, 3), np.float32)), (3,))
    assert ops.transpose(dev(np.zeros((0, 3), np.float32))).shape == (3, 0)


# ------------------------------------------------------------------ batch norm, global average pooling
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(32, 16, 28, 28), (8, 32, 14, 14), (5, 3, 7, 9), (256, 64), (33, 7), (4, 130, 6, 6), (64, 32, 32, 32)])
@pytest.mark.parametrize("act", [0, 1])
def test_batch_norm_forward_backward(ops, oracle, dtype, shape, act):
    rng = np.random.default_rng(sum(shape) + act)
    C = shape[1]
    x = (rng.standard_normal(shape) * 1.5 + 0.3).astype(dtype)
    gamma = (1 + 0.2 * rng.standard_normal(C)).astype(dtype)
    beta = (0.1 * rng.standard_normal(C)).astype(dtype)
    rm, rv = rng.standard_normal(C).astype(dtype), (rng.random(C) + 0.5).astype(dtype)
    rm_t, rv_t = dev(rm), dev(rv)
    z_ref, mean_ref, var_ref = oracle.batch_norm_fwd(x, gamma, beta, 1e-3, rm, rv, 0.1, training=True)
    y_ref = oracle.act_fwd(z_ref, act) if act else z_ref
    y, mean, var = ops.batch_norm_forward(dev(x), dev(gamma), dev(beta), 1e-3, 0.1, rm_t, rv_t, True, act)
    assert_parity(mean, mean_ref, "batch mean")
    assert_parity(var, var_ref, "batch variance")
    assert_parity(y, y_ref, "batch norm output")
    assert_parity(rm_t, rm, "running mean")
    assert_parity(rv_t, rv, "running variance")
    dy = rng.standard_normal(shape).astype(dtype)
    dz = oracle.act_bwd(dy, z_ref, 1) if act else dy
    dx_ref, dg_ref, db_ref = oracle.batch_norm_bwd(x, dz, gamma, mean_ref, var_ref, 1e-3)
    # same statistics and activation values on both sides, so the ReLU mask is identical
    dx, dg, db = ops.batch_norm_backward(dev(x), dev(dy), dev(gamma), dev(mean_ref), dev(var_ref), 1e-3, dev(y_ref) if act else None, act)
    assert_parity(dx, dx_ref, "batch norm dX")
    assert_parity(dg, dg_ref, "batch norm dgamma")
    assert_parity(db, db_ref, "batch norm dbeta")
    dx2, dg2, db2 = ops.batch_norm_backward(dev(x), dev(dy), dev(gamma), dev(mean_ref), dev(var_ref), 1e-3, dev(y_ref) if act else None, act)
    assert torch.equal(dx, dx2) and torch.equal(dg, dg2) and torch.equal(db, db2)
    # inference mode: running statistics, no workspace
    yi = ops.batch_norm_forward(dev(x), dev(gamma), dev(beta), 1e-3, 0.1, dev(rm), dev(rv), False, 0)
    assert_parity(yi, oracle.batch_norm_fwd(x, gamma, beta, 1e-3, rm, rv, training=False), "batch norm inference")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1, 1, 4, 4), (32, 32, 28, 28), (7, 5, 3, 3), (4, 256, 4, 4), (3, 2, 1, 1), (2, 3, 56, 56), (2, 3, 5, 7)])
def test_global_avg_pool(ops, oracle, dtype, shape):
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal(shape).astype(dtype)
    assert_parity(ops.global_avg_pool_forward(dev(x)), oracle.global_avg_pool_fwd(x), "GAP forward")
    assert ops.global_avg_pool_forward(dev(x), flatten=False).shape == (shape[0], shape[1], 1, 1)
    dy = rng.standard_normal(shape[:2]).astype(dtype)
    got = host(ops.global_avg_pool_backward(dev(dy), shape))
    assert np.array_equal(got, oracle.global_avg_pool_bwd(dy, shape))  # one multiply per element: bit-exact


def test_norm_errors(ops):
    from ferrox_b200.cuda_ops import FerroxB200Error
    with pytest.raises(FerroxB200Error, match="at least 2D"):
        ops.batch_norm_forward(dev(np.zeros((4,), np.float32)), None, None)
    with pytest.raises(FerroxB200Error, match="requires 4D input"):
        ops.global_avg_pool_forward(dev(np.zeros((4, 3), np.float32)))
