"""GPU parity of whole training steps (forward, loss, every gradient, optimizer update) against the
CPU oracle composed like the reference graph, on the BASELINE network configurations."""
import numpy as np
import pytest
import torch

from test_gpu_parity import assert_parity, dev

pytestmark = pytest.mark.gpu


def _oracle_layers(layers):
    from ferrox_b200.cuda_ops import act_code
    return [dict(kind=L["kind"], stride=L.get("stride", 1), pad=L.get("pad", 0), act=act_code(L.get("act"))) for L in layers]


def _run(ops, oracle, layers, in_shape, batch, x, dtype, optimizer, lr, steps=2):
    from ferrox_b200.train import SequentialNet, Trainer, kaiming_uniform_params
    rng = np.random.default_rng(20261125)
    params = kaiming_uniform_params(layers, in_shape, rng, dtype)
    params = [(w, (rng.standard_normal(b.shape) * 0.05).astype(dtype)) for w, b in params]
    labels = rng.integers(0, 10, batch)
    t = np.eye(10, dtype=dtype)[labels]
    net = SequentialNet(ops, layers, batch, in_shape, torch.float32 if dtype == np.float32 else torch.float64)
    net.set_params(params)
    tr = Trainer(net, optimizer=optimizer, lr=lr)
    cpu_params = [(w.copy(), b.copy()) for w, b in params]
    m = [(np.zeros_like(w), np.zeros_like(b)) for w, b in params]
    v = [(np.zeros_like(w), np.zeros_like(b)) for w, b in params]
    xd, td = dev(x), dev(t)
    for step in range(1, steps + 1):
        tr.step(xd, td)
        loss_ref, grads_ref = oracle.net_forward_backward(_oracle_layers(layers), cpu_params, x, t)
        assert_parity(net.loss_slot[0], np.asarray(loss_ref), f"loss step {step}")
        for i, ((dw, db), (rw, rb)) in enumerate(zip(net.get_grads(), grads_ref)):
            assert_parity(dw, rw, f"dW layer {i} step {step}")
            assert_parity(db, rb, f"db layer {i} step {step}")
        # Optimizer parity: the oracle's update applied to the gradient values the GPU produced.
        # (Chaining the CPU gradients instead would test Adam's conditioning, not the kernels: on the
        # first steps the update is ~lr*g/(|g|+eps), so two f32 gradients that agree to 1e-9 can still
        # move a weight with |g| ~ eps by different amounts.)
        gpu_grads = net.get_grads()
        for i, ((w, b), (gw, gb)) in enumerate(zip(cpu_params, gpu_grads)):
            for p, g, mm, vv in ((w, gw, m[i][0], v[i][0]), (b, gb, m[i][1], v[i][1])):
                if optimizer == "adam":
                    oracle.adam_step(p.reshape(-1), g.reshape(-1), mm.reshape(-1), vv.reshape(-1), step, lr=lr)
                else:
                    oracle.sgd_step(p.reshape(-1), g.reshape(-1), lr=lr)
        for i, ((w, b), (rw, rb)) in enumerate(zip(net.get_params(), cpu_params)):
            assert_parity(w, rw, f"W layer {i} after step {step}")
            assert_parity(b, rb, f"b layer {i} after step {step}")
        # next step starts from the same parameter bits on both sides
        cpu_params = [(w.copy(), b.copy()) for w, b in net.get_params()]
    ops.check_device_status()
    net.close()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_small_cnn_classifier_step(ops, oracle, dtype):
    """Config 1: 32x1x28x28, conv16-relu-conv32-relu-flatten-fc10, SGD lr 0.01."""
    from ferrox_b200.train import small_cnn_layers
    layers, in_shape = small_cnn_layers()
    x = np.random.default_rng(1).random((32, 1, 28, 28)).astype(dtype)
    _run(ops, oracle, layers, in_shape, 32, x, dtype, "sgd", 0.01)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_mlp_step(ops, oracle, dtype):
    """Config 2: 256x784, 784-512-512-10 with relu."""
    from ferrox_b200.train import mlp_layers
    layers, in_shape = mlp_layers()
    x = np.random.default_rng(2).standard_normal((256, 784)).astype(dtype)
    _run(ops, oracle, layers, in_shape, 256, x, dtype, "sgd", 0.01)


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_deep_cnn_step_adam(ops, oracle, dtype):
    """Config 4's network (3->64->128->256->256, strides 1,2,2,2, fc 4096->10, Adam) at a batch the
    oracle finishes in seconds."""
    from ferrox_b200.train import deep_cnn_layers
    layers, in_shape = deep_cnn_layers()
    x = np.random.default_rng(3).standard_normal((16, 3, 32, 32)).astype(dtype)
    _run(ops, oracle, layers, in_shape, 16, x, dtype, "adam", 1e-3)


def test_sharded_step_equals_global_step_on_one_gpu(ops, oracle):
    """Two half-batch shards with the 1/world loss seed, gradients added, give the global-batch
    gradient (the arithmetic of the data-parallel step without the process group)."""
    from ferrox_b200.train import SequentialNet, deep_cnn_layers, kaiming_uniform_params
    layers, in_shape = deep_cnn_layers()
    rng = np.random.default_rng(7)
    params = kaiming_uniform_params(layers, in_shape, rng, np.float64)
    x = rng.standard_normal((8, 3, 32, 32))
    t = np.eye(10)[rng.integers(0, 10, 8)]
    full = SequentialNet(ops, layers, 8, in_shape, torch.float64)
    full.set_params(params)
    xd, td = dev(x), dev(t)
    full.forward(xd); full.loss(td); full.backward_range(xd, full.n_param_layers - 1, 0)
    half = SequentialNet(ops, layers, 4, in_shape, torch.float64)
    half.set_params(params)
    acc = torch.zeros_like(half.grads)
    for r in range(2):
        xs, ts = dev(x[4 * r: 4 * r + 4]), dev(t[4 * r: 4 * r + 4])
        half.forward(xs); half.loss(ts, 0.5); half.backward_range(xs, half.n_param_layers - 1, 0)
        acc += half.grads
    assert_parity(acc[:-1], full.grads[:-1].cpu().numpy(), "summed shard gradients")
    assert_parity(acc[-1] / 2, full.grads[-1].cpu().numpy(), "mean of shard losses")
    full.close(); half.close()


def test_graph_replayed_step_equals_eager_step(ops, oracle):
    """The train step captured once into a CUDA graph (after three eager steps) and replayed gives the same
    parameters, bit for bit, as eager launches; Adam's step count lives on the device in that mode."""
    from ferrox_b200.train import SequentialNet, Trainer, deep_cnn_layers, kaiming_uniform_params
    layers, in_shape = deep_cnn_layers()
    rng = np.random.default_rng(11)
    params = kaiming_uniform_params(layers, in_shape, rng, np.float32)
    batches = [(dev(rng.standard_normal((16, 3, 32, 32)).astype(np.float32)),
                dev(np.eye(10, dtype=np.float32)[rng.integers(0, 10, 16)])) for _ in range(7)]
    results = []
    for use_graph in (False, True):
        net = SequentialNet(ops, layers, 16, in_shape, torch.float32)
        net.set_params(params)
        tr = Trainer(net, optimizer="adam", lr=1e-3, use_graph=use_graph)
        losses = []
        for x, t in batches:
            tr.step(x, t)
            losses.append(tr.loss_value())
        assert tr.step_count == len(batches)
        if use_graph:
            assert tr._graph is not None and int(tr.step_dev.item()) == len(batches)
        results.append((losses, net.params.clone()))
        net.close()
    assert np.allclose(results[0][0], results[1][0], rtol=1e-6, atol=0)
    # the device-side bias correction uses powf on the GPU, the eager path pow on the host: allow an ulp or two
    assert_parity(results[1][1], results[0][1].cpu().numpy(), "parameters after 7 steps, graph vs eager")
    ops.check_device_status()


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_adam_with_device_step_count(ops, oracle, dtype):
    rng = np.random.default_rng(5)
    n = 5003
    p, g = rng.standard_normal(n).astype(dtype), rng.standard_normal(n).astype(dtype)
    pc, m, v = p.copy(), np.zeros(n, dtype), np.zeros(n, dtype)
    pt, mt, vt = dev(p), dev(np.zeros(n, dtype)), dev(np.zeros(n, dtype))
    step_dev = torch.zeros(1, dtype=torch.int64, device="cuda:0")
    for step in range(1, 6):
        oracle.adam_step(pc, g, m, v, step, wd=0.01)
        ops.adam_step_devcount_(pt, dev(g), mt, vt, step_dev, weight_decay=0.01)
    assert int(step_dev.item()) == 5
    assert_parity(pt, pc, "adam with device step count")
