"""CPU test (gloo, world_size 2) of the data-parallel step's host logic: batch sharding, the 1/world
loss seed, the two gradient buckets of the flat buffer and the SUM all-reduce give every rank the
global-batch mean loss and gradient.  The per-rank compute is the CPU oracle (no GPU needed here)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import cpu_oracle as orc
        from ferrox_b200.train import flat_offsets, kaiming_uniform_params, layer_param_shapes, plan_buckets, conv, flatten, linear
        layers = [conv(4, stride=1), conv(6, stride=2), conv(8, stride=2), flatten(), linear(10)]
        in_shape = (3, 8, 8)
        rng = np.random.default_rng(5)
        params = kaiming_uniform_params(layers, in_shape, rng, np.float64)
        B = 8
        x = rng.standard_normal((B, *in_shape))
        t = np.eye(10)[rng.integers(0, 10, B)]
        olayers = [dict(kind=L["kind"], stride=L.get("stride", 1), pad=L.get("pad", 0), act=1 if L.get("act") == "relu" else 0)
                   for L in layers]
        lb = B // world
        xs, ts = x[rank * lb:(rank + 1) * lb], t[rank * lb:(rank + 1) * lb]
        loss, grads = orc.net_forward_backward(olayers, params, xs, ts)
        shapes = layer_param_shapes(layers, in_shape)
        offs = flat_offsets(shapes)
        nparams = offs[-1][2]
        flat = np.zeros(nparams + 1)
        for (wo, bo, eo), (dw, db) in zip(offs, grads):
            flat[wo:bo] = dw.ravel() / world      # what the 1/world loss seed does to every gradient
            flat[bo:eo] = db.ravel() / world
        flat[nparams] = loss
        split_layer, split_off = plan_buckets(offs, nparams)
        assert 0 < split_layer < len(offs) and split_off == offs[split_layer][0]
        from ferrox_b200.train import plan_bucket_list
        assert plan_bucket_list(offs, nparams) == [(split_layer, split_off, nparams + 1), (0, 0, split_off)]
        buckets = plan_bucket_list(offs, nparams, [3, 1])   # three buckets, last layers (+ loss slot) first
        assert [b[0] for b in buckets] == [3, 1, 0] and buckets[0][2] == nparams + 1 and buckets[-1][1] == 0
        assert all(buckets[i][1] == buckets[i + 1][2] for i in range(2))   # the buckets tile the buffer
        buf = torch.from_numpy(flat)
        works = [dist.all_reduce(buf[start:end], async_op=True) for _, start, end in buckets]
        for w in works:
            w.wait()
        gl, gg = orc.net_forward_backward(olayers, params, x, t)
        ref = np.concatenate([np.concatenate([dw.ravel(), db.ravel()]) for dw, db in gg])
        err = np.abs(buf[:nparams].numpy() - ref).max()
        lerr = abs(buf[nparams].item() / world - gl)
        q.put((rank, float(err), float(lerr)))
    finally:
        dist.destroy_process_group()


def test_two_rank_bucketed_allreduce_matches_global_batch():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, lerr in res:
        assert err < 1e-12 and lerr < 1e-12, (rank, err, lerr)


def test_bucket_plans_of_the_benchmark_networks():
    """The tail bucket is the shortest run of last layers that holds at least half of the parameters; bucket lists
    tile the flat gradient buffer (plus the loss slot) exactly once, last layers first."""
    from ferrox_b200.train import deep_cnn_layers, flat_offsets, layer_param_shapes, mlp_layers, plan_bucket_list, plan_buckets
    for make, want_split in ((deep_cnn_layers, 3), (mlp_layers, 1)):
        layers, in_shape = make()
        offs = flat_offsets(layer_param_shapes(layers, in_shape))
        nparams = offs[-1][2]
        split_layer, split_off = plan_buckets(offs, nparams)
        assert split_layer == want_split and split_off == offs[split_layer][0]
        if split_layer > 1 or 2 * (nparams - split_off) >= nparams:
            assert 2 * (nparams - split_off) >= nparams                  # the tail holds at least half ...
        else:
            assert split_layer == 1                                      # ... or everything but the first layer
        if split_layer + 1 < len(offs):
            assert 2 * (nparams - offs[split_layer + 1][0]) < nparams    # and no shorter tail holds half
        for splits in (None, [3, 1], [1], [4, 3, 2, 1], [0, 99]):
            buckets = plan_bucket_list(offs, nparams, splits)
            assert buckets[0][2] == nparams + 1 and buckets[-1][1] == 0
            assert all(a[1] == b[2] for a, b in zip(buckets, buckets[1:]))
            assert [b[0] for b in buckets] == sorted({b[0] for b in buckets}, reverse=True)
    assert plan_buckets(offs, nparams, tail_layers=1)[0] == len(offs) - 1
