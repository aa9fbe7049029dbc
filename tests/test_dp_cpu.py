"""Data-parallel algebra on CPU ranks (gloo, world size 2): row shards of the batch, the
global element count in the MSE seed, gradients summed over ranks, the same update on every
rank.  The result must equal the single-process step on the full batch."""
import socket
import tempfile

import numpy as np
import pytest
import torch.multiprocessing as mp

from oracle.oracle import Oracle
from tests import dp_common as dpc


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("opt,real,tol", [("sgd_momentum", "f64", 1e-12), ("adam", "f64", 1e-9), ("sgd_momentum", "f32", 1e-5)])
def test_two_cpu_ranks_reproduce_the_full_batch_step(opt, real, tol):
    world = 2
    out = tempfile.mkdtemp()
    mp.spawn(dpc.oracle_shard_worker, args=(world, _free_port(), opt, real, out), nprocs=world, join=True)
    x, y, ws, bs = dpc.inputs()
    o = Oracle(dpc.LAYERS, "silu", opt, dpc.GLOBAL_BATCH, real=real)
    for i, (w, b) in enumerate(zip(ws, bs)):
        o.set_params(i, w, b)
    losses = []
    for _ in range(dpc.STEPS):
        o.step(x, y, 0.01)
        losses.append(o.loss())
    pw, pb = o.get_params()
    ranks = [np.load("%s/rank%d.npz" % (out, r)) for r in range(world)]
    for r in ranks:
        np.testing.assert_allclose(r["losses"], losses, rtol=max(tol, 1e-6) if real == "f32" else 1e-9)
        for i in range(len(pw)):
            assert np.max(np.abs(r["w%d" % i] - pw[i])) <= tol * np.max(np.abs(pw[i]))
            assert np.max(np.abs(r["b%d" % i] - pb[i])) <= tol * max(np.max(np.abs(pb[i])), 1e-3)
    # replicas stay bit-identical
    for i in range(len(pw)):
        assert np.array_equal(ranks[0]["w%d" % i], ranks[1]["w%d" % i])
        assert np.array_equal(ranks[0]["b%d" % i], ranks[1]["b%d" % i])


def test_two_cpu_ranks_draw_their_slice_of_the_single_process_dropout_stream():
    """Dropout under data parallelism: one draw per hidden element of the GLOBAL batch in layer, row, column order
    (mlp_train_rust_codegen.rs:773-788); a rank takes the draws of its own rows and skips the others', so the
    sharded step equals the single-process one - which is what the GPU ranks do with a jump-ahead generator."""
    world, opt = 2, "sgd_momentum"
    out = tempfile.mkdtemp()
    mp.spawn(dpc.oracle_shard_worker, args=(world, _free_port(), opt, "f64", out, "relu", 0.3), nprocs=world, join=True)
    x, y, ws, bs = dpc.inputs()
    o = Oracle(dpc.LAYERS, "relu", opt, dpc.GLOBAL_BATCH, real="f64", dropout_p=0.3)
    for i, (w, b) in enumerate(zip(ws, bs)):
        o.set_params(i, w, b)
    losses = []
    for _ in range(dpc.STEPS):
        o.step(x, y, 0.01)
        losses.append(o.loss())
    pw, pb = o.get_params()
    for r in (np.load("%s/rank%d.npz" % (out, k)) for k in range(world)):
        np.testing.assert_allclose(r["losses"], losses, rtol=1e-9)
        for i in range(len(pw)):
            assert np.max(np.abs(r["w%d" % i] - pw[i])) <= 1e-12 * np.max(np.abs(pw[i]))
    # a wrong slice (every rank drawing from the start of each layer's share) does NOT reproduce it
    plain = Oracle(dpc.LAYERS, "relu", opt, dpc.GLOBAL_BATCH // 2, real="f64", dropout_p=0.3)
    plain.set_global_batch(dpc.GLOBAL_BATCH)
    for i, (w, b) in enumerate(zip(ws, bs)):
        plain.set_params(i, w, b)
    half = dpc.GLOBAL_BATCH // 2
    plain.grad_step(x[half:], y[half:])
    shard = Oracle(dpc.LAYERS, "relu", opt, half, real="f64", dropout_p=0.3)
    shard.set_global_batch(dpc.GLOBAL_BATCH)
    shard.set_shard_row0(half)
    for i, (w, b) in enumerate(zip(ws, bs)):
        shard.set_params(i, w, b)
    shard.grad_step(x[half:], y[half:])
    assert not np.allclose(plain.get_grads()[0][0], shard.get_grads()[0][0])
