"""Data parallelism on real GPUs (needs >= 2): two ranks of libvolta_b200 with bucketed NCCL
all-reduce against the single-process oracle on the full batch; replicas bit-identical; two
runs bit-identical."""
import socket
import tempfile

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from oracle.oracle import Oracle
from tests import dp_common as dpc

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_data_parallel_path_on_a_single_rank_matches_the_plain_path():
    """The whole data-parallel machinery (NCCL communicator, per-layer buckets reduced on a
    side stream inside the captured graph, loss travelling in the bias bucket) with one rank:
    a sum over one rank changes nothing, so results must equal the plain handle bit for bit."""
    from volta_b200 import TrainHandle
    from volta_b200.train import dp_unique_id
    x, y, ws, bs = dpc.inputs()
    outs = []
    for dp in (False, True):
        # step_kernel=1: both handles on the per-kernel schedule (at this batch a plain handle would otherwise take
        # the persistent step kernel, whose sums are ordered differently)
        h = TrainHandle(dpc.LAYERS, "silu", "adam", dpc.GLOBAL_BATCH, force_dp=dp, unique_id=dp_unique_id() if dp else None,
                        step_kernel=1)
        for i, (w, b) in enumerate(zip(ws, bs)):
            h.set_params(i, w, b)
        losses = []
        for _ in range(dpc.STEPS):
            h.step(x, y, 0.01)
            losses.append(np.float32(h.loss()))
        outs.append((losses, sum(h.get_params(), [])))
        h.free()
    assert outs[0][0] == outs[1][0]
    for a, b in zip(outs[0][1], outs[1][1]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("exchange", ["peer_kernel", "peer_copy"])
@pytest.mark.parametrize("opt", ["adam", "sgd_momentum"])
def test_fused_peer_memory_update_on_a_single_rank_matches_the_plain_path(opt, exchange):
    """The fused reduce + update + redistribute kernels (or, by copy, the gather + update kernels) and their flag
    barriers with one rank (its own arena as the only peer): a sum over one rank adds nothing, so the bits must
    equal the plain handle's."""
    from volta_b200 import TrainHandle
    from volta_b200.train import dp_unique_id
    x, y, ws, bs = dpc.inputs()
    outs = []
    for fused in (False, True):
        h = TrainHandle(dpc.LAYERS, "silu", opt, dpc.GLOBAL_BATCH, force_dp=fused, unique_id=dp_unique_id() if fused else None,
                        step_kernel=1, dp_exchange=exchange if fused else "nccl")
        if fused:
            h.attach_peers([h.ipc_handle()])
        for i, (w, b) in enumerate(zip(ws, bs)):
            h.set_params(i, w, b)
        losses = []
        for _ in range(dpc.STEPS):
            h.step(x, y, 0.01)
            losses.append(np.float32(h.loss()))
        outs.append((losses, sum(h.get_params(), [])))
        h.free()
    assert outs[0][0] == outs[1][0]
    for a, b in zip(outs[0][1], outs[1][1]):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mode", ["nccl", "fused", "copy"])
@pytest.mark.parametrize("opt", ["sgd_momentum", "adam"])
def test_gpu_ranks_match_the_full_batch_oracle(opt, mode, world):
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    out = tempfile.mkdtemp()
    mp.spawn(dpc.gpu_shard_worker, args=(world, _free_port(), opt, out, 2, {"nccl": False, "fused": True, "copy": "copy"}[mode]),
             nprocs=world, join=True)
    x, y, ws, bs = dpc.inputs()
    o = Oracle(dpc.LAYERS, "silu", opt, dpc.GLOBAL_BATCH)
    for i, (w, b) in enumerate(zip(ws, bs)):
        o.set_params(i, w, b)
    losses = []
    for _ in range(dpc.STEPS):
        o.step(x, y, 0.01)
        losses.append(o.loss())
    pw, pb = o.get_params()
    runs = [[np.load("%s/rank%d_rep%d.npz" % (out, r, rep)) for r in range(world)] for rep in range(2)]
    for rep in runs:
        for r in rep:
            np.testing.assert_allclose(r["losses"], losses, rtol=1e-5)
            for i in range(len(pw)):
                diff = np.abs(r["w%d" % i] - pw[i])
                lim = 1e-4 * np.max(np.abs(pw[i]))
                if opt == "adam":
                    # Adam's update is sign-like where a gradient sits at the fp32 noise floor, so a
                    # few weights move by up to 2*lr per step between two correct summation orders
                    assert np.mean(diff > lim) <= 2e-3 and np.max(diff) <= 2 * 0.01 * dpc.STEPS
                else:
                    assert np.max(diff) <= lim
        for i in range(len(pw)):  # replicas bit-identical
            assert np.array_equal(rep[0]["w%d" % i], rep[1]["w%d" % i])
            assert np.array_equal(rep[0]["b%d" % i], rep[1]["b%d" % i])
    for i in range(len(pw)):      # run-to-run bit-identical at a fixed GPU count
        assert np.array_equal(runs[0][0]["w%d" % i], runs[1][0]["w%d" % i])
    assert np.array_equal(runs[0][0]["losses"], runs[1][0]["losses"])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_ranks_with_the_optional_stages_match_the_full_batch_oracle():
    """relu -> LayerNorm -> dropout with the clip active, rows split over two ranks: each rank draws its
    rows' slice of the single-process mask stream, the LayerNorm gradients travel in the last bucket and
    the clip's norm is summed over the ranks in mid-step; the result is the full-batch oracle's."""
    world, opt = 2, "sgd"
    options = dict(use_layernorm=True, dropout_p=0.25, clip_grad=0.02)
    out = tempfile.mkdtemp()
    mp.spawn(dpc.gpu_shard_worker, args=(world, _free_port(), opt, out, 2, False, "relu", options), nprocs=world, join=True)
    x, y, ws, bs = dpc.inputs()
    o = Oracle(dpc.LAYERS, "relu", opt, dpc.GLOBAL_BATCH, **options)
    o64 = Oracle(dpc.LAYERS, "relu", opt, dpc.GLOBAL_BATCH, real="f64", **options)
    for i, (w, b) in enumerate(zip(ws, bs)):
        o.set_params(i, w, b)
        o64.set_params(i, w, b)
    losses = []
    for _ in range(dpc.STEPS):
        o.step(x, y, 0.01)
        o64.step(x, y, 0.01)
        losses.append(o64.loss())
    pw, pw32 = o64.get_params()[0], o.get_params()[0]
    runs = [[np.load("%s/rank%d_rep%d.npz" % (out, r, rep)) for r in range(world)] for rep in range(2)]
    for rep in runs:
        for r in rep:
            np.testing.assert_allclose(r["losses"], losses, rtol=2e-5)
            for i in range(len(pw)):
                err = np.max(np.abs(r["w%d" % i] - pw[i])) / np.max(np.abs(pw[i]))
                ref = np.max(np.abs(pw32[i] - pw[i])) / np.max(np.abs(pw[i]))
                assert err <= max(2e-5, 4 * ref)
        for i in range(len(pw)):
            assert np.array_equal(rep[0]["w%d" % i], rep[1]["w%d" % i])
    for i in range(len(pw)):
        assert np.array_equal(runs[0][0]["w%d" % i], runs[1][0]["w%d" % i])
    assert np.array_equal(runs[0][0]["losses"], runs[1][0]["losses"])


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange", ["peer_kernel", "peer_copy"])
def test_a_rank_that_sits_a_step_out_is_detected_and_no_update_is_applied(monkeypatch, exchange):
    """Failure detection on the peer-memory paths, made on the host: rank 1 stays alive with its arena
    mapped but does not take the third step.  Rank 0's barrier gives up after its limit (200 ms), the
    reduce + update kernels then touch no rank's memory, the step reports VB200_ERR_DEVICE_WAIT, rank 0's
    parameters are bit-identical to before the step and further steps are refused.  No rank is killed."""
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    out = tempfile.mkdtemp()
    mp.spawn(dpc.gpu_missing_rank_worker, args=(2, _free_port(), out, 200, exchange), nprocs=2, join=True)
    r = np.load("%s/rank0.npz" % out)
    assert int(r["code"]) == 5 and "did not reach a barrier" in str(r["msg"])
    assert int(r["get_params_rc"]) == 5 and int(r["refused"]) == 5
    n = sum(1 for k in r.files if k.startswith("before"))
    for i in range(n):
        assert np.array_equal(r["before%d" % i].view(np.uint32), r["after%d" % i].view(np.uint32)), i
