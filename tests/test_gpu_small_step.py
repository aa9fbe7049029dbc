"""The persistent step kernel (one launch per step for batches of at most 64 rows) against the CPU oracle, the
per-kernel schedule of the same library, and itself run twice.  step_kernel = 2 makes creation fail where the
kernel does not apply, so these tests cannot pass on the other path by accident."""
import numpy as np
import pytest
import torch

from oracle.oracle import Oracle
from tests.test_gpu_parity import LOSS_TOL, assert_one_step_parity, rel_err
from volta_b200 import CONFIGS, TrainHandle, VoltaB200Error, synth

pytestmark = pytest.mark.gpu


def pair(layers, act, opt, B, step_kernel=2, seed=0):
    ws, bs = synth.kaiming_uniform_weights(layers, 42)
    rs = np.random.RandomState(seed + 3)
    bs = [(rs.randn(*b.shape) * 0.05).astype(np.float32) for b in bs]
    g = TrainHandle(layers, act, opt, B, step_kernel=step_kernel)
    o = Oracle(layers, act, opt, B)
    for i, (w, b) in enumerate(zip(ws, bs)):
        g.set_params(i, w, b)
        o.set_params(i, w, b)
    return g, o


@pytest.mark.parametrize("act", ["relu", "sigmoid", "tanh", "leaky_relu", "silu", "gelu"])
@pytest.mark.parametrize("opt", ["sgd", "adam", "adamw", "adagrad", "sgd_momentum"])
def test_every_activation_and_optimizer(act, opt):
    layers, B = [24, 40, 36, 3], 16        # last width 3: the loaders' scalar path
    g, o = pair(layers, act, opt, B)
    assert g.kernels_per_step == 1
    x = synth.rows("normal", 1234, 0, B, layers[0])
    y = synth.rows("normal", 4321, 0, B, layers[-1])
    before = o.state()
    for step in range(5):
        g.step(x, y, 1e-2)
        o.step(x, y, 1e-2)
        assert abs(g.loss() - o.loss()) <= 1e-5 * abs(o.loss())
        if step == 0:
            assert_one_step_parity(g, o, opt, 1e-2, before)
    for a, b in zip(sum(g.get_params(), []), sum(o.get_params(), [])):
        assert rel_err(a, b) <= 1e-4
    g.free()


SHAPES = [
    ([256, 512, 512, 256, 1], 64),          # configuration 1
    ([512, 1024, 1024, 512, 256, 1], 64),   # configuration 2
    ([512, 2048, 2048, 512, 1], 64),        # configuration 3: two staged tiles per phase, widest slabs
    ([5, 9, 2], 3),                         # nothing a multiple of four
    ([100, 2100, 36, 7], 61),               # close to the widest layer the kernel takes; ragged batch
    ([64, 64], 1),                          # one layer, one row
    ([300, 20, 300, 20, 4], 33),
    # width-one outputs, which get no phases of their own: behind the FIRST layer (no barrier ahead of the partial
    # dot products), behind the widest hidden layer the kernel takes (16 rows of the output weights per CTA), behind
    # a hidden layer narrower than the cluster count (most clusters write no partial), a ragged batch, and a
    # single-layer model (nothing to fuse into: the output layer keeps its own phases)
    ([40, 2100, 1], 61),
    ([128, 24, 1], 5),
    ([96, 160, 130, 1], 64),
    ([70, 1], 9),
]


@pytest.mark.parametrize("layers,B", SHAPES)
@pytest.mark.parametrize("act,opt", [("relu", "adam"), ("gelu", "sgd_momentum")])
def test_shapes_against_the_oracle_and_the_per_kernel_schedule(layers, B, act, opt):
    g, o = pair(layers, act, opt, B)
    k, _ = pair(layers, act, opt, B, step_kernel=1)
    assert g.kernels_per_step == 1 and k.kernels_per_step > 1
    x = synth.rows("normal", 1234, 0, B, layers[0])
    y = synth.rows("normal", 4321, 0, B, layers[-1])
    lr = 1e-3 if opt == "adam" else 1e-2
    before = o.state()
    for step in range(3):
        for h in (g, k, o):
            h.step(x, y, lr)
        # the first step from identical state is held to the one-step bars; later steps of an Adam run
        # amplify any admissible difference (sign-like updates near zero gradients), so they get the
        # bar stated for whole runs
        tol = 1e-5 if step == 0 else LOSS_TOL
        assert abs(g.loss() - o.loss()) <= tol * abs(o.loss()), step
        assert abs(g.loss() - k.loss()) <= tol * abs(k.loss()), step
        if step == 0:
            assert_one_step_parity(g, o, opt, lr, before)
    g.free()
    k.free()


@pytest.mark.parametrize("name", ["c1", "c2", "c3_b64"])
def test_benchmark_configurations_repeat_bit_for_bit_and_hold_the_loss_bar(name):
    cfg = CONFIGS[name]
    layers, B = list(cfg.layers), cfg.batch
    ws, bs = synth.kaiming_uniform_weights(layers, 42)
    x = synth.rows(cfg.x_dist, 1234, 0, B, layers[0])
    y = synth.rows(cfg.y_dist, 4321, 0, B, layers[-1])
    runs = []
    for _ in range(2):
        g = TrainHandle(layers, cfg.activation, cfg.optimizer, B, step_kernel=2)
        for i, (w, b) in enumerate(zip(ws, bs)):
            g.set_params(i, w, b)
        losses = []
        for _ in range(8):
            g.step(x, y, cfg.lr)
            losses.append(np.float32(g.loss()).view(np.uint32))
        runs.append((losses, [p.view(np.uint32).copy() for p in sum(g.get_params(), [])]))
        g.free()
    assert runs[0][0] == runs[1][0]
    for a, b in zip(runs[0][1], runs[1][1]):
        assert np.array_equal(a, b)


def test_inputs_on_the_device_plain_launches_profile_and_inference():
    layers, B = [64, 96, 48, 2], 32
    x = synth.rows("normal", 1, 0, B, layers[0])
    y = synth.rows("normal", 2, 0, B, layers[-1])
    out = []
    for mode in ("host", "device", "plain"):
        g = TrainHandle(layers, "silu", "adamw", B, step_kernel=2, use_graph=(mode != "plain"))
        xs, ys = (torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()) if mode == "device" else (x, y)
        for _ in range(4):
            g.step(xs, ys, 1e-3)
        out.append((np.float32(g.loss()).view(np.uint32), [p.copy() for p in sum(g.get_params(), [])]))
        if mode == "host":
            recs = g.profile_step(x, y, 1e-3)          # one more step, as plain launches with events
            assert [r[0] for r in recs] == ["small_step"] and recs[0][1] > 0.0
            o = Oracle(layers, "silu", "adamw", B)
            for i, (w, b) in enumerate(zip(*g.get_params())):
                o.set_params(i, w, b)
            o.grad_step(x, y)
            assert rel_err(g.infer(x), o.get_act(o.n)) <= 1e-5
        g.free()
    for other in out[1:]:
        assert other[0] == out[0][0]
        for a, b in zip(other[1], out[0][1]):
            assert np.array_equal(a, b)


def test_where_the_kernel_does_not_apply_it_is_refused_or_bypassed():
    with pytest.raises(VoltaB200Error) as e:
        TrainHandle([32, 32, 1], "relu", "sgd", 65, step_kernel=2)            # more than 64 rows
    assert e.value.code == 6
    with pytest.raises(VoltaB200Error):
        TrainHandle([32, 4096, 1], "relu", "sgd", 8, step_kernel=2)           # wider than the slabs allow
    with pytest.raises(VoltaB200Error):
        TrainHandle([32, 32, 1], "relu", "sgd", 8, step_kernel=2, dropout_p=0.1)
    g = TrainHandle([32, 4096, 1], "relu", "sgd", 8)                           # auto: the per-kernel schedule
    assert g.kernels_per_step > 1
    g.free()
    g = TrainHandle([32, 32, 1], "relu", "sgd", 8, gemm_path="ffma")           # an explicit GEMM path also means per-kernel
    assert g.kernels_per_step > 1
    g.free()


@pytest.mark.parametrize("opt", ["adam", "adamw", "adagrad"])
@pytest.mark.parametrize("wide", [0, 1])
def test_step_kernel_optimizer_arithmetic_equals_the_streaming_optimizers(opt, wide):
    """The persistent kernel runs its elements side by side through straight-line division / square-root cores
    (vb_optimizer.cuh) where the streaming optimizer calls the library's IEEE routines.  Bit for bit the same, on
    operands from the range training produces (nearly all groups take the cores) and on operands from all
    exponents (most groups fail the pre-check and take the library path; those at the edges of the cores' range
    do not)."""
    import ctypes as C
    from volta_b200 import load_library
    lib = load_library()
    code = {"adam": 1, "adamw": 2, "adagrad": 3}[opt]
    for t in (1, 7, 100000):
        counts = (C.c_uint64 * 3)()
        groups = 1 << 22
        rc = lib.volta_b200_update_selftest(code, 20240 + t, groups, wide, t, C.byref(counts))
        assert rc == 0
        assert counts[1] + counts[2] == groups
        assert counts[0] == 0, (opt, wide, t, list(counts))
        if wide:
            assert counts[1] > 1000 and counts[2] > groups // 2
        else:
            # (Adagrad's sum is drawn with either sign here; a negative one sends its group to the library path)
            assert counts[1] > groups * (0.02 if opt == "adagrad" else 0.9)
