"""Failure paths on a GPU, without failing a GPU: a bounded device-side wait that is made to run out
(nobody ever writes the flag it waits for) returns an error status and leaves the context usable; the
non-finite guard reports what the reference's runtime loop reports; a Volta-named checkpoint imports."""
import ctypes as C
import time

import numpy as np
import pytest

from volta_b200 import TrainHandle, VoltaB200Error, synth
from volta_b200.checkpoint import Checkpoint

pytestmark = pytest.mark.gpu

ERR_DEVICE_WAIT, ERR_NONFINITE = 5, 8


def small():
    layers, B = [48, 64, 32, 1], 16
    return layers, B, synth.rows("normal", 1, 0, B, layers[0]), synth.rows("normal", 2, 0, B, 1)


def test_a_barrier_wait_that_nobody_answers_gives_up_and_the_handle_survives():
    """One barrier kernel with a declared world of two ranks on one GPU: the other rank's flag is never
    written.  The wait ends after its limit (50 ms here, 4 s by default), the status bit reaches the host as
    VB200_ERR_DEVICE_WAIT, later steps are refused, and the handle can still be read and destroyed; other
    handles on the same GPU are unaffected."""
    layers, B, x, y = small()
    g = TrainHandle(layers, "relu", "sgd", B)
    g.step(x, y, 0.01)
    before = [p.copy() for p in sum(g.get_params(), [])]
    t0 = time.perf_counter()
    with pytest.raises(VoltaB200Error) as e:
        g.dp_wait_selftest(2, 50)
    waited = time.perf_counter() - t0
    assert e.value.code == ERR_DEVICE_WAIT and "wait gave up" in str(e.value)
    assert 0.04 <= waited < 2.0, waited
    with pytest.raises(VoltaB200Error) as e2:      # sticky: no further steps
        g.step(x, y, 0.01)
    assert e2.value.code == ERR_DEVICE_WAIT
    with pytest.raises(VoltaB200Error):
        g.loss()
    # the parameters are still there, untouched (read through the C ABI, whose return code is the sticky status)
    fp = C.POINTER(C.c_float)
    wo, bo = (fp * g.n)(), (fp * g.n)()
    assert g.lib.volta_b200_get_params(g.h, wo, bo) == ERR_DEVICE_WAIT
    w0 = np.ctypeslib.as_array(wo[0], shape=(layers[0], layers[1]))
    assert np.array_equal(w0, before[0])
    g.free()
    h = TrainHandle(layers, "relu", "sgd", B)       # the context is healthy
    h.step(x, y, 0.01)
    assert np.isfinite(h.loss())
    h.free()


def test_selftest_arguments_are_checked():
    layers, B, x, y = small()
    g = TrainHandle(layers, "relu", "sgd", B)
    for world, ms in ((1, 50), (9, 50), (2, 0), (2, 20000)):
        with pytest.raises(VoltaB200Error) as e:
            g.dp_wait_selftest(world, ms)
        assert e.value.code == 1
    g.step(x, y, 0.01)           # refused calls leave the handle healthy
    assert np.isfinite(g.loss())
    g.free()


@pytest.mark.parametrize("opt", ["sgd", "adam"])
def test_non_finite_guard_names_the_first_bad_element(opt):
    """check_finite mirrors the fail-fast checks of the reference's runtime loop (src/engine/ir/train.rs:670-773:
    "Non-finite {stage} {label} at element {index}"); the generated step has none, and neither has a handle
    created without the switch."""
    layers, B, x, y = small()
    ws, bs = synth.kaiming_uniform_weights(layers, 42)
    bad = ws[1].copy()
    bad[3, 5] = np.nan
    for guarded in (False, True):
        g = TrainHandle(layers, "tanh", opt, B, check_finite=guarded)
        for i, (w, b) in enumerate(zip(ws, bs)):
            g.set_params(i, bad if i == 1 else w, b)
        g.step(x, y, 0.01)
        if not guarded:
            assert np.isnan(g.loss())           # as the reference's generated step: NaN flows, nothing is raised
        else:
            with pytest.raises(VoltaB200Error) as e:
                g.loss()
            assert e.value.code == ERR_NONFINITE
            assert str(e.value).split(": ", 1)[-1].startswith("Non-finite train gradient 'layer0.weight' at element 0")
            with pytest.raises(VoltaB200Error):
                g.step(x, y, 0.01)
        g.free()
    # an infinite target: the loss itself is the first thing that is not finite ... after the gradients it poisons
    g = TrainHandle(layers, "relu", opt, B, check_finite=True)
    yy = y.copy()
    yy[2, 0] = np.inf
    g.step(x, yy, 0.01)
    with pytest.raises(VoltaB200Error) as e:
        g.loss()
    assert e.value.code == ERR_NONFINITE and "Non-finite train" in str(e.value)
    g.free()


def test_guarded_healthy_run_is_bit_identical_to_the_unguarded_one():
    layers, B, x, y = small()
    out = []
    for guarded in (False, True):
        g = TrainHandle(layers, "silu", "adamw", B, check_finite=guarded)
        for _ in range(5):
            g.step(x, y, 1e-3)
        out.append((np.float32(g.loss()).view(np.uint32), [p.copy() for p in sum(g.get_params(), [])], g.kernels_per_step))
        g.free()
    assert out[0][0] == out[1][0]
    for a, b in zip(out[0][1], out[1][1]):
        assert np.array_equal(a, b)
    assert out[1][2] == out[0][2] + 1           # the guard is one more launch, and only when asked for


def test_checkpoint_with_volta_layer_names_imports(tmp_path):
    """A file as Volta's save_checkpoint writes it for a model whose layers are called fc1, fc2, fc3
    ("{name}.weight", "{name}.bias"; src/engine/model/layers.rs:52-58) loads into a handle, with and without
    the caller naming the layers; a file that names nothing of the topology is refused."""
    layers, B, x, y = small()
    src = TrainHandle(layers, "relu", "adam", B)
    for _ in range(3):
        src.step(x, y, 1e-3)
    names = ["fc1", "fc2", "fc3"]
    ck = src.export_checkpoint(with_state=True, layer_names=names)
    assert "fc2.weight" in ck.tensors() and "fc2.weight.m" in ck.tensors() and "layer0.weight" not in ck.tensors()
    p = tmp_path / "volta.ckpt"
    ck.save(p, 2)
    want = sum(src.get_params(), [])
    for given in (None, names):
        dst = TrainHandle(layers, "relu", "adam", B)
        dst.import_checkpoint(Checkpoint.load(p), layer_names=given)
        for a, b in zip(sum(dst.get_params(), []), want):
            assert np.array_equal(a, b)
        dst.free()
    # resumed training continues bit for bit (moments and step counter travelled under the same names)
    dst = TrainHandle(layers, "relu", "adam", B)
    dst.import_checkpoint(Checkpoint.load(p), layer_names=names)
    for hnd in (src, dst):
        hnd.step(x, y, 1e-3)
    assert np.float32(src.loss()).view(np.uint32) == np.float32(dst.loss()).view(np.uint32)
    for a, b in zip(sum(src.get_params(), []), sum(dst.get_params(), [])):
        assert np.array_equal(a, b)
    other = Checkpoint()
    other.add("encoder.weight", np.zeros((3, 3), np.float32))
    with pytest.raises(VoltaB200Error) as e:
        dst.import_checkpoint(other)
    assert e.value.code == 1
    dst.step(x, y, 1e-3)          # a refused import leaves the handle healthy
    assert np.isfinite(dst.loss())
    src.free()
    dst.free()
