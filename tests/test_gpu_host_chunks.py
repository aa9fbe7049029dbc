"""Large host inputs travel to the device in row chunks, and the forward pass (row-independent) runs as one
captured graph per chunk as soon as its rows have landed.  The rows, the kernels and every reduction over the
batch (dW, db, loss: taken after all chunks) are the same as in the single-graph step, so the result must not
depend on how the input arrived.  Forced here with VOLTA_B200_IN_CHUNKS on shapes the oracle finishes in
seconds; the automatic rule (>= 64 MB of input, chunks of >= 8192 rows) is exercised by bench.py's e2e leg."""
import numpy as np
import pytest
import torch

from oracle.oracle import Oracle
from volta_b200 import TrainHandle, synth

pytestmark = pytest.mark.gpu

LAYERS = [96, 160, 128, 1]
BATCH = 512
STEPS = 3


def _run(chunks, monkeypatch, device_inputs, opt="adam", act="silu", layers=LAYERS, gemm_path="auto"):
    monkeypatch.setenv("VOLTA_B200_IN_CHUNKS", str(chunks))
    x = synth.rows("uniform", 1234, 0, BATCH, layers[0])
    y = synth.rows("normal", 4321, 0, BATCH, layers[-1])
    ws, bs = synth.kaiming_uniform_weights(layers, 42)
    h = TrainHandle(layers, act, opt, BATCH, step_kernel=1, gemm_path=gemm_path)
    for i, (w, b) in enumerate(zip(ws, bs)):
        h.set_params(i, w, b)
    xi, yi = (torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()) if device_inputs else (x, y)
    losses = []
    for _ in range(STEPS):
        h.step(xi, yi, 0.01)
        losses.append(np.float32(h.loss()))
    params = sum(h.get_params(), [])
    h.free()
    return losses, params, (x, y, ws, bs)


@pytest.mark.parametrize("chunks", [2, 4, 8])
@pytest.mark.parametrize("opt", ["adam", "sgd_momentum"])
def test_chunked_host_inputs_agree_with_the_single_graph_step(monkeypatch, opt, chunks):
    """The chunked step (host inputs) against the single-graph step.  Device inputs never take the chunked path,
    so with the same switch they must give the single-graph bits; the chunked run itself repeats bit for bit; and
    the two agree to fp32 rounding (a chunk's GEMM may split its reduction differently from the full batch's)."""
    la, pa, _ = _run(chunks, monkeypatch, device_inputs=False, opt=opt)
    la2, pa2, _ = _run(chunks, monkeypatch, device_inputs=False, opt=opt)
    lb, pb, _ = _run(1, monkeypatch, device_inputs=False, opt=opt)
    lc, pc, _ = _run(chunks, monkeypatch, device_inputs=True, opt=opt)
    assert la == la2 and lb == lc
    np.testing.assert_allclose(la, lb, rtol=1e-5)
    for a, a2, b, c in zip(pa, pa2, pb, pc):
        assert np.array_equal(a.view(np.uint32), a2.view(np.uint32))
        assert np.array_equal(b.view(np.uint32), c.view(np.uint32))
        lim = 1e-4 if opt == "adam" else 2e-6   # Adam's update is sign-like where a gradient sits at the noise floor
        assert np.max(np.abs(a - b)) <= lim * max(float(np.max(np.abs(b))), 1e-30)


def test_chunked_step_matches_the_oracle(monkeypatch):
    losses, params, (x, y, ws, bs) = _run(4, monkeypatch, device_inputs=False, opt="sgd_momentum")
    o = Oracle(LAYERS, "silu", "sgd_momentum", BATCH)
    for i, (w, b) in enumerate(zip(ws, bs)):
        o.set_params(i, w, b)
    ref = []
    for _ in range(STEPS):
        o.step(x, y, 0.01)
        ref.append(o.loss())
    np.testing.assert_allclose(losses, ref, rtol=1e-5)
    pw, pb = o.get_params()
    for got, want in zip(params, pw + pb):
        assert np.max(np.abs(got - want)) <= 1e-5 * max(float(np.max(np.abs(want))), 1e-30)


def test_chunked_tensor_core_step_stays_within_the_tensor_path_tolerance(monkeypatch):
    """Tensor-core shapes (every GEMM on tcgen05 kernels): a chunk's GEMM may split K differently from the full
    batch's, so the bar is the tensor path's own tolerance against the unchunked run, and bit identity between two
    chunked runs."""
    layers = [512, 768, 512, 1]
    la, pa, _ = _run(2, monkeypatch, device_inputs=False, opt="sgd_momentum", layers=layers, gemm_path="tensor")
    lb, pb, _ = _run(1, monkeypatch, device_inputs=False, opt="sgd_momentum", layers=layers, gemm_path="tensor")
    lc, pc, _ = _run(2, monkeypatch, device_inputs=False, opt="sgd_momentum", layers=layers, gemm_path="tensor")
    np.testing.assert_allclose(la, lb, rtol=1e-5)
    for a, b, c in zip(pa, pb, pc):
        assert np.max(np.abs(a - b)) <= 2e-5 * max(float(np.max(np.abs(b))), 1e-30)
        assert np.array_equal(a.view(np.uint32), c.view(np.uint32))
