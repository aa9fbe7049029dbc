"""GPU parity of the template's optional stages - softmax as hidden activation, LayerNorm, dropout
with the reference's LCG mask stream, the delta-scaling clip
(src/engine/ir/codegen/mlp_train_rust_codegen.rs:727-788, 829-916, 936-955) - against the oracle.

Floating-point results are judged against the fp64 oracle, with the fp32 oracle's own distance
from it as the yardstick (tolerance written in `close`); the dropout mask is integer work and must
agree bit for bit, which shows as gradients that agree to rounding on every step of a run (a single
flipped keep flag changes a whole row of dW by far more than the tolerance)."""
import numpy as np
import pytest

from oracle.oracle import Oracle
from volta_b200 import TrainHandle, VoltaB200Error, synth
from volta_b200.train import dp_unique_id

pytestmark = pytest.mark.gpu


def rel_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b)) / max(float(np.max(np.abs(b))), 1e-30))


def close(gpu, o32, o64, floor=2e-5):
    """gpu within max(floor, 4 x the fp32 oracle's own error) of the fp64 oracle, max-norm relative."""
    return rel_err(gpu, o64) <= max(floor, 4.0 * rel_err(o32, o64))


def trio(layers, act, opt, B, seed=0, **options):
    """GPU handle, fp32 oracle and fp64 oracle with the same weights and options."""
    ws, bs = synth.kaiming_uniform_weights(layers, 42)
    rs = np.random.RandomState(seed + 3)
    bs = [rs.randn(*b.shape).astype(np.float32) * 0.05 for b in bs]
    handle_kw = {k: options.pop(k) for k in list(options) if k in ("force_dp", "unique_id", "use_graph", "gemm_path")}
    g = TrainHandle(layers, act, opt, B, **options, **handle_kw)
    o32 = Oracle(layers, act, opt, B, real="f32", **options)
    o64 = Oracle(layers, act, opt, B, real="f64", **options)
    for i, (w, b) in enumerate(zip(ws, bs)):
        for h in (g, o32, o64):
            h.set_params(i, w, b)
    return g, o32, o64


def run_and_compare(layers, act, opt, B, steps=4, lr=1e-2, y_scale=1.0, **options):
    g, o32, o64 = trio(layers, act, opt, B, **options)
    x = synth.rows("normal", 1234, 0, B, layers[0])
    y = synth.rows("normal", 4321, 0, B, layers[-1]) * np.float32(y_scale)
    for step in range(steps):
        for h in (g, o32, o64):
            h.step(x, y, lr)
        assert abs(g.loss() - o64.loss()) <= max(2e-5 * abs(o64.loss()), 4 * abs(o32.loss() - o64.loss())), step
        if step == 0 and not (opt == "sgd" and options.get("fuse_sgd")):
            for a, b, c in zip(sum(g.get_grads(), []), sum(o32.get_grads(), []), sum(o64.get_grads(), [])):
                assert close(a, b, c), "gradient after the first step"
    # Adam's first steps are sign-like: a gradient element near zero moves its weight by +-lr either way
    floor = 2e-5 if opt in ("sgd", "adagrad", "sgd_momentum") else 5e-3
    for a, b, c in zip(sum(g.get_params(), []), sum(o32.get_params(), []), sum(o64.get_params(), [])):
        assert close(a, b, c, floor)
    return g, o32, o64


@pytest.mark.parametrize("opt", ["sgd", "adam"])
@pytest.mark.parametrize("layers,B", [([24, 40, 36, 3], 16), ([64, 300, 1000, 5], 70)])
def test_softmax_hidden_activation(opt, layers, B):
    g, _, _ = run_and_compare(layers, "softmax", opt, B, lr=0.05)
    g.free()


@pytest.mark.parametrize("act,opt", [("relu", "sgd"), ("gelu", "adam"), ("tanh", "adagrad"), ("leaky_relu", "adamw")])
def test_layernorm_and_its_own_sgd_update(act, opt):
    layers, B = [32, 300, 72, 4], 48
    g, o32, o64 = run_and_compare(layers, act, opt, B, use_layernorm=True)
    for li in range(len(layers) - 2):
        gg, gb = g.get_layernorm(li)
        (g32, b32), (g64, b64) = o32.get_layernorm(li), o64.get_layernorm(li)
        assert close(gg, g32, g64) and close(gb, b32, b64)
        assert np.max(np.abs(gg - 1.0)) > 0 and np.max(np.abs(gb)) > 0   # they did move
    g.free()


@pytest.mark.parametrize("layers,B,p", [([20, 40, 36, 3], 16, 0.25), ([64, 300, 1000, 5], 70, 0.5),
                                        ([16, 24, 2], 1500, 0.1)])
def test_dropout_mask_is_the_reference_lcg_stream(layers, B, p):
    """Widths below, between and above the CTA's 256 threads (one, two and four draws per thread),
    and more rows than CTAs; the stream position carries on from step to step."""
    g, _, _ = run_and_compare(layers, "relu", "sgd", B, steps=5, dropout_p=p)
    g.free()


def test_dropout_keep_flags_bit_for_bit():
    """With W0 = identity-like positive weights, relu and zero bias, the first hidden output is
    exactly keep * scale * x for positive x: read the keep flags back through the gradients' sparsity
    pattern and compare them with the integer recurrence restated here."""
    B, c, p = 6, 300, 0.3
    layers = [c, c, 1]
    g = TrainHandle(layers, "relu", "sgd", B, dropout_p=p)
    g.set_params(0, np.eye(c, dtype=np.float32), np.zeros(c, np.float32))
    g.set_params(1, np.ones((c, 1), np.float32), np.zeros(1, np.float32))
    x = np.abs(synth.rows("normal", 7, 0, B, c)) + np.float32(0.5)
    y = np.zeros((B, 1), np.float32)
    state = 12345678
    for step in range(3):
        g.step(x, y, 0.0)
        keep = np.empty(B * c, dtype=bool)
        for k in range(B * c):
            state = (state * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
            keep[k] = np.float32(state >> 33) / np.float32(2147483648.0) >= np.float32(p)
        # dW0[i, j] = sum_rows x[row, i] * delta0[row, j]; delta0[row, j] = keep * scale * w1[j] * seed(row) != 0
        # exactly where the flag is set (seed(row) = 2*out/nt > 0 here), so column j of dW0 is non-zero
        # iff some row kept j; the per-row pattern shows in db0 only summed, hence the one-row probes below
        dws, dbs = g.get_grads()
        kept_any = keep.reshape(B, c).any(axis=0)
        assert np.array_equal(dbs[0] != 0, kept_any), step
    g.free()
    # one row per handle: the flags themselves
    state = 12345678
    g = TrainHandle(layers, "relu", "sgd", 1, dropout_p=p)
    g.set_params(0, np.eye(c, dtype=np.float32), np.zeros(c, np.float32))
    g.set_params(1, np.ones((c, 1), np.float32), np.zeros(1, np.float32))
    for step in range(4):
        g.step(x[:1], y[:1], 0.0)
        keep = np.empty(c, dtype=bool)
        for k in range(c):
            state = (state * 6364136223846793005 + 1442695040888963407) & ((1 << 64) - 1)
            keep[k] = np.float32(state >> 33) / np.float32(2147483648.0) >= np.float32(p)
        assert np.array_equal(g.get_grads()[1][0] != 0, keep), step
    g.free()


def test_clip_scales_deltas_only_when_the_norm_exceeds_it():
    layers, B = [28, 44, 36, 2], 40
    x = synth.rows("normal", 1234, 0, B, layers[0])
    y = synth.rows("normal", 4321, 0, B, layers[-1]) * np.float32(3.0)
    probe = Oracle(layers, "relu", "sgd", B, real="f64")
    ws, bs = synth.kaiming_uniform_weights(layers, 42)
    rs = np.random.RandomState(3)
    bs = [rs.randn(*b.shape).astype(np.float32) * 0.05 for b in bs]
    for i, (w, b) in enumerate(zip(ws, bs)):
        probe.set_params(i, w, b)
    probe.grad_step(x, y)
    norm = float(np.sqrt(sum(np.sum(probe.get_delta(i) ** 2) for i in range(3))))
    for clip in (0.5 * norm, 10.0 * norm):
        g, o32, o64 = trio(layers, "relu", "sgd", B, clip_grad=clip)
        for h in (g, o32, o64):
            h.step(x, y, 1e-2)
        for a, b, c in zip(sum(g.get_grads(), []), sum(o32.get_grads(), []), sum(o64.get_grads(), [])):
            assert close(a, b, c)
        if clip < norm:   # dW halved, db untouched (it was summed before the scaling)
            gw, gb = g.get_grads()
            pw, pb = probe.get_grads()
            for a, b in zip(gw, pw):
                assert rel_err(a, 0.5 * b) <= 1e-4
            for a, b in zip(gb, pb):
                assert rel_err(a, b) <= 1e-4
        g.free()


@pytest.mark.parametrize("opt", ["adam", "sgd"])
def test_all_stages_together(opt):
    """relu -> LayerNorm -> dropout with the clip active, several steps.  (The reference rebuilds the
    LayerNorm input from the stored, already-dropped output in this combination; the oracle restates
    that, the GPU path follows.)"""
    g, _, _ = run_and_compare([32, 96, 300, 3], "relu", opt, 33, steps=4, y_scale=3.0, use_layernorm=True,
                              dropout_p=0.2, clip_grad=0.05)
    g.free()


def test_sgd_folded_into_dw_with_the_clip():
    layers, B = [64, 96, 80, 3], 32
    kw = dict(clip_grad=0.05, dropout_p=0.25)
    a = TrainHandle(layers, "relu", "sgd", B, **kw)
    b = TrainHandle(layers, "relu", "sgd", B, fuse_sgd=True, **kw)
    x = synth.rows("normal", 1234, 0, B, layers[0])
    y = synth.rows("normal", 4321, 0, B, layers[-1]) * np.float32(3.0)
    for _ in range(3):
        a.step(x, y, 1e-2)
        b.step(x, y, 1e-2)
    assert abs(a.loss() - b.loss()) <= 1e-6 * abs(a.loss())
    for p, q in zip(sum(a.get_params(), []), sum(b.get_params(), [])):
        assert rel_err(p, q) <= 1e-6
    a.free()
    b.free()


@pytest.mark.parametrize("act,ln", [("softmax", False), ("relu", True), ("softmax", True)])
def test_infer_applies_softmax_and_layernorm_but_never_dropout(act, ln):
    layers, B = [24, 300, 40, 3], 32
    g, o32, o64 = trio(layers, act, "sgd", B, use_layernorm=ln)
    gd = TrainHandle(layers, act, "sgd", B, use_layernorm=ln, dropout_p=0.5)
    for i, (w, b) in enumerate(zip(*g.get_params())):
        gd.set_params(i, w, b)
    x = synth.rows("normal", 99, 0, B, layers[0])
    y = np.zeros((B, layers[-1]), np.float32)
    o32.grad_step(x, y)
    o64.grad_step(x, y)
    n = len(layers) - 1
    out = g.infer(x)
    assert close(out, o32.get_act(n).reshape(B, -1), o64.get_act(n).reshape(B, -1))
    assert np.array_equal(out, gd.infer(x))
    part = g.infer(x[:5])                     # at most 8 rows: another kernel, same values to rounding
    assert rel_err(part, out[:5]) <= 1e-5
    assert np.array_equal(g.infer(x[:16]), out[:16])
    g.free()
    gd.free()


def test_steps_with_every_stage_are_bit_identical_run_to_run():
    layers, B = [64, 512, 300, 4], 256
    x = synth.rows("normal", 1234, 0, B, layers[0])
    y = synth.rows("normal", 4321, 0, B, layers[-1])
    runs = []
    for _ in range(2):
        g = TrainHandle(layers, "gelu", "adam", B, use_layernorm=True, dropout_p=0.3, clip_grad=0.01)
        for _ in range(6):
            g.step(x, y, 1e-3)
        runs.append((np.float32(g.loss()), g.get_params(), [g.get_layernorm(i) for i in range(2)]))
        g.free()
    assert runs[0][0].view(np.uint32) == runs[1][0].view(np.uint32)
    for p, q in zip(sum(runs[0][1], []), sum(runs[1][1], [])):
        assert np.array_equal(p, q)
    for (a, b), (c, d) in zip(runs[0][2], runs[1][2]):
        assert np.array_equal(a, c) and np.array_equal(b, d)


def test_state_carries_the_mask_stream_position():
    layers, B = [16, 40, 1], 8
    x = synth.rows("normal", 1, 0, B, 16)
    y = synth.rows("normal", 2, 0, B, 1)
    kw = dict(dropout_p=0.4, use_layernorm=True)
    a = TrainHandle(layers, "relu", "adam", B, **kw)
    for _ in range(3):
        a.step(x, y, 1e-2)
    state, t = a.save_state()
    assert state.size == 2 * a.state_offsets()[2] + 2
    ws, bs = a.get_params()
    b = TrainHandle(layers, "relu", "adam", B, **kw)
    for i in range(2):
        b.set_params(i, ws[i], bs[i])
    b.set_layernorm(0, *a.get_layernorm(0))
    b.load_state(state, t)
    for _ in range(3):
        a.step(x, y, 1e-2)
        b.step(x, y, 1e-2)
    assert np.float32(a.loss()).view(np.uint32) == np.float32(b.loss()).view(np.uint32)
    for p, q in zip(sum(a.get_params(), []), sum(b.get_params(), [])):
        assert np.array_equal(p, q)
    a.free()
    b.free()


def test_single_rank_data_parallel_path_with_every_stage_equals_the_plain_path():
    """World size one through the communicator: the all-reduces (LayerNorm gradients in the last
    bucket, the clip's norm in mid-step) are identities, so the results must not change by a bit."""
    layers, B = [32, 96, 300, 3], 40
    kw = dict(use_layernorm=True, dropout_p=0.2, clip_grad=0.05)
    x = synth.rows("normal", 1234, 0, B, layers[0])
    y = synth.rows("normal", 4321, 0, B, layers[-1]) * np.float32(3.0)
    a = TrainHandle(layers, "relu", "adam", B, **kw)
    b = TrainHandle(layers, "relu", "adam", B, force_dp=True, unique_id=dp_unique_id(), **kw)
    for _ in range(4):
        a.step(x, y, 1e-2)
        b.step(x, y, 1e-2)
    assert np.float32(a.loss()).view(np.uint32) == np.float32(b.loss()).view(np.uint32)
    for p, q in zip(sum(a.get_params(), []), sum(b.get_params(), [])):
        assert np.array_equal(p, q)
    assert np.array_equal(a.get_layernorm(1)[0], b.get_layernorm(1)[0])
    a.free()
    b.free()


def test_option_arguments_are_validated():
    for kw in (dict(dropout_p=1.0), dict(dropout_p=-0.1), dict(clip_grad=-1.0)):
        with pytest.raises(VoltaB200Error):
            TrainHandle([4, 4, 1], "relu", "sgd", 2, **kw)
    with pytest.raises(VoltaB200Error):
        TrainHandle([4, 60000, 1], "softmax", "sgd", 2)
    g = TrainHandle([4, 4, 1], "relu", "sgd", 2)
    with pytest.raises(VoltaB200Error):
        g.get_layernorm(0)
    g.step(np.zeros((2, 4), np.float32), np.zeros((2, 1), np.float32), 0.1)   # the handle stays usable
    assert g.loss() == 0.0
    g.free()


@pytest.mark.parametrize("fmt", [1, 2])
@pytest.mark.parametrize("opt", ["adam", "adagrad", "sgd_momentum"])
def test_checkpoint_file_resumes_training_bit_exactly(tmp_path, fmt, opt):
    """export -> file in the reference's v1 text / v2 binary format -> load -> import into a fresh
    handle: parameters, LayerNorm scale/shift, optimizer moments, the Adam counter and the mask
    stream position all travel, so both handles continue identically."""
    from volta_b200.checkpoint import Checkpoint
    layers, B = [16, 40, 24, 2], 8
    x = synth.rows("normal", 1, 0, B, 16)
    y = synth.rows("normal", 2, 0, B, 2)
    kw = dict(dropout_p=0.4, use_layernorm=True)
    a = TrainHandle(layers, "gelu", opt, B, **kw)
    for _ in range(3):
        a.step(x, y, 1e-2)
    path = tmp_path / "ck"
    a.export_checkpoint().save(path, fmt)
    ck = Checkpoint.load(path)
    names = set(ck.tensors())
    assert {"layer0.weight", "layer2.bias", "layer1.ln_gamma", "meta.dropout_rng"} <= names
    assert ("meta.adam_step" in names) == (opt == "adam")
    b = TrainHandle(layers, "gelu", opt, B, **kw)
    b.import_checkpoint(ck)
    for _ in range(3):
        a.step(x, y, 1e-2)
        b.step(x, y, 1e-2)
    assert np.float32(a.loss()).view(np.uint32) == np.float32(b.loss()).view(np.uint32)
    for p, q in zip(sum(a.get_params(), []), sum(b.get_params(), [])):
        assert np.array_equal(p, q)
    # parameters only: what the reference's own checkpoint holds
    only = a.export_checkpoint(with_state=False).tensors()
    assert not any(n.startswith("meta.") or n.endswith((".m", ".v", ".acc", ".mom")) for n in only)
    # a tensor of the wrong shape is refused and the handle stays usable
    bad = Checkpoint()
    bad.add("layer0.weight", np.zeros((16, 41), np.float32))
    with pytest.raises(VoltaB200Error, match="wrong shape"):
        b.import_checkpoint(bad)
    b.step(x, y, 1e-2)
    a.free()
    b.free()


@pytest.mark.parametrize("act,kw", [("relu", {"dropout_p": 0.2}), ("relu", {"use_layernorm": True}), ("softmax", {})])
def test_reference_option_examples_at_full_size(act, kw):
    """examples/bench_dropout.vt, bench_layernorm.vt, bench_softmax.vt: layers 512 1024 1024 512 256 1,
    batch 64, SGD lr 0.01 - against the oracle at full size."""
    g, _, _ = run_and_compare([512, 1024, 1024, 512, 256, 1], act, "sgd", 64, steps=4, lr=0.01, **kw)
    g.free()


def test_generated_inference_library_embeds_the_checkpoint(tmp_path):
    """`volta-b200-codegen --infer --checkpoint F`: one exported function, volta_infer(in, in_n, out, out_n)
    (src/engine/ir/codegen/inner.rs:194-198), weights from the embedded checkpoint file; called the way
    examples/bench_infer.c calls it (one row, then 64 rows), then with more rows than the first handle holds."""
    import ctypes as C
    from volta_b200 import codegen
    layers = [48, 300, 64, 3]
    g = TrainHandle(layers, "gelu", "adam", 200, use_layernorm=True)
    x = synth.rows("normal", 5, 0, 200, layers[0])
    y = synth.rows("normal", 6, 0, 200, layers[-1])
    for _ in range(3):
        g.step(x, y, 1e-2)
    ck = tmp_path / "model.ckpt"
    g.export_checkpoint(with_state=False).save(ck, 2)
    lib = C.CDLL(codegen.compile_model(layers, "gelu", "adam", str(tmp_path / "model.infer.so"), infer=True,
                                       checkpoint=str(ck), use_layernorm=True))
    fp = C.POINTER(C.c_float)
    lib.volta_infer.argtypes = [fp, C.c_int64, fp, C.c_int64]
    lib.volta_infer.restype = None
    want = g.infer(x)
    for rows in (1, 64, 1, 200, 64):
        out = np.full((rows, layers[-1]), np.nan, np.float32)
        xin = np.ascontiguousarray(x[:rows])
        lib.volta_infer(xin.ctypes.data_as(fp), xin.size, out.ctypes.data_as(fp), out.size)
        assert np.array_equal(out, g.infer(xin)), rows
        assert rel_err(out, want[:rows]) <= 1e-5
    bad = np.full((1, layers[-1]), 7.0, np.float32)   # lengths that do not fit: a no-op
    lib.volta_infer(x.ctypes.data_as(fp), 47, bad.ctypes.data_as(fp), bad.size)
    assert np.all(bad == 7.0)
    g.free()
