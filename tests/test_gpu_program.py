"""Runtime-backend slice on the GPU: every op against numpy (float64) on seeded inputs, the MLP
training graph as the runtime builds it (forward + autograd nodes) fused and unfused, a training
loop through bind/run/update against the reference's PyTorch parity fixtures
(tests/pytorch_parity.rs:1949-2417, tolerance 1e-5 as there) and against the oracle at a larger size."""
import json
import os

import numpy as np
import pytest

from oracle.oracle import Oracle
from tests.program_common import evaluate, mlp_training_graph
from volta_b200 import VoltaB200Error, synth
from volta_b200.program import GraphBuilder, Program

pytestmark = pytest.mark.gpu
GOLD = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "mlp_parity.json")))


def run_graph(g, feed, outputs, fuse=True):
    p = g.emit(Program(), outputs)
    info = p.compile(fuse)
    for vid, arr in feed.items():
        p.bind(vid, np.asarray(arr, np.float32))
    p.run()
    got = {v: p.fetch(v, g.shape[v]) for v in outputs}
    p.free()
    return got, info


def close(a, ref, tol=2e-6):
    ref = np.asarray(ref, np.float64)
    return float(np.max(np.abs(np.asarray(a, np.float64) - ref))) <= tol * max(float(np.max(np.abs(ref))), 1e-30)


BINARY_SHAPES = [((7, 33), (7, 33)), ((7, 33), (1, 33)), ((7, 33), (33,)), ((7, 33), (7, 1)), ((1, 33), (7, 1)),
                 ((7, 33), ()), ((1,), (5, 4)), ((300, 260), (300, 260))]


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("sa,sb", BINARY_SHAPES)
def test_binary_ops_broadcast_like_the_reference(op, sa, sb):
    rs = np.random.RandomState(len(sa) * 7 + len(sb))
    g = GraphBuilder()
    a, b = g.input(sa), g.input(sb)
    out = getattr(g, op)(a, b)
    feed = {a: rs.randn(*sa).astype(np.float32), b: (np.abs(rs.randn(*sb)) + 0.5).astype(np.float32)}
    got, _ = run_graph(g, feed, [out])
    want = evaluate(g, feed)[out]
    assert got[out].shape == want.shape and close(got[out], want)


@pytest.mark.parametrize("op", ["neg", "relu", "sigmoid", "gelu", "exp", "log", "softmax", "transpose", "identity"])
@pytest.mark.parametrize("shape", [(5, 37), (64, 300), (1, 1000)])
def test_unary_ops(op, shape):
    rs = np.random.RandomState(3)
    g = GraphBuilder()
    a = g.input(shape)
    out = getattr(g, op)(a)
    x = rs.randn(*shape).astype(np.float32)
    feed = {a: np.abs(x) + 0.1 if op == "log" else x}
    got, _ = run_graph(g, feed, [out])
    assert close(got[out], evaluate(g, feed)[out])


@pytest.mark.parametrize("op", ["relu_backward", "sigmoid_backward", "gelu_backward"])
def test_activation_backward_takes_the_input_and_the_upstream_gradient(op):
    rs = np.random.RandomState(4)
    g = GraphBuilder()
    x, up = g.input((33, 70)), g.input((33, 70))
    out = getattr(g, op)(x, up)
    feed = {x: rs.randn(33, 70).astype(np.float32), up: rs.randn(33, 70).astype(np.float32)}
    got, _ = run_graph(g, feed, [out])
    assert close(got[out], evaluate(g, feed)[out])


@pytest.mark.parametrize("kind", ["reduce_sum", "reduce_mean"])
@pytest.mark.parametrize("shape,axis,keep", [((40, 70), None, False), ((40, 70), None, True), ((40, 70), 0, False),
                                             ((40, 70), 0, True), ((40, 70), 1, False), ((40, 70), 1, True),
                                             ((5000,), 0, False), ((5000,), None, False), ((3000, 130), 0, False),
                                             ((300, 5000), 1, False), ((), None, False)])
def test_reductions(kind, shape, axis, keep):
    rs = np.random.RandomState(5)
    g = GraphBuilder()
    a = g.input(shape)
    out = getattr(g, kind)(a, axis, keep)
    feed = {a: np.asarray(rs.randn(*shape), np.float32)}
    got, _ = run_graph(g, feed, [out])
    want = evaluate(g, feed)[out]
    scale = float(np.sum(np.abs(feed[a]), axis=axis).max()) / (1 if kind == "reduce_sum" else max(1, feed[a].size if axis is None else (shape[axis] if shape else 1)))
    assert got[out].shape == want.shape
    assert float(np.max(np.abs(got[out] - want))) <= 2e-6 * max(scale, 1e-30)


@pytest.mark.parametrize("m,k,n", [(1, 64, 48), (5, 33, 7), (64, 512, 1024), (300, 260, 72), (2048, 1024, 512)])
@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (False, True), (True, True)])
def test_matmul_with_transposed_operands_folded_or_not(m, k, n, ta, tb):
    rs = np.random.RandomState(m + n)
    A, B = rs.randn(k, m) if ta else rs.randn(m, k), rs.randn(n, k) if tb else rs.randn(k, n)
    res = {}
    for fuse in (True, False):
        g = GraphBuilder()
        a, b = g.input(A.shape), g.input(B.shape)
        out = g.matmul(g.transpose(a) if ta else a, g.transpose(b) if tb else b)
        got, info = run_graph(g, {a: A.astype(np.float32), b: B.astype(np.float32)}, [out], fuse)
        res[fuse] = got[out]
        expect = 1 + (int(ta) + int(tb) if not fuse else int(ta and tb))   # both transposed: only the right one folds
        assert info.launches == expect
    ref = (A.T if ta else A).astype(np.float32).astype(np.float64) @ (B.T if tb else B).astype(np.float32).astype(np.float64)
    scale = np.abs(A.T if ta else A) @ np.abs(B.T if tb else B)
    for fuse in (True, False):
        assert np.max(np.abs(res[fuse] - ref) / scale) <= 4e-7


@pytest.mark.parametrize("activation", ["relu", "sigmoid", "gelu"])
@pytest.mark.parametrize("layers,batch", [((16, 32, 4), 8), ((64, 300, 130, 10), 96), ((256, 512, 512, 256, 1), 64)])
def test_mlp_training_graph_fused_and_unfused_match_numpy(activation, layers, batch):
    g, x, y, pred, loss, params, grads = mlp_training_graph(layers, batch, activation)
    rs = np.random.RandomState(9)
    feed = {x: rs.randn(batch, layers[0]).astype(np.float32), y: rs.randn(batch, layers[-1]).astype(np.float32)}
    ws, bs = synth.kaiming_uniform_weights(list(layers), 42)
    for i in range(len(layers) - 1):
        feed[params[2 * i]] = ws[i]
        feed[params[2 * i + 1]] = (rs.randn(1, layers[i + 1]) * 0.05).astype(np.float32)
    want = evaluate(g, feed)
    outs = [loss, pred] + grads
    fused, fi = run_graph(g, feed, outs, True)
    plain, pi = run_graph(g, feed, outs, False)
    assert fi.launches < pi.launches and fi.peak_bytes <= pi.peak_bytes
    for v in outs:
        assert close(fused[v], want[v], 1e-5) and close(plain[v], want[v], 1e-5), v
    # the same gradients as the compiled training step's oracle (W [in x out], MSE mean over all elements)
    if activation != "sigmoid" or True:
        o = Oracle(list(layers), activation, "sgd", batch, real="f64")
        for i in range(len(layers) - 1):
            o.set_params(i, feed[params[2 * i]], feed[params[2 * i + 1]].ravel())
        o.grad_step(feed[x], feed[y])
        gw, gb = o.get_grads()
        for i in range(len(layers) - 1):
            assert close(fused[grads[2 * i]], gw[i], 1e-5) and close(fused[grads[2 * i + 1]].ravel(), gb[i], 1e-5)


@pytest.mark.parametrize("batch,classes", [(6, 5), (64, 10), (700, 1000), (3000, 37)])
def test_softmax_cross_entropy_loss_and_its_gradient(batch, classes):
    """SoftmaxCrossEntropyLossFromLogits (interpreter.rs:776-815) with one-hot targets behind a small classifier,
    and the gradient nodes autograd.rs:467-530 emits for it (Softmax, Sub, Div by the batch size, Mul)."""
    rs = np.random.RandomState(batch)
    g = GraphBuilder()
    x, t = g.input((batch, 24)), g.input((batch, classes))
    logits, params = g.mlp([24, 48, classes], "relu", x)
    loss = g.softmax_xent(logits, t)
    grads = g.backward(loss, params)
    feed = {x: rs.randn(batch, 24).astype(np.float32), t: np.eye(classes, dtype=np.float32)[rs.randint(0, classes, batch)]}
    ws, bs = synth.kaiming_uniform_weights([24, 48, classes], 42)
    for i in range(2):
        feed[params[2 * i]], feed[params[2 * i + 1]] = ws[i], (rs.randn(1, ws[i].shape[1]) * 0.1).astype(np.float32)
    want = evaluate(g, feed)
    got, _ = run_graph(g, feed, [loss] + grads)
    assert got[loss].shape == () and abs(float(got[loss]) - float(want[loss])) <= 2e-6 * abs(float(want[loss]))
    for v in grads:
        assert close(got[v], want[v], 1e-5)
    import torch
    tw = [torch.tensor(feed[p_], dtype=torch.float64, requires_grad=True) for p_ in params]
    h = torch.relu(torch.tensor(feed[x], dtype=torch.float64) @ tw[0] + tw[1]) @ tw[2] + tw[3]
    ref = torch.nn.functional.cross_entropy(h, torch.tensor(feed[t].argmax(axis=1)))
    ref.backward()
    assert abs(float(got[loss]) - float(ref.detach())) <= 1e-5 * abs(float(ref.detach()))
    for v, w in zip(grads, tw):
        assert close(got[v], w.grad.numpy(), 1e-5)


def fixture_program(activation="relu"):
    g = GraphBuilder()
    B, L = GOLD["batch"], GOLD["layers"]
    x, y = g.input((B, L[0])), g.input((B, L[-1]))
    pred, params = g.mlp(L, activation, x)
    loss = g.mse(pred, y)
    grads = g.backward(loss, params)
    p = g.emit(Program(), [loss] + grads)
    p.compile()
    return g, p, x, y, loss, params, grads


@pytest.mark.parametrize("name,opt", [("sgd", "sgd"), ("adam", "adam"), ("adamw", "adamw"), ("adagrad", "adagrad"),
                                      ("long_sgd", "sgd"), ("long_adam", "adam"), ("long_adamw", "adamw")])
def test_training_loop_through_the_backend_calls_reproduces_the_reference_fixtures(name, opt):
    """compile once; per sample bind x, y -> run -> fetch the loss -> update (apply_gradients), parameters
    resident on the device throughout.  AdamW here is the runtime's (decay on every tensor), which is what the
    PyTorch vectors hold."""
    case, hp, init = GOLD["cases"]["mlp_train_loop_" + name], GOLD["hyper"][name], GOLD["init"]
    g, p, x, y, loss, params, grads = fixture_program()
    L = GOLD["layers"]
    for vid, key, shape in zip(params, ("w1", "b1", "w2", "b2"), ((L[0], L[1]), (1, L[1]), (L[1], L[2]), (1, L[2]))):
        p.bind(vid, np.array(init[key], np.float32).reshape(shape))
    trace, t = [], 0
    for _ in range(hp["epochs"]):
        for d in GOLD["dataset"]:
            p.bind(x, np.array(d["x"], np.float32))
            p.bind(y, np.array(d["y"], np.float32))
            p.run()
            trace.append(float(p.fetch(loss, ())))
            t += 1
            p.update(opt, params, grads, hp["lr"], t, weight_decay=0.01 if opt == "adamw" else 0.0)
    np.testing.assert_allclose(trace, case["loss_trace"], atol=1e-5)
    for vid, key in zip(params, ("w1", "b1", "w2", "b2")):
        np.testing.assert_allclose(p.fetch(vid, g.shape[vid]).ravel(), case["final_parameters"][key], atol=1e-5)
    p.free()


def test_training_loop_matches_the_oracle_at_a_benchmark_size_and_is_reproducible():
    layers, batch, steps, lr = (256, 512, 512, 256, 1), 64, 6, 0.01
    ws, bs = synth.kaiming_uniform_weights(list(layers), 42)
    xs = synth.rows("uniform", 1234, 0, batch, layers[0])
    ys = synth.rows("normal", 4321, 0, batch, layers[-1])
    o = Oracle(list(layers), "relu", "adam", batch)
    for i, (w, b) in enumerate(zip(ws, bs)):
        o.set_params(i, w, b)
    ref = []
    for _ in range(steps):
        o.step(xs, ys, lr)
        ref.append(o.loss())
    runs = []
    for _ in range(2):
        g, x, y, pred, loss, params, grads = mlp_training_graph(layers, batch, "relu")
        p = g.emit(Program(), [loss] + grads)
        p.compile()
        for i in range(len(layers) - 1):
            p.bind(params[2 * i], ws[i])
            p.bind(params[2 * i + 1], bs[i].reshape(1, -1))
        p.bind(x, xs)
        p.bind(y, ys)
        trace = []
        for t in range(1, steps + 1):
            p.run()
            trace.append(float(p.fetch(loss, ())))
            p.update("adam", params, grads, lr, t)
        runs.append((trace, [p.fetch(v, g.shape[v]) for v in params]))
        p.free()
    np.testing.assert_allclose(runs[0][0], ref, rtol=1e-4)
    assert runs[0][0] == runs[1][0]
    for a, b in zip(runs[0][1], runs[1][1]):
        assert np.array_equal(a, b)


def test_temporaries_are_not_fetchable_and_bind_checks_its_target():
    g = GraphBuilder()
    a = g.input((4, 4))
    t = g.relu(a)
    out = g.output(g.neg(t))
    p = g.emit(Program())
    p.compile()
    p.bind(a, np.eye(4, dtype=np.float32))
    p.run()
    assert np.array_equal(p.fetch(out, (4, 4)), -np.eye(4, dtype=np.float32))
    with pytest.raises(VoltaB200Error, match="is a temporary"):
        p.fetch(t, (4, 4))
    with pytest.raises(VoltaB200Error, match="neither an input nor a parameter"):
        p.bind(t, np.zeros((4, 4), np.float32))
    with pytest.raises(VoltaB200Error, match="takes 16 floats"):
        p.bind(a, np.zeros(3, np.float32))
    with pytest.raises(VoltaB200Error, match="already compiled"):
        p.add("relu", 99, (a,), (4, 4))
    import torch
    p.bind(a, torch.full((4, 4), 2.0, device="cuda"))       # device-resident input
    p.run()
    assert np.array_equal(p.fetch(out, (4, 4)), np.full((4, 4), -2.0, np.float32))
    p.free()
