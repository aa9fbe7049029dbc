"""Runtime-backend slice, host half: node validation with the reference's shape rules, the fused
lowering (how many kernels a schedule becomes) and the memory plan - none of which needs a GPU -
and the loud failure when the device half is asked for without one."""
import numpy as np
import pytest
import torch

from volta_b200 import VoltaB200Error
from tests.program_common import evaluate, mlp_training_graph
from volta_b200.program import GraphBuilder, Program


def plan(g, outputs, fuse):
    p = g.emit(Program(), outputs)
    try:
        p.compile(fuse)
    except VoltaB200Error as e:          # no GPU here: planning has run, the device half refused
        assert e.code == 2 and "no CPU fallback" in str(e)
    return p.info


def test_lowering_folds_transposes_and_epilogues():
    g, x, y, pred, loss, params, grads = mlp_training_graph()
    fused, plain = plan(g, [loss] + grads, True), plan(g, [loss] + grads, False)
    assert fused.schedule_len == plain.schedule_len == len(g.nodes)
    kinds = [n[0] for n in g.nodes]
    sources = sum(k in ("input", "parameter", "const") for k in kinds)
    aliases = sum(k in ("reshape", "identity", "output") for k in kinds)
    assert plain.launches == len(g.nodes) - sources - aliases          # one kernel per computing node
    # fused: 4 transposes become operand layouts (autograd also differentiates towards the input x),
    # 2 bias adds + 1 relu ride forward epilogues, 1 relu_backward rides the dX GEMM
    assert fused.launches == plain.launches - 4 - 3 - 1
    assert fused.peak_bytes <= fused.unshared_bytes and fused.unshared_bytes < plain.unshared_bytes
    assert fused.fingerprint == plain.fingerprint != 0


def test_fingerprint_tells_schedules_apart():
    a = plan(mlp_training_graph()[0], [], True).fingerprint
    b = plan(mlp_training_graph(layers=(16, 33, 4))[0], [], True).fingerprint
    c = plan(mlp_training_graph()[0], [], True).fingerprint
    assert a == c and a != b


@pytest.mark.parametrize("build,message", [
    (lambda p: p.add("add", 0, (5,), (2, 2)), "before its definition"),
    (lambda p: (p.add("input", 0, (), (2, 3)), p.add("input", 0, (), (2, 3))), "already defined"),
    (lambda p: (p.add("input", 0, (), (2, 3)), p.add("input", 1, (), (4, 3)), p.add("add", 2, (0, 1), (4, 3))), "Cannot broadcast"),
    (lambda p: (p.add("input", 0, (), (2, 3)), p.add("input", 1, (), (4, 5)), p.add("matmul", 2, (0, 1), (2, 5))), "MatMul shape mismatch"),
    (lambda p: (p.add("input", 0, (), (2, 3)), p.add("transpose", 1, (0,), (2, 3))), "Transpose expects"),
    (lambda p: (p.add("input", 0, (), (2, 3)), p.add("relu", 1, (0,), (3, 2))), "Shape mismatch"),
    (lambda p: (p.add("input", 0, (), (2, 3)), p.add("input", 1, (), (2, 2)), p.add("relu_backward", 2, (0, 1), (2, 3))), "Shape mismatch"),
    (lambda p: (p.add("input", 0, (), (2, 3)), p.add("reduce_sum", 1, (0,), (2,), (2, 0))), "axis out of range"),
    (lambda p: (p.add("input", 0, (), (2, 3)), p.add("reduce_sum", 1, (0,), (2,), (0, 0))), "output shape mismatch"),
    (lambda p: (p.add("input", 0, (), (2, 3)), p.add("reshape", 1, (0,), (4, 2))), "changes the element count"),
    (lambda p: p.add("input", 0, (), (2, 3, 4)), "rank above 2"),
    (lambda p: (p.add("input", 0, (), (2, 3)), p.add("input", 1, (), (2, 4)), p.add("softmax_xent", 2, (0, 1), ())), "SoftmaxCrossEntropyLossFromLogits"),
    (lambda p: p.add("const", 0, (), (2, 2), (1.0, 2.0)), "does not match its shape"),
    (lambda p: p.add(99, 0, (), (2, 2)), "unsupported op kind"),
    (lambda p: p.mark_output(3), "unknown value"),
])
def test_malformed_nodes_are_refused(build, message):
    p = Program()
    with pytest.raises(VoltaB200Error, match=message):
        build(p)


def test_a_refused_node_leaves_the_program_usable():
    p = Program()
    p.add("input", 0, (), (2, 3))
    with pytest.raises(VoltaB200Error):
        p.add("relu", 1, (0,), (9, 9))
    p.add("relu", 1, (0,), (2, 3))       # the same id is still free
    with pytest.raises(VoltaB200Error, match="compile the program first"):
        p.run()


def test_builder_backward_matches_torch_on_the_host():
    """The node lists handed to the library are right: evaluate them with numpy and compare the gradients
    with torch autograd (the builder restates lowering.rs + autograd.rs; this pins the restatement)."""
    g, x, y, pred, loss, params, grads = mlp_training_graph(layers=(5, 7, 3), batch=4, activation="sigmoid")
    rs = np.random.RandomState(0)
    feed = {x: rs.randn(4, 5), y: rs.randn(4, 3)}
    for p_ in params:
        feed[p_] = rs.randn(*g.shape[p_]) * 0.5
    val = evaluate(g, feed)
    tw = {k: torch.tensor(v, dtype=torch.float64, requires_grad=k in params) for k, v in feed.items()}
    h = tw[x]
    for i in range(2):
        h = h @ tw[params[2 * i]] + tw[params[2 * i + 1]]
        if i == 0:
            h = torch.sigmoid(h)
    l = torch.mean((h - tw[y]) ** 2)
    l.backward()
    assert abs(float(l.detach()) - float(val[loss])) < 1e-12
    for p_, gr in zip(params, grads):
        assert g.shape[gr] == g.shape[p_]
        # 1/n of the ReduceMean backward is an f32 ConstTensor, as in the reference (autograd.rs:1633-1640)
        np.testing.assert_allclose(val[gr], tw[p_].grad.numpy(), rtol=1e-6, atol=1e-9)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_compile_fails_loudly_without_a_gpu():
    g = mlp_training_graph()[0]
    p = g.emit(Program())
    with pytest.raises(VoltaB200Error, match="no CPU fallback"):
        p.compile()
    with pytest.raises(VoltaB200Error, match="compile the program first"):
        p.run()


def launches(build, outputs, fuse=True):
    g = GraphBuilder()
    outs = build(g)
    return plan(g, [outs[i] for i in outputs] if outputs else [], fuse).launches


def test_lowering_corner_cases():
    """What folds and what does not, read off the number of kernels a schedule becomes."""
    def both_transposed(g):
        a, b = g.input((8, 4)), g.input((6, 8))
        return [g.matmul(g.transpose(a), g.transpose(b))]
    assert launches(both_transposed, [0]) == 2            # only the right operand folds; the left transpose runs
    assert launches(both_transposed, [0], fuse=False) == 3

    def add_full_matrix(g):
        a, w, c = g.input((8, 4)), g.parameter((4, 6)), g.input((8, 6))
        return [g.add(g.matmul(a, w), c)]
    assert launches(add_full_matrix, [0]) == 2            # not a row bias: stays an elementwise add

    def kept_matmul(g):
        a, w, b = g.input((8, 4)), g.parameter((4, 6)), g.parameter((1, 6))
        mm = g.matmul(a, w)
        return [mm, g.add(mm, b)]
    assert launches(kept_matmul, [1]) == 1                # bias rides the GEMM
    assert launches(kept_matmul, [0, 1]) == 2             # ... unless the raw product itself must stay readable

    def bias_relu_with_pre_reader(g):
        a, w, b, up = g.input((8, 4)), g.parameter((4, 6)), g.parameter((1, 6)), g.input((8, 6))
        pre = g.add(g.matmul(a, w), b)
        return [g.relu(pre), g.relu_backward(pre, up)]
    assert launches(bias_relu_with_pre_reader, [0, 1]) == 2   # one GEMM writing act and pre, one backward kernel

    def backward_of_a_product(g):
        x, up, w = g.input((8, 6)), g.input((8, 5)), g.parameter((6, 5))
        return [g.relu_backward(x, g.matmul(up, g.transpose(w))), g.sigmoid_backward(x, g.matmul(up, g.transpose(w)))]
    # relu backward rides its GEMM (transpose folded too); sigmoid backward needs sigmoid(x) and stays a kernel
    assert launches(backward_of_a_product, [0, 1]) == 3

    def bias_defined_late(g):
        a, w = g.input((8, 4)), g.parameter((4, 6))
        mm = g.matmul(a, w)
        b = g.parameter((1, 6))                           # defined after the product: the fused launch could not read it yet
        return [g.add(mm, b)]
    assert launches(bias_defined_late, [0]) == 2

    def aliases_cost_nothing(g):
        a = g.input((4, 6))
        return [g.output(g.reshape(g.identity(g.neg(a)), (6, 4)))]
    assert launches(aliases_cost_nothing, [0]) == 1
