"""Host-side mirror of the runtime-backend slice (include/volta_b200.h, volta_b200_program_*).

`Program` is the thin ctypes wrapper.  `GraphBuilder` builds scheduled graphs the way Volta's
runtime does for an MLP - the forward ops of its lowering (src/engine/ir/lowering.rs:90-153:
MatMul, Add(bias [1, out]), Relu/Sigmoid, MSE as Sub, Mul, ReduceMean) and the backward ops its
autograd emits for them (src/engine/ir/autograd.rs:119-450, 1557-1650, 1947-2040: Transpose +
MatMul, ReluBackward(input, upstream), unbroadcast by ReduceSum + Reshape, ReduceMean backward as
ones * upstream * 1/n) - with shape inference on the host, so that tests and tools can hand the
library exactly the node lists a `B200Backend` would receive.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .lib import CompiledProgram, OptimizerConfig, VoltaB200Error, load_library
from .train import OPTIMIZERS, _ptr

OPS = {"input": 0, "parameter": 1, "const": 2, "add": 3, "sub": 4, "mul": 5, "div": 6, "neg": 7, "transpose": 8,
       "matmul": 9, "relu": 10, "relu_backward": 11, "sigmoid": 12, "sigmoid_backward": 13, "gelu": 14,
       "gelu_backward": 15, "softmax": 16, "log": 17, "exp": 18, "reduce_sum": 19, "reduce_mean": 20, "identity": 21,
       "output": 22, "reshape": 23, "softmax_xent": 24}


class Program:
    def __init__(self):
        self.lib = load_library()
        self.h = C.c_void_p(self.lib.volta_b200_program_new())
        self.info = None

    def _check(self, rc):
        if rc:
            raise VoltaB200Error(rc, self.lib.volta_b200_program_error(self.h).decode())

    def add(self, kind, value_id, inputs=(), shape=(), attrs=()):
        kind = OPS[kind] if isinstance(kind, str) else int(kind)
        ins = (C.c_int32 * max(len(inputs), 1))(*inputs)
        shp = (C.c_int64 * max(len(shape), 1))(*shape)
        at = np.ascontiguousarray(attrs, dtype=np.float32).ravel()
        self._check(self.lib.volta_b200_program_add(self.h, kind, int(value_id), ins, len(inputs), shp, len(shape),
                                                    at.ctypes.data_as(C.POINTER(C.c_float)), at.size))

    def mark_output(self, value_id):
        self._check(self.lib.volta_b200_program_mark_output(self.h, int(value_id)))

    def compile(self, fuse=True):
        """Backend::compile: returns the CompiledProgram record (also kept as .info)."""
        info = CompiledProgram()
        self.info = info        # filled as far as planning got, even when no GPU is present
        self._check(self.lib.volta_b200_program_compile(self.h, 1 if fuse else 0, C.byref(info)))
        return info

    def bind(self, value_id, data):
        if isinstance(data, np.ndarray):
            data = np.ascontiguousarray(data, dtype=np.float32)
        n = int(np.prod(data.shape)) if len(data.shape) else 1
        self._check(self.lib.volta_b200_program_bind(self.h, int(value_id), _ptr(data), n))

    def run(self):
        self._check(self.lib.volta_b200_program_run(self.h))

    def fetch(self, value_id, shape):
        out = np.empty(shape, dtype=np.float32)
        self._check(self.lib.volta_b200_program_fetch(self.h, int(value_id), out.ctypes.data, out.size))
        return out

    def update(self, optimizer, params, grads, lr, step, beta1=0.0, beta2=0.0, eps=0.0, weight_decay=0.0, momentum=0.0):
        """Backend::apply_gradients for the listed (parameter, gradient) value ids."""
        cfg = OptimizerConfig(OPTIMIZERS[optimizer] if isinstance(optimizer, str) else int(optimizer), lr, beta1, beta2,
                              eps, weight_decay, momentum)
        n = len(params)
        pa, ga = (C.c_int32 * max(n, 1))(*params), (C.c_int32 * max(n, 1))(*grads)
        self._check(self.lib.volta_b200_program_update(self.h, C.byref(cfg), pa, ga, n, int(step)))

    def free(self):
        if getattr(self, "h", None):
            self.lib.volta_b200_program_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def _broadcast(a, b):
    n = max(len(a), len(b))
    a2, b2 = (1,) * (n - len(a)) + tuple(a), (1,) * (n - len(b)) + tuple(b)
    out = []
    for x, y in zip(a2, b2):
        if x != y and x != 1 and y != 1:
            raise ValueError("Cannot broadcast %r and %r" % (a, b))
        out.append(max(x, y))
    return tuple(out)


class GraphBuilder:
    """Scheduled node list with host-side shape inference; value ids are handed out in order."""

    def __init__(self):
        self.nodes = []      # (kind, id, inputs, shape, attrs)
        self.shape = {}
        self.kind = {}
        self.inputs = {}
        self.attrs = {}

    def _push(self, kind, inputs, shape, attrs=()):
        vid = len(self.nodes)
        self.nodes.append((kind, vid, tuple(inputs), tuple(int(s) for s in shape), tuple(attrs)))
        self.shape[vid], self.kind[vid], self.inputs[vid], self.attrs[vid] = tuple(shape), kind, tuple(inputs), tuple(attrs)
        return vid

    # sources
    def input(self, shape): return self._push("input", (), shape)
    def parameter(self, shape): return self._push("parameter", (), shape)
    def const(self, array):
        a = np.asarray(array, dtype=np.float32)
        return self._push("const", (), a.shape, a.ravel())

    # elementwise
    def _binary(self, kind, a, b): return self._push(kind, (a, b), _broadcast(self.shape[a], self.shape[b]))
    def add(self, a, b): return self._binary("add", a, b)
    def sub(self, a, b): return self._binary("sub", a, b)
    def mul(self, a, b): return self._binary("mul", a, b)
    def div(self, a, b): return self._binary("div", a, b)
    def _unary(self, kind, a): return self._push(kind, (a,), self.shape[a])
    def neg(self, a): return self._unary("neg", a)
    def relu(self, a): return self._unary("relu", a)
    def sigmoid(self, a): return self._unary("sigmoid", a)
    def gelu(self, a): return self._unary("gelu", a)
    def softmax(self, a): return self._unary("softmax", a)
    def log(self, a): return self._unary("log", a)
    def exp(self, a): return self._unary("exp", a)
    def identity(self, a): return self._unary("identity", a)
    def output(self, a): return self._unary("output", a)
    def relu_backward(self, x, up): return self._push("relu_backward", (x, up), self.shape[x])
    def sigmoid_backward(self, x, up): return self._push("sigmoid_backward", (x, up), self.shape[x])
    def gelu_backward(self, x, up): return self._push("gelu_backward", (x, up), self.shape[x])

    def transpose(self, a):
        r, c = self.shape[a]
        return self._push("transpose", (a,), (c, r))

    def matmul(self, a, b):
        (m, k), (k2, n) = self.shape[a], self.shape[b]
        if k != k2:
            raise ValueError("MatMul shape mismatch")
        return self._push("matmul", (a, b), (m, n))

    def reshape(self, a, shape): return self._push("reshape", (a,), shape)

    def softmax_xent(self, logits, targets):
        """SoftmaxCrossEntropyLossFromLogits (lowering.rs:156-170): scalar mean over the batch."""
        if self.shape[logits] != self.shape[targets] or len(self.shape[logits]) != 2:
            raise ValueError("Shape mismatch in SoftmaxCrossEntropyLossFromLogits")
        return self._push("softmax_xent", (logits, targets), ())

    def _reduce(self, kind, a, axis, keepdims):
        s = self.shape[a]
        if axis is None:
            out = (1,) * len(s) if keepdims else ()
        else:
            out = tuple(1 if i == axis else d for i, d in enumerate(s)) if keepdims else tuple(d for i, d in enumerate(s) if i != axis)
        return self._push(kind, (a,), out, (-1 if axis is None else axis, 1 if keepdims else 0))

    def reduce_sum(self, a, axis=None, keepdims=False): return self._reduce("reduce_sum", a, axis, keepdims)
    def reduce_mean(self, a, axis=None, keepdims=False): return self._reduce("reduce_mean", a, axis, keepdims)

    # ---- the runtime's MLP forward graph and MSE loss (lowering.rs:90-153)
    def mlp(self, layers, activation, x):
        params, cur = [], x
        for i, (r, c) in enumerate(zip(layers[:-1], layers[1:])):
            w, b = self.parameter((r, c)), self.parameter((1, c))
            params += [w, b]
            cur = self.add(self.matmul(cur, w), b)
            if i < len(layers) - 2:
                cur = {"relu": self.relu, "sigmoid": self.sigmoid, "gelu": self.gelu}[activation](cur)
        return cur, params

    def mse(self, pred, target):
        err = self.sub(pred, target)
        return self.reduce_mean(self.mul(err, err))

    # ---- reverse mode with the backward ops of autograd.rs for the ops above
    def _unbroadcast(self, grad, target_shape):
        shape = list(self.shape[grad])
        if tuple(shape) == tuple(target_shape):
            return grad
        while len(shape) > len(target_shape):
            grad = self.reduce_sum(grad, 0, False)
            shape.pop(0)
            if not shape:
                shape.append(1)
        for axis in reversed([i for i, (c, t) in enumerate(zip(shape, target_shape)) if t == 1 and c != 1]):
            grad = self.reduce_sum(grad, axis, False)
            shape.pop(axis)
            if not shape:
                shape.append(1)
        if tuple(shape) != tuple(target_shape):
            grad = self.reshape(grad, target_shape)
        return grad

    def backward(self, loss, wrt):
        """Gradient value ids of `loss` (a scalar) with respect to the values in `wrt`."""
        seed = self.const(np.ones(self.shape[loss] or (), np.float32))     # "__loss_grad" = 1
        grads = {loss: seed}

        def acc(v, g):
            grads[v] = g if v not in grads else self.add(grads[v], g)

        for kind, vid, ins, shape, attrs in reversed(list(self.nodes[:loss + 1])):
            if vid not in grads:
                continue
            up = grads[vid]
            if kind == "add":
                acc(ins[0], self._unbroadcast(up, self.shape[ins[0]]))
                acc(ins[1], self._unbroadcast(up, self.shape[ins[1]]))
            elif kind == "sub":
                acc(ins[0], self._unbroadcast(up, self.shape[ins[0]]))
                acc(ins[1], self._unbroadcast(self.neg(up), self.shape[ins[1]]))
            elif kind == "mul":
                acc(ins[0], self._unbroadcast(self.mul(up, ins[1]), self.shape[ins[0]]))
                acc(ins[1], self._unbroadcast(self.mul(up, ins[0]), self.shape[ins[1]]))
            elif kind == "neg":
                acc(ins[0], self.neg(up))
            elif kind == "matmul":
                acc(ins[0], self.matmul(up, self.transpose(ins[1])))
                acc(ins[1], self.matmul(self.transpose(ins[0]), up))
            elif kind == "relu":
                acc(ins[0], self.relu_backward(ins[0], up))
            elif kind == "sigmoid":
                acc(ins[0], self.sigmoid_backward(ins[0], up))
            elif kind == "gelu":
                acc(ins[0], self.gelu_backward(ins[0], up))
            elif kind == "transpose":
                acc(ins[0], self.transpose(up))
            elif kind in ("reshape", "identity", "output"):
                acc(ins[0], up if kind != "reshape" else self.reshape(up, self.shape[ins[0]]))
            elif kind == "softmax_xent":
                # autograd.rs:467-530: (softmax(logits) - targets) / batch, times the upstream scalar; no
                # gradient flows to the targets
                diff = self.sub(self.softmax(ins[0]), ins[1])
                bs = self.const(np.float32(self.shape[ins[0]][0]))
                acc(ins[0], self.mul(self.div(diff, bs), up))
            elif kind == "reduce_mean" and attrs[0] < 0:
                n = int(np.prod(self.shape[ins[0]]))
                ones = self.const(np.ones(self.shape[ins[0]], np.float32))
                acc(ins[0], self.mul(self.mul(ones, up), self.const(np.array([1.0 / n], np.float32))))
            elif kind == "reduce_sum" and attrs[0] < 0:
                acc(ins[0], self.mul(self.const(np.ones(self.shape[ins[0]], np.float32)), up))
            elif kind in ("input", "parameter", "const"):
                pass
            else:
                raise NotImplementedError("backward of %s" % kind)
        return [grads[v] for v in wrt]

    def emit(self, program: Program, outputs=()):
        for kind, vid, ins, shape, attrs in self.nodes:
            program.add(kind, vid, ins, shape, attrs)
        for v in outputs:
            program.mark_output(v)
        return program
