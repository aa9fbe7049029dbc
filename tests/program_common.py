"""Shared pieces of the runtime-backend tests: the MLP training graph as the runtime builds it and a
numpy (float64) evaluation of a node list, the checker the GPU program is compared with."""
import numpy as np

from volta_b200.program import GraphBuilder


def mlp_training_graph(layers=(16, 32, 4), batch=8, activation="relu"):
    g = GraphBuilder()
    x, y = g.input((batch, layers[0])), g.input((batch, layers[-1]))
    pred, params = g.mlp(list(layers), activation, x)
    loss = g.mse(pred, y)
    grads = g.backward(loss, params)
    return g, x, y, pred, loss, params, grads


def evaluate(g, feed):
    """numpy (float64) evaluation of a GraphBuilder node list: the checker for the GPU program tests."""
    v = {}
    sig = lambda t: 1.0 / (1.0 + np.exp(-t))

    def gelu(t):
        return 0.5 * t * (1.0 + np.tanh(0.7978845608 * (t + 0.044715 * t ** 3)))

    def dgelu(t):
        u = 0.7978845608 * (t + 0.044715 * t ** 3)
        th = np.tanh(u)
        return 0.5 * (1.0 + th) + 0.5 * t * (1.0 - th * th) * 0.7978845608 * (1.0 + 3 * 0.044715 * t * t)

    for kind, vid, ins, shape, attrs in g.nodes:
        a = [v[i] for i in ins]
        if kind in ("input", "parameter"):
            r = np.asarray(feed[vid], np.float64).reshape(shape)
        elif kind == "const":
            r = np.asarray(attrs, np.float64).reshape(shape)
        elif kind == "add": r = a[0] + a[1]
        elif kind == "sub": r = a[0] - a[1]
        elif kind == "mul": r = a[0] * a[1]
        elif kind == "div": r = a[0] / a[1]
        elif kind == "neg": r = -a[0]
        elif kind == "transpose": r = a[0].T
        elif kind == "matmul": r = a[0] @ a[1]
        elif kind == "relu": r = np.where(a[0] > 0, a[0], 0.0)
        elif kind == "relu_backward": r = np.where(a[0] > 0, a[1], 0.0)
        elif kind == "sigmoid": r = sig(a[0])
        elif kind == "sigmoid_backward": r = a[1] * sig(a[0]) * (1 - sig(a[0]))
        elif kind == "gelu": r = gelu(a[0])
        elif kind == "gelu_backward": r = a[1] * dgelu(a[0])
        elif kind == "softmax":
            e = np.exp(a[0] - a[0].max(axis=-1, keepdims=True)); r = e / e.sum(axis=-1, keepdims=True)
        elif kind == "log": r = np.log(a[0])
        elif kind == "exp": r = np.exp(a[0])
        elif kind in ("reduce_sum", "reduce_mean"):
            axis = None if attrs[0] < 0 else int(attrs[0])
            r = (np.sum if kind == "reduce_sum" else np.mean)(a[0], axis=axis, keepdims=bool(attrs[1]))
        elif kind == "softmax_xent":
            m = a[0].max(axis=1, keepdims=True)
            lse = m + np.log(np.exp(a[0] - m).sum(axis=1, keepdims=True))
            r = np.mean(-(a[1] * (a[0] - lse)).sum(axis=1))
        elif kind in ("identity", "output"): r = a[0]
        elif kind == "reshape": r = a[0].reshape(shape)
        else: raise NotImplementedError(kind)
        v[vid] = np.asarray(r, np.float64).reshape(shape)
    return v
