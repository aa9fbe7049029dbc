"""fp64 restatement of the training step in torch, the arbiter for shapes the scalar C oracle cannot
finish in seconds.  Test infrastructure only.

Same definitions as the generated step (src/engine/ir/codegen/mlp_train_rust_codegen.rs:699-994): W is
[in x out], the loss is the mean of (out - y)^2 over ALL elements, Adam uses beta 0.9/0.999, eps 1e-8 and
bias corrections 1 - beta^t, AdamW adds lr*0.01*w on weights only (:962-966), Adagrad eps 1e-8, momentum
0.9 (PyTorch form, no dampening).  Forward and backward are written out (no autograd) so that the
activations and deltas are available as the scales gradient errors are measured against.  Pinned against
the C oracle's fp64 build in tests/test_oracle.py::test_torch_fp64_helper_matches_the_oracle."""
from __future__ import annotations

import numpy as np
import torch

def _f32(v):
    """The constant as the reference's f32 source text holds it."""
    return float(np.float32(v))


_C, _K, _SLOPE = _f32(0.7978845608), _f32(0.044715), _f32(0.01)
_B1, _B2, _EPS, _WD, _MU = _f32(0.9), _f32(0.999), _f32(1e-8), _f32(0.01), _f32(0.9)


def _act(name, z):
    if name == "relu":
        return torch.clamp_min(z, 0.0)
    if name == "sigmoid":
        return torch.sigmoid(z)
    if name == "tanh":
        return torch.tanh(z)
    if name == "leaky_relu":
        return torch.where(z > 0, z, _SLOPE * z)
    if name == "silu":
        return z * torch.sigmoid(z)
    if name == "gelu":
        return 0.5 * z * (1.0 + torch.tanh(_C * (z + _K * z ** 3)))
    raise ValueError(name)


def _dact(name, z, a):
    """f'(.) from the pre-activation z and the output a, as the reference takes it (:894-916)."""
    if name == "relu":
        return (z > 0).to(z.dtype)
    if name == "sigmoid":
        return a * (1.0 - a)
    if name == "tanh":
        return 1.0 - a * a
    if name == "leaky_relu":
        return torch.where(z > 0, torch.ones_like(z), torch.full_like(z, _SLOPE))
    if name == "silu":
        s = torch.sigmoid(z)
        return s * (1.0 + z * (1.0 - s))
    if name == "gelu":
        t = torch.tanh(_C * (z + _K * z ** 3))
        return 0.5 * (1.0 + t) + 0.5 * z * (1.0 - t * t) * _C * (1.0 + 3.0 * _K * z * z)
    raise ValueError(name)


class TorchMlp64:
    def __init__(self, layers, activation, optimizer, ws, bs, threads: int | None = None):
        if threads:
            torch.set_num_threads(threads)
        self.layers, self.act, self.opt = list(layers), activation, optimizer
        self.n = len(self.layers) - 1
        self.w = [torch.tensor(np.asarray(w, np.float32), dtype=torch.float64) for w in ws]
        self.b = [torch.tensor(np.asarray(b, np.float32).reshape(-1), dtype=torch.float64) for b in bs]
        z = lambda t: torch.zeros_like(t)
        self.s1w, self.s1b = [z(w) for w in self.w], [z(b) for b in self.b]
        self.s2w, self.s2b = [z(w) for w in self.w], [z(b) for b in self.b]
        self.t = 0
        self.loss_value = float("nan")
        self.dw, self.db, self.acts, self.deltas = [], [], [], []

    def grad_step(self, x, y, global_rows: int | None = None):
        """Forward, loss and backward on rows x; with global_rows the seed gradient is scaled for a shard of a
        larger batch, so that shard gradients add up (data parallelism)."""
        a = torch.tensor(np.asarray(x, np.float32), dtype=torch.float64)
        ty = torch.tensor(np.asarray(y, np.float32), dtype=torch.float64)
        acts, pres = [a], []
        for i in range(self.n):
            zpre = acts[-1] @ self.w[i] + self.b[i]
            pres.append(zpre)
            acts.append(_act(self.act, zpre) if i < self.n - 1 else zpre)
        d = acts[-1] - ty
        nt = float((global_rows or a.shape[0]) * self.layers[-1])
        self.loss_sum = float((d * d).sum())
        self.loss_value = self.loss_sum / nt
        delta = 2.0 * d / nt
        self.dw, self.db, self.deltas = [None] * self.n, [None] * self.n, [None] * self.n
        for i in range(self.n - 1, -1, -1):
            self.deltas[i] = delta
            self.dw[i] = acts[i].T @ delta
            self.db[i] = delta.sum(dim=0)
            if i > 0:
                delta = (delta @ self.w[i].T) * _dact(self.act, pres[i - 1], acts[i])
        self.acts, self.pres = acts, pres

    def update(self, lr: float):
        lr = float(np.float32(lr))   # the step takes lr as an f32 (volta_train_step's signature)
        opt = self.opt
        if opt in ("adam", "adamw"):
            self.t += 1
            bc1, bc2 = 1.0 - _B1 ** self.t, 1.0 - _B2 ** self.t
        for p, g, s1, s2, is_w in ([(self.w[i], self.dw[i], self.s1w[i], self.s2w[i], True) for i in range(self.n)] +
                                   [(self.b[i], self.db[i], self.s1b[i], self.s2b[i], False) for i in range(self.n)]):
            if opt == "sgd":
                p -= lr * g
            elif opt == "sgd_momentum":
                s1.mul_(_MU).add_(g)
                p -= lr * s1
            elif opt == "adagrad":
                s1 += g * g
                p -= lr * g / (torch.sqrt(s1) + _EPS)
            else:
                s1.mul_(_B1).add_((1.0 - _B1) * g)
                s2.mul_(_B2).add_((1.0 - _B2) * g * g)
                wd = _WD if (opt == "adamw" and is_w) else 0.0
                p -= lr * ((s1 / bc1) / (torch.sqrt(s2 / bc2) + _EPS) + wd * p)

    def step(self, x, y, lr: float):
        self.grad_step(x, y)
        self.update(lr)

    def loss(self) -> float:
        return self.loss_value

    # numpy views for comparisons
    def params(self):
        return [w.numpy() for w in self.w] + [b.numpy() for b in self.b]

    def grads(self):
        return [g.numpy() for g in self.dw] + [g.numpy() for g in self.db]

    def state_before_lists(self):
        """(s1 list, s2 list) in the order of params(); copies."""
        return ([t.clone().numpy() for t in self.s1w + self.s1b], [t.clone().numpy() for t in self.s2w + self.s2b], self.t)

    def gradient_scales(self):
        """Per gradient tensor (order of grads()) the size of the terms summed: max |act|^T.|delta| and
        max sum_rows |delta|, amplified where the residual is small against the outputs."""
        sw = [float((self.acts[i].abs().T @ self.deltas[i].abs()).max()) for i in range(self.n)]
        sb = [float(self.deltas[i].abs().sum(dim=0).max()) for i in range(self.n)]
        out_max = float(self.acts[-1].abs().max())
        resid_rms = max(self.loss_value, 1e-300) ** 0.5
        amplify = max(1.0, out_max / resid_rms)
        return [v * amplify for v in sw + sb]

    def fragile_units(self, band: float = 1e-5):
        """Hidden units whose pre-activation lies inside the fp32 noise of its own sum, |pre| <= band * (|act| . |W|
        + |b|): for relu / leaky_relu their derivative (0 or 1) may come out differently in two correct fp32
        evaluations.  Returns, per hidden layer i, the sorted column indices with at least one such row, and the total
        count of (row, column) cases.  Empty for smooth activations."""
        cols, total = [], 0
        if self.act not in ("relu", "leaky_relu"):
            return [np.zeros(0, np.int64) for _ in range(self.n - 1)], 0
        for i in range(self.n - 1):
            bound = self.acts[i].abs() @ self.w[i].abs() + self.b[i].abs()
            frag = self.pres[i].abs() <= band * bound
            total += int(frag.sum())
            cols.append(torch.nonzero(frag.any(dim=0)).reshape(-1).numpy())
        return cols, total
