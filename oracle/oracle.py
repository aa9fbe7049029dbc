"""ctypes face of the CPU oracle (oracle/volta_oracle.c).  Test infrastructure only:
imported by tests/, by the smoke check and by the CPU-baseline leg of the benchmark,
never by the shipped package."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

ACTIVATIONS = {"relu": 0, "sigmoid": 1, "tanh": 2, "leaky_relu": 3, "silu": 4, "gelu": 5, "softmax": 6}
OPTIMIZERS = {"sgd": 0, "adam": 1, "adamw": 2, "adagrad": 3, "sgd_momentum": 4}

_libs: dict = {}


def _lib(real: str):
    if real not in _libs:
        paths = _build.build_oracle()
        lib = C.CDLL(paths[real])
        rp = C.POINTER(C.c_float if real == "f32" else C.c_double)
        lib.oracle_create.restype = C.c_void_p
        lib.oracle_create.argtypes = [C.POINTER(C.c_int), C.c_int, C.c_int, C.c_int, C.c_int]
        lib.oracle_free.argtypes = [C.c_void_p]
        lib.oracle_set_momentum.argtypes = [C.c_void_p, C.c_double]
        lib.oracle_set_decay_bias.argtypes = [C.c_void_p, C.c_int]
        lib.oracle_set_global_batch.argtypes = [C.c_void_p, C.c_longlong]
        lib.oracle_set_shard_row0.argtypes = [C.c_void_p, C.c_longlong]
        lib.oracle_grad_step.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        lib.oracle_update.argtypes = [C.c_void_p, C.c_float]
        lib.oracle_get_state.argtypes = [C.c_void_p] + [C.POINTER(rp)] * 4
        lib.oracle_get_adam_step.restype = C.c_uint64
        lib.oracle_get_adam_step.argtypes = [C.c_void_p]
        lib.oracle_set_adam_step.argtypes = [C.c_void_p, C.c_uint64]
        lib.oracle_set_options.argtypes = [C.c_void_p, C.c_double, C.c_int, C.c_double]
        lib.oracle_get_ln.restype = rp
        lib.oracle_get_ln.argtypes = [C.c_void_p, C.c_int, C.c_int]
        lib.oracle_set_gemm.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        lib.oracle_set_params.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        lib.oracle_get_params.argtypes = [C.c_void_p, C.POINTER(rp), C.POINTER(rp)]
        lib.oracle_get_grads.argtypes = [C.c_void_p, C.POINTER(rp), C.POINTER(rp)]
        lib.oracle_get_act.restype = rp
        lib.oracle_get_act.argtypes = [C.c_void_p, C.c_int]
        lib.oracle_get_delta.restype = rp
        lib.oracle_get_delta.argtypes = [C.c_void_p, C.c_int]
        lib.oracle_loss.restype = C.c_double
        lib.oracle_loss.argtypes = [C.c_void_p]
        lib.oracle_step.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_float]
        lib.oracle_lcg_xavier.argtypes = [C.POINTER(C.c_float), C.c_int64, C.c_int, C.c_int, C.POINTER(C.c_uint64)]
        lib.oracle_keep_scale.restype = C.c_float
        lib.oracle_keep_scale.argtypes = [C.c_float]
        lib.oracle_apply_update.argtypes = [C.c_int, rp, rp, rp, rp, C.c_int64, C.c_double, C.c_double,
                                            C.c_double, C.c_uint64]
        _libs[real] = (lib, rp)
    return _libs[real]


def _fp(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_float))


class Oracle:
    """One training handle of the oracle; mirrors volta_train_init/_step/_loss/_get_params/
    _set_params/_free of the reference's generated library."""

    def __init__(self, layers, activation="relu", optimizer="sgd", batch=1, real="f32", momentum=0.9, dropout_p=0.0,
                 use_layernorm=False, clip_grad=0.0):
        self.layers = [int(x) for x in layers]
        self.n = len(self.layers) - 1
        self.batch = int(batch)
        self.real = real
        self.dtype = np.float32 if real == "f32" else np.float64
        self.lib, self._rp = _lib(real)
        arr = (C.c_int * len(self.layers))(*self.layers)
        self.h = self.lib.oracle_create(arr, len(self.layers), ACTIVATIONS[activation], OPTIMIZERS[optimizer],
                                        self.batch)
        if not self.h:
            raise ValueError("oracle_create rejected the topology")
        self.lib.oracle_set_momentum(self.h, float(np.float32(momentum)))   # an f32 hyper-parameter, in both builds
        if dropout_p or use_layernorm or clip_grad:
            self.lib.oracle_set_options(self.h, float(dropout_p), int(bool(use_layernorm)), float(clip_grad))
        self._shim = None

    def use_reference_gemm(self) -> str | None:
        """Route the GEMMs through the compiled reference gemm_shim.c (fp32 handle only).
        Returns the flavour in use, or None when no prebuilt shim fits this CPU."""
        assert self.real == "f32"
        _build.build_ref()
        pick = _build.pick_ref_shim()
        if pick is None:
            return None
        flavour, path = pick
        self._shim = C.CDLL(path)
        g = C.cast(self._shim.volta_gemm_f32, C.c_void_p)
        t = C.cast(self._shim.volta_transpose_f32, C.c_void_p)
        self.lib.oracle_set_gemm(self.h, g, t)
        return flavour

    def set_decay_bias(self, on: bool):
        """AdamW decay on biases too (runtime-optimizer / PyTorch form); default off as in the generated step."""
        self.lib.oracle_set_decay_bias(self.h, int(bool(on)))

    def set_params(self, li: int, w: np.ndarray, b: np.ndarray):
        w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
        b = np.ascontiguousarray(b, dtype=np.float32).reshape(-1)
        if 0 <= li < self.n:
            assert w.size == self.layers[li] * self.layers[li + 1] and b.size == self.layers[li + 1]
        self.lib.oracle_set_params(self.h, li, _fp(w), _fp(b))

    def _ptr_lists(self, fn):
        wo = (self._rp * self.n)()
        bo = (self._rp * self.n)()
        fn(self.h, wo, bo)
        ws, bs = [], []
        for i in range(self.n):
            r, c = self.layers[i], self.layers[i + 1]
            ws.append(np.ctypeslib.as_array(wo[i], shape=(r, c)).copy())
            bs.append(np.ctypeslib.as_array(bo[i], shape=(c,)).copy())
        return ws, bs

    def get_params(self):
        return self._ptr_lists(self.lib.oracle_get_params)

    def get_grads(self):
        return self._ptr_lists(self.lib.oracle_get_grads)

    def get_act(self, i: int) -> np.ndarray:
        return np.ctypeslib.as_array(self.lib.oracle_get_act(self.h, i), shape=(self.batch, self.layers[i])).copy()

    def get_delta(self, i: int) -> np.ndarray:
        return np.ctypeslib.as_array(self.lib.oracle_get_delta(self.h, i),
                                     shape=(self.batch, self.layers[i + 1])).copy()

    def step(self, x: np.ndarray, y: np.ndarray, lr: float):
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.ascontiguousarray(y, dtype=np.float32)
        assert x.size == self.batch * self.layers[0] and y.size == self.batch * self.layers[-1]
        self.lib.oracle_step(self.h, _fp(x), _fp(y), float(lr))

    def set_shard_row0(self, row0: int):
        """This handle holds rows [row0, row0 + batch) of the global batch (the dropout stream skips the rest)."""
        self.lib.oracle_set_shard_row0(self.h, int(row0))

    def set_global_batch(self, gb: int):
        """This handle holds one shard of a global batch of gb rows (data parallel)."""
        self.lib.oracle_set_global_batch(self.h, int(gb))

    def grad_step(self, x: np.ndarray, y: np.ndarray):
        """Forward + backward + gradients, no update."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.ascontiguousarray(y, dtype=np.float32)
        self.lib.oracle_grad_step(self.h, _fp(x), _fp(y))

    def update(self, lr: float):
        self.lib.oracle_update(self.h, float(lr))

    def grad_views(self):
        """Writable numpy views of the gradients held in the handle (for an external all-reduce)."""
        wo = (self._rp * self.n)()
        bo = (self._rp * self.n)()
        self.lib.oracle_get_grads(self.h, wo, bo)
        ws = [np.ctypeslib.as_array(wo[i], shape=(self.layers[i], self.layers[i + 1])) for i in range(self.n)]
        bs = [np.ctypeslib.as_array(bo[i], shape=(self.layers[i + 1],)) for i in range(self.n)]
        return ws, bs

    def state(self):
        """Copies of the optimizer state: (s1w, s1b, s2w, s2b) lists (None where unused) and the Adam step count."""
        arrs = [(self._rp * self.n)() for _ in range(4)]
        self.lib.oracle_get_state(self.h, *arrs)
        out = []
        for k, a in enumerate(arrs):
            lst = []
            for i in range(self.n):
                shape = (self.layers[i], self.layers[i + 1]) if k % 2 == 0 else (self.layers[i + 1],)
                lst.append(np.ctypeslib.as_array(a[i], shape=shape).copy() if a[i] else None)
            out.append(lst)
        return out[0], out[1], out[2], out[3], int(self.lib.oracle_get_adam_step(self.h))

    def get_layernorm(self, i: int):
        """(gamma, beta) of the LayerNorm behind hidden layer i."""
        c = self.layers[i + 1]
        return tuple(np.ctypeslib.as_array(self.lib.oracle_get_ln(self.h, i, w), shape=(c,)).copy() for w in (0, 1))

    def loss(self) -> float:
        return float(self.lib.oracle_loss(self.h))

    def free(self):
        if self.h:
            self.lib.oracle_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def lcg_xavier(layers) -> list[np.ndarray]:
    """Default-initialised weights of a fresh handle: one LCG stream from seed 42."""
    lib, _ = _lib("f32")
    rng = C.c_uint64(42)
    out = []
    for r, c in zip(layers[:-1], layers[1:]):
        w = np.empty(r * c, dtype=np.float32)
        lib.oracle_lcg_xavier(_fp(w), r * c, r, c, C.byref(rng))
        out.append(w.reshape(r, c))
    return out


def apply_update(optimizer: str, p, g, s1=None, s2=None, lr=0.01, wd=0.01, momentum=0.9, t=1, real="f32"):
    """Bare optimizer update on arrays (in place on copies); returns (p, s1, s2)."""
    lib, rp = _lib(real)
    dt = np.float32 if real == "f32" else np.float64
    p = np.array(p, dtype=dt).reshape(-1).copy()
    g = np.array(g, dtype=dt).reshape(-1).copy()
    s1 = np.zeros_like(p) if s1 is None else np.array(s1, dtype=dt).reshape(-1).copy()
    s2 = np.zeros_like(p) if s2 is None else np.array(s2, dtype=dt).reshape(-1).copy()
    cast = lambda a: a.ctypes.data_as(rp)
    lib.oracle_apply_update(OPTIMIZERS[optimizer], cast(p), cast(s1), cast(s2), cast(g), p.size, float(lr),
                            float(wd), float(momentum), int(t))
    return p, s1, s2


def keep_scale(p: float) -> float:
    """The dropout rescale 1/(1-p) exactly as the generated step holds it (f32 arithmetic)."""
    lib, _ = _lib("f32")
    return float(lib.oracle_keep_scale(float(p)))
