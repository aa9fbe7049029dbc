"""Host-side mirror of the reference's training-library interface.

The reference's generated library exports, per model, volta_train_init / _step / _loss /
_get_params / _set_params / _free (src/engine/ir/codegen/mlp_train_rust_codegen.rs:641-699).
TrainHandle exposes the same six operations, with the same argument meaning and the same
lenient error behaviour (an out-of-range layer in set_params is ignored), on top of the
C ABI of libvolta_b200.  The topology that the reference compiles in (MlpTopology,
:28-39) is passed to the constructor.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .lib import Config, KernelRecord, VoltaB200Error, load_library

ACTIVATIONS = {"relu": 0, "sigmoid": 1, "tanh": 2, "leaky_relu": 3, "leakyrelu": 3, "silu": 4, "gelu": 5, "softmax": 6,
               "": 0}
OPTIMIZERS = {"sgd": 0, "adam": 1, "adamw": 2, "adagrad": 3, "sgd_momentum": 4}
GEMM_PATHS = {"auto": 0, "ffma": 1, "tensor": 2, "tensor_pair": 3}
DP_EXCHANGE = {"nccl": 0, "peer_kernel": 1, "peer_copy": 2}


def _ptr(a):
    """Raw address of a numpy array (host) or of anything exposing data_ptr() (a torch tensor)."""
    if a is None:
        return None
    if isinstance(a, int):
        return a
    if isinstance(a, np.ndarray):
        if a.dtype != np.float32 or not a.flags["C_CONTIGUOUS"]:
            raise TypeError("expected a C-contiguous float32 array")
        return a.ctypes.data
    if hasattr(a, "data_ptr"):
        if str(a.dtype) != "torch.float32" or not a.is_contiguous():
            raise TypeError("expected a contiguous float32 tensor")
        return a.data_ptr()
    raise TypeError("unsupported buffer type %r" % type(a))


def dp_unique_id() -> bytes:
    """128-byte id for a data-parallel group; create on rank 0, hand to every rank."""
    lib = load_library()
    buf = (C.c_uint8 * 128)()
    rc = lib.volta_b200_dp_unique_id(C.byref(buf))
    if rc:
        raise VoltaB200Error(rc, "could not obtain an NCCL unique id")
    return bytes(buf)


class TrainHandle:
    """volta_train_init(batch) for a given topology; methods mirror the other five entry points."""

    def __init__(self, layers, activation="relu", optimizer="sgd", batch=1, *, global_batch=0, world_size=1, rank=0,
                 unique_id: bytes | None = None, momentum=0.0, weight_decay=0.0, gemm_path="auto", use_graph=True,
                 force_dp=False, fuse_sgd=False, dropout_p=0.0, use_layernorm=False, clip_grad=0.0, device_wait_ms=0,
                 check_finite=False, step_kernel=0, dp_exchange="nccl"):
        act = activation.lower()
        opt = optimizer.lower()
        if act not in ACTIVATIONS:
            raise VoltaB200Error(6, "unsupported activation %r" % activation)
        if opt not in OPTIMIZERS:
            # the reference rejects optimizers outside its list before generating code
            # (src/engine/executor.rs:3147-3189)
            raise VoltaB200Error(6, "unsupported optimizer %r" % optimizer)
        self.lib = load_library()
        self.layers = [int(x) for x in layers]
        self.n = len(self.layers) - 1
        self.batch = int(batch)
        cfg = Config()
        cfg.n_sizes = len(self.layers)
        for i, v in enumerate(self.layers[:32]):
            cfg.layers[i] = v
        cfg.activation = ACTIVATIONS[act]
        cfg.optimizer = OPTIMIZERS[opt]
        cfg.batch = self.batch
        cfg.global_batch = int(global_batch)
        cfg.world_size = int(world_size)
        cfg.rank = int(rank)
        if world_size > 1 or force_dp:
            cfg.force_dp = 1 if force_dp else 0
            if unique_id is None or len(unique_id) != 128:
                raise VoltaB200Error(1, "world_size > 1 needs the 128-byte unique id")
            for i, b in enumerate(unique_id):
                cfg.nccl_unique_id[i] = b
        cfg.momentum = float(momentum)
        cfg.weight_decay = float(weight_decay)
        cfg.gemm_path = GEMM_PATHS[gemm_path]
        cfg.use_graph = 1 if use_graph else 2
        cfg.fuse_sgd = 1 if fuse_sgd else 0
        # MlpTopology's dropout_p / use_layernorm / clip_grad (mlp_train_rust_codegen.rs:34-38)
        cfg.dropout_p = float(dropout_p)
        cfg.use_layernorm = 1 if use_layernorm else 0
        cfg.clip_grad = float(clip_grad)
        cfg.device_wait_ms = int(device_wait_ms)
        cfg.check_finite = 1 if check_finite else 0
        cfg.step_kernel = int(step_kernel)   # 0 auto, 1 per-kernel schedule, 2 require the persistent step kernel
        # what attach_peers switches the exchange to: "nccl"/"peer_kernel" (the fused kernel) or "peer_copy"
        cfg.dp_exchange = DP_EXCHANGE[dp_exchange]
        self.dropout_p = float(dropout_p)
        self._cfg = cfg
        h = C.c_void_p()
        rc = self.lib.volta_b200_create(C.byref(cfg), C.byref(h))
        if rc:
            raise VoltaB200Error(rc, self.lib.volta_b200_last_error(None).decode())
        self.h = h

    # -- the reference's six operations ---------------------------------------------------
    def step(self, x, y, lr: float):
        """volta_train_step(h, X, Y, lr). x/y: float32 numpy arrays (host) or CUDA tensors."""
        rc = self.lib.volta_b200_step(self.h, _ptr(x), _ptr(y), float(lr))
        self._check(rc)

    def loss(self) -> float:
        """volta_train_loss(h)."""
        v = float(self.lib.volta_b200_loss(self.h))
        self._check(self.lib.volta_b200_status(self.h))
        return v

    def set_params(self, li: int, w, b):
        """volta_train_set_params(h, li, w, b); li out of range is ignored.  w and b: numpy arrays, or CUDA
        tensors (copied device to device)."""
        if hasattr(w, "data_ptr") and hasattr(b, "data_ptr"):
            if 0 <= li < self.n and (w.numel() != self.layers[li] * self.layers[li + 1] or b.numel() != self.layers[li + 1]):
                raise ValueError("set_params: wrong tensor size for layer %d" % li)
            fp = C.POINTER(C.c_float)
            self._check(self.lib.volta_b200_set_params(self.h, int(li), C.cast(_ptr(w), fp), C.cast(_ptr(b), fp)))
            return
        w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
        b = np.ascontiguousarray(b, dtype=np.float32).reshape(-1)
        if 0 <= li < self.n:
            if w.size != self.layers[li] * self.layers[li + 1] or b.size != self.layers[li + 1]:
                raise ValueError("set_params: wrong tensor size for layer %d" % li)
        fp = C.POINTER(C.c_float)
        self._check(self.lib.volta_b200_set_params(self.h, int(li), w.ctypes.data_as(fp), b.ctypes.data_as(fp)))

    def _lists(self, fn):
        fp = C.POINTER(C.c_float)
        wo, bo = (fp * self.n)(), (fp * self.n)()
        self._check(fn(self.h, wo, bo))
        ws, bs = [], []
        for i in range(self.n):
            r, c = self.layers[i], self.layers[i + 1]
            ws.append(np.ctypeslib.as_array(wo[i], shape=(r, c)).copy())
            bs.append(np.ctypeslib.as_array(bo[i], shape=(c,)).copy())
        return ws, bs

    def get_params(self):
        """volta_train_get_params(h, wo, bo): copies of every layer's W [in x out] and b."""
        return self._lists(self.lib.volta_b200_get_params)

    def free(self):
        """volta_train_free(h)."""
        if getattr(self, "h", None):
            self.lib.volta_b200_destroy(self.h)
            self.h = None

    def infer(self, x):
        """Forward pass with the current weights (the reference's volta_infer, for up to `batch` rows).
        x: [rows x L0] float32 numpy array or CUDA tensor; returns a numpy array [rows x Ln]."""
        n_in = int(np.prod(x.shape))
        rows = n_in // self.layers[0]
        out = np.empty((rows, self.layers[-1]), dtype=np.float32)
        self._check(self.lib.volta_b200_infer(self.h, _ptr(x), n_in, out.ctypes.data, out.size))
        return out

    # -- extensions -------------------------------------------------------------------------
    def get_layernorm(self, li: int):
        """(gamma, beta) of hidden layer li; the handle must have been created with use_layernorm."""
        c = self.layers[li + 1] if 0 <= li < self.n - 1 else 1
        g, b = np.empty(c, np.float32), np.empty(c, np.float32)
        fp = C.POINTER(C.c_float)
        self._check(self.lib.volta_b200_get_layernorm(self.h, int(li), g.ctypes.data_as(fp), b.ctypes.data_as(fp)))
        return g, b

    def set_layernorm(self, li: int, gamma, beta):
        g = np.ascontiguousarray(gamma, dtype=np.float32).reshape(-1)
        b = np.ascontiguousarray(beta, dtype=np.float32).reshape(-1)
        if 0 <= li < self.n - 1 and (g.size != self.layers[li + 1] or b.size != self.layers[li + 1]):
            raise ValueError("set_layernorm: wrong tensor size for layer %d" % li)
        fp = C.POINTER(C.c_float)
        self._check(self.lib.volta_b200_set_layernorm(self.h, int(li), g.ctypes.data_as(fp), b.ctypes.data_as(fp)))

    def get_grads(self):
        return self._lists(self.lib.volta_b200_get_grads)

    def save_state(self):
        n = int(self.lib.volta_b200_state_floats(self.h))
        buf = np.zeros(max(n, 1), dtype=np.float32)
        step = C.c_uint64(0)
        self._check(self.lib.volta_b200_save_state(self.h, buf.ctypes.data_as(C.POINTER(C.c_float)), n, C.byref(step)))
        return buf[:n], int(step.value)

    def load_state(self, buf: np.ndarray, step: int):
        buf = np.ascontiguousarray(buf, dtype=np.float32)
        self._check(self.lib.volta_b200_load_state(self.h, buf.ctypes.data_as(C.POINTER(C.c_float)), buf.size, int(step)))

    def state_offsets(self):
        """Float offsets of every W_i and b_i inside one flat state/parameter region: all
        weights first, then all biases, each tensor padded to a multiple of 64 floats."""
        pad = lambda v: (v + 63) // 64 * 64
        off, ow, ob = 0, [], []
        for r, c in zip(self.layers[:-1], self.layers[1:]):
            ow.append(off)
            off += pad(r * c)
        for c in self.layers[1:]:
            ob.append(off)
            off += pad(c)
        return ow, ob, off

    def load_state_tensors(self, s1w, s1b, s2w, s2b, step: int):
        """Import per-layer optimizer state (lists of arrays; None where unused) and the step count."""
        ow, ob, total = self.state_offsets()
        n = int(self.lib.volta_b200_state_floats(self.h))
        moments = n - (2 if self.dropout_p > 0.0 else 0)   # the mask stream position rides behind the moments
        buf = np.zeros(max(n, 1), dtype=np.float32)
        if moments < n:
            buf[moments:n] = self.save_state()[0][moments:n]
        for base, (ws, bs) in ((0, (s1w, s1b)), (total, (s2w, s2b))):
            if base >= moments:
                break
            for i in range(self.n):
                if ws[i] is not None:
                    buf[base + ow[i]: base + ow[i] + ws[i].size] = np.asarray(ws[i], np.float32).ravel()
                if bs[i] is not None:
                    buf[base + ob[i]: base + ob[i] + bs[i].size] = np.asarray(bs[i], np.float32).ravel()
        self.load_state(buf[:n], step)

    def _names(self, layer_names):
        if layer_names is None:
            return None, 0
        arr = (C.c_char_p * len(layer_names))(*[None if v is None else str(v).encode() for v in layer_names])
        return arr, len(layer_names)

    def export_checkpoint(self, with_state: bool = True, layer_names=None):
        """Parameters (and, with_state, optimizer moments and counters) as a named-tensor Checkpoint.
        layer_names: one name per weight layer (Volta names tensors "{layer name}.weight"); default "layer<i>"."""
        from .checkpoint import Checkpoint
        ck = Checkpoint()
        arr, n = self._names(layer_names)
        self._check(self.lib.volta_b200_export_checkpoint_named(self.h, ck.h, 1 if with_state else 0, arr, n))
        return ck

    def import_checkpoint(self, ck, layer_names=None):
        """Take every tensor the checkpoint names for this topology; other names are ignored.  Without
        layer_names: "layer<i>.*", else the checkpoint's "<X>.weight"/"<X>.bias" pairs in sorted order.
        A checkpoint in which no parameter tensor is found raises."""
        arr, n = self._names(layer_names)
        self._check(self.lib.volta_b200_import_checkpoint_named(self.h, ck.h, arr, n))

    def dp_wait_selftest(self, declared_world: int = 2, wait_ms: int = 50):
        """One barrier kernel whose peers never answer: raises VoltaB200Error (device wait) after wait_ms."""
        self._check(self.lib.volta_b200_dp_wait_selftest(self.h, int(declared_world), int(wait_ms)))

    def ipc_handle(self) -> bytes:
        """64-byte handle of this rank's arena, to be exchanged among the data-parallel ranks."""
        buf = (C.c_uint8 * 64)()
        self._check(self.lib.volta_b200_dp_ipc_handle(self.h, C.byref(buf)))
        return bytes(buf)

    def attach_peers(self, handles):
        """Switch to the fused peer-memory gradient exchange; `handles` lists every rank's ipc_handle() by rank."""
        blob = b"".join(handles)
        self._check(self.lib.volta_b200_dp_attach_peers(self.h, blob, len(handles)))

    def synchronize(self):
        self._check(self.lib.volta_b200_synchronize(self.h))

    @property
    def stream(self) -> int:
        return int(self.lib.volta_b200_stream(self.h) or 0)

    @property
    def arena_bytes(self) -> int:
        return int(self.lib.volta_b200_arena_bytes(self.h))

    @property
    def kernels_per_step(self) -> int:
        return int(self.lib.volta_b200_kernels_per_step(self.h))

    def profile_step(self, x, y, lr: float):
        """One step as plain launches, timed per kernel. Returns [(name, ms, flops, bytes)]."""
        recs = (KernelRecord * 256)()
        n = self.lib.volta_b200_profile_step(self.h, _ptr(x), _ptr(y), float(lr), recs, 256)
        if n < 0:
            self._check(-n)
        return [(recs[i].name.decode(), float(recs[i].ms), float(recs[i].flops), float(recs[i].bytes))
                for i in range(n)]

    def _check(self, rc: int):
        if rc:
            raise VoltaB200Error(rc, self.lib.volta_b200_last_error(self.h).decode())

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.free()
