"""Checkpoint files in the reference's formats (src/engine/model/checkpoint.rs), through the C ABI.

`Checkpoint` is a set of named float32 tensors on the host; `save`/`load` write and read the v1 text
and v2 binary files that Volta's save_checkpoint / load_checkpoint(_compressed) use.  The file code
lives in the library (csrc/vb_checkpoint.cpp); this is its thin mirror for tests and tools.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .lib import VoltaB200Error, load_library

TEXT_V1, BINARY_V2 = 1, 2


class Checkpoint:
    def __init__(self, _handle=None):
        self.lib = load_library()
        self.h = C.c_void_p(_handle) if _handle else C.c_void_p(self.lib.volta_b200_checkpoint_new())

    @classmethod
    def load(cls, path: str) -> "Checkpoint":
        """load_checkpoint / load_checkpoint_compressed (checkpoint.rs:46-87, 215-231): either format."""
        lib = load_library()
        h = lib.volta_b200_checkpoint_load(str(path).encode())
        if not h:
            raise VoltaB200Error(1, lib.volta_b200_last_error(None).decode())
        return cls(h)

    def save(self, path: str, format: int = TEXT_V1):
        """save_checkpoint (format 1, checkpoint.rs:14-44) / save_checkpoint_compressed (format 2, :167-213)."""
        rc = self.lib.volta_b200_checkpoint_save(self.h, str(path).encode(), int(format))
        if rc:
            raise VoltaB200Error(rc, self.lib.volta_b200_last_error(None).decode())

    def add(self, name: str, array):
        a = np.ascontiguousarray(array, dtype=np.float32)
        shape = (C.c_int64 * max(a.ndim, 1))(*a.shape)
        rc = self.lib.volta_b200_checkpoint_add(self.h, name.encode(), shape, a.ndim,
                                                a.ctypes.data_as(C.POINTER(C.c_float)))
        if rc:
            raise VoltaB200Error(rc, "checkpoint_add refused %r" % name)

    def tensors(self) -> dict:
        out = {}
        for i in range(int(self.lib.volta_b200_checkpoint_count(self.h))):
            name, shape, ndim = C.c_char_p(), C.POINTER(C.c_int64)(), C.c_int32()
            data, count = C.POINTER(C.c_float)(), C.c_int64()
            self.lib.volta_b200_checkpoint_entry(self.h, i, C.byref(name), C.byref(shape), C.byref(ndim), C.byref(data),
                                                 C.byref(count))
            dims = tuple(int(shape[k]) for k in range(ndim.value))
            vals = np.ctypeslib.as_array(data, shape=(count.value,)).copy() if count.value else np.zeros(0, np.float32)
            out[name.value.decode()] = vals.reshape(dims)
        return out

    def free(self):
        if getattr(self, "h", None):
            self.lib.volta_b200_checkpoint_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
