"""Loads libvolta_b200.so and declares its C ABI (include/volta_b200.h) for ctypes."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
VB200_MAX_LAYERS = 32


class VoltaB200Error(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__("libvolta_b200 error %d: %s" % (code, message))
        self.code = code


class Config(C.Structure):
    _fields_ = [
        ("n_sizes", C.c_int32), ("layers", C.c_int32 * VB200_MAX_LAYERS), ("activation", C.c_int32),
        ("optimizer", C.c_int32), ("batch", C.c_int32), ("global_batch", C.c_int32), ("world_size", C.c_int32),
        ("rank", C.c_int32), ("nccl_unique_id", C.c_uint8 * 128), ("momentum", C.c_float),
        ("weight_decay", C.c_float), ("gemm_path", C.c_int32), ("use_graph", C.c_int32),
        ("force_dp", C.c_int32), ("fuse_sgd", C.c_int32), ("use_layernorm", C.c_int32), ("dropout_p", C.c_float),
        ("clip_grad", C.c_float), ("device_wait_ms", C.c_int32), ("check_finite", C.c_int32),
        ("step_kernel", C.c_int32), ("dp_exchange", C.c_int32),
    ]


class CompiledProgram(C.Structure):
    _fields_ = [("schedule_len", C.c_int64), ("launches", C.c_int64), ("peak_bytes", C.c_int64),
                ("unshared_bytes", C.c_int64), ("fingerprint", C.c_uint64)]


class OptimizerConfig(C.Structure):
    _fields_ = [("optimizer", C.c_int32), ("lr", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float),
                ("eps", C.c_float), ("weight_decay", C.c_float), ("momentum", C.c_float)]


class KernelRecord(C.Structure):
    _fields_ = [("name", C.c_char * 48), ("ms", C.c_float), ("flops", C.c_double), ("bytes", C.c_double)]


# every symbol include/volta_b200.h declares
EXPORTS = [
    "volta_b200_create", "volta_b200_destroy", "volta_b200_step", "volta_b200_loss", "volta_b200_set_params",
    "volta_b200_get_params", "volta_b200_infer", "volta_b200_get_layernorm", "volta_b200_set_layernorm", "volta_b200_get_grads", "volta_b200_state_floats", "volta_b200_save_state",
    "volta_b200_load_state", "volta_b200_status", "volta_b200_last_error", "volta_b200_stream",
    "volta_b200_synchronize", "volta_b200_arena_bytes", "volta_b200_plan", "volta_b200_kernels_per_step",
    "volta_b200_profile_step", "volta_b200_dp_unique_id", "volta_b200_dp_ipc_handle", "volta_b200_dp_attach_peers", "volta_b200_optimizer_apply", "volta_b200_gemm",
    "volta_b200_colsum_scratch_floats", "volta_b200_colsum", "volta_b200_colsum_noalloc", "volta_b200_version",
    "volta_b200_checkpoint_new", "volta_b200_checkpoint_free", "volta_b200_checkpoint_add", "volta_b200_checkpoint_save",
    "volta_b200_checkpoint_load", "volta_b200_checkpoint_parse", "volta_b200_checkpoint_count", "volta_b200_checkpoint_entry",
    "volta_b200_export_checkpoint", "volta_b200_import_checkpoint", "volta_b200_export_checkpoint_named",
    "volta_b200_import_checkpoint_named", "volta_b200_checkpoint_match", "volta_b200_dp_wait_selftest", "volta_b200_dp_check",
    "volta_b200_gemm_route", "volta_b200_update_selftest", "volta_b200_config_size",
    "volta_b200_program_new", "volta_b200_program_free", "volta_b200_program_error", "volta_b200_program_add",
    "volta_b200_program_mark_output", "volta_b200_program_compile", "volta_b200_program_bind", "volta_b200_program_run",
    "volta_b200_program_fetch", "volta_b200_program_update",
]

_lib = None


def library_path() -> str:
    return os.environ.get("VOLTA_B200_LIB", os.path.join(HERE, "libvolta_b200.so"))


def load_library():
    """Load the compiled library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise VoltaB200Error(-1, "%s is missing: build it with `python -m volta_b200.build` "
                                 "(there is no CPU or PyTorch fallback)" % path)
    lib = C.CDLL(path)
    fp, vp, i32, i64 = C.POINTER(C.c_float), C.c_void_p, C.c_int32, C.c_int64
    fpp = C.POINTER(fp)
    sig = {
        "volta_b200_create": (C.c_int, [C.POINTER(Config), C.POINTER(vp)]),
        "volta_b200_destroy": (None, [vp]),
        "volta_b200_step": (C.c_int, [vp, vp, vp, C.c_float]),
        "volta_b200_loss": (C.c_float, [vp]),
        "volta_b200_set_params": (C.c_int, [vp, i32, fp, fp]),
        "volta_b200_get_params": (C.c_int, [vp, fpp, fpp]),
        "volta_b200_infer": (C.c_int, [vp, vp, i64, vp, i64]),
        "volta_b200_get_layernorm": (C.c_int, [vp, i32, fp, fp]),
        "volta_b200_set_layernorm": (C.c_int, [vp, i32, fp, fp]),
        "volta_b200_get_grads": (C.c_int, [vp, fpp, fpp]),
        "volta_b200_state_floats": (i64, [vp]),
        "volta_b200_save_state": (C.c_int, [vp, fp, i64, C.POINTER(C.c_uint64)]),
        "volta_b200_load_state": (C.c_int, [vp, fp, i64, C.c_uint64]),
        "volta_b200_status": (C.c_int, [vp]),
        "volta_b200_last_error": (C.c_char_p, [vp]),
        "volta_b200_stream": (vp, [vp]),
        "volta_b200_synchronize": (C.c_int, [vp]),
        "volta_b200_arena_bytes": (i64, [vp]),
        "volta_b200_kernels_per_step": (i32, [vp]),
        "volta_b200_plan": (C.c_int, [C.POINTER(Config), C.POINTER(i64), C.POINTER(i64), C.c_char_p, i64]),
        "volta_b200_profile_step": (C.c_int, [vp, vp, vp, C.c_float, C.POINTER(KernelRecord), i32]),
        "volta_b200_dp_unique_id": (C.c_int, [C.POINTER(C.c_uint8 * 128)]),
        "volta_b200_dp_ipc_handle": (C.c_int, [vp, C.POINTER(C.c_uint8 * 64)]),
        "volta_b200_dp_attach_peers": (C.c_int, [vp, C.c_char_p, i32]),
        "volta_b200_optimizer_apply": (C.c_int, [i32, vp, vp, vp, vp, i64, i64, C.c_float, C.c_float, C.c_float,
                                                 C.c_uint64, vp]),
        "volta_b200_gemm": (C.c_int, [i32, i32, vp, vp, vp, i64, i64, i64, vp]),
        "volta_b200_colsum_scratch_floats": (i64, [i64, i64]),
        "volta_b200_colsum": (C.c_int, [vp, vp, i64, i64, vp, vp]),
        "volta_b200_colsum_noalloc": (C.c_int, [vp, vp, i64, i64, vp]),
        "volta_b200_version": (C.c_char_p, []),
        "volta_b200_checkpoint_new": (vp, []),
        "volta_b200_checkpoint_free": (None, [vp]),
        "volta_b200_checkpoint_add": (C.c_int, [vp, C.c_char_p, C.POINTER(i64), i32, fp]),
        "volta_b200_checkpoint_save": (C.c_int, [vp, C.c_char_p, i32]),
        "volta_b200_checkpoint_load": (vp, [C.c_char_p]),
        "volta_b200_checkpoint_parse": (vp, [C.c_char_p, i64]),
        "volta_b200_checkpoint_count": (i32, [vp]),
        "volta_b200_checkpoint_entry": (C.c_int, [vp, i32, C.POINTER(C.c_char_p), C.POINTER(C.POINTER(i64)),
                                                  C.POINTER(i32), C.POINTER(fp), C.POINTER(i64)]),
        "volta_b200_export_checkpoint": (C.c_int, [vp, vp, i32]),
        "volta_b200_import_checkpoint": (C.c_int, [vp, vp]),
        "volta_b200_export_checkpoint_named": (C.c_int, [vp, vp, i32, C.POINTER(C.c_char_p), i32]),
        "volta_b200_import_checkpoint_named": (C.c_int, [vp, vp, C.POINTER(C.c_char_p), i32]),
        "volta_b200_checkpoint_match": (C.c_int, [C.POINTER(Config), vp, C.POINTER(C.c_char_p), i32]),
        "volta_b200_dp_wait_selftest": (C.c_int, [vp, i32, i32]),
        "volta_b200_dp_check": (C.c_int, [C.c_char_p, i32, i32, vp, i64, vp]),
        "volta_b200_gemm_route": (C.c_int, [i32, i32, i64, i64, i64, C.POINTER(i32)]),
        "volta_b200_update_selftest": (C.c_int, [i32, C.c_uint64, i64, i32, C.c_uint64, C.POINTER(C.c_uint64 * 3)]),
        "volta_b200_config_size": (i32, []),
        "volta_b200_program_new": (vp, []),
        "volta_b200_program_free": (None, [vp]),
        "volta_b200_program_error": (C.c_char_p, [vp]),
        "volta_b200_program_add": (C.c_int, [vp, i32, i32, C.POINTER(i32), i32, C.POINTER(i64), i32, fp, i32]),
        "volta_b200_program_mark_output": (C.c_int, [vp, i32]),
        "volta_b200_program_compile": (C.c_int, [vp, i32, C.POINTER(CompiledProgram)]),
        "volta_b200_program_bind": (C.c_int, [vp, i32, vp, i64]),
        "volta_b200_program_run": (C.c_int, [vp]),
        "volta_b200_program_fetch": (C.c_int, [vp, i32, vp, i64]),
        "volta_b200_program_update": (C.c_int, [vp, C.POINTER(OptimizerConfig), C.POINTER(i32), C.POINTER(i32), i32, C.c_uint64]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.volta_b200_config_size() != C.sizeof(Config):
        raise VoltaB200Error(-1, "%s was built with a vb200_config of %d bytes, this binding mirrors %d: rebuild the library"
                             % (path, lib.volta_b200_config_size(), C.sizeof(Config)))
    _lib = lib
    return lib
