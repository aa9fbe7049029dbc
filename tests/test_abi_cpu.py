"""CPU-side checks of the C-ABI boundary: the library loads, exports every symbol the
header declares, plans memory without a GPU, and refuses to run without one."""
import ctypes as C
import os
import re

import pytest
import torch

from volta_b200 import CONFIGS, VoltaB200Error, load_library
from volta_b200.lib import EXPORTS, Config
from volta_b200.train import ACTIVATIONS, OPTIMIZERS, TrainHandle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "volta_b200.h")).read()
    return sorted(set(re.findall(r"\b(volta_b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = load_library()
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), "libvolta_b200.so does not export %s" % name
    assert sorted(EXPORTS) == declared, "volta_b200/lib.py and include/volta_b200.h disagree"
    assert b"sm_100a" in lib.volta_b200_version()


def test_binding_mirrors_the_configuration_struct_byte_for_byte():
    """The ctypes mirror and the header's struct have the same size (the loader refuses a library that disagrees),
    and the mirror names every field of the header in the header's order."""
    lib = load_library()
    assert lib.volta_b200_config_size() == C.sizeof(Config)
    text = open(os.path.join(ROOT, "include", "volta_b200.h")).read()
    body = text[text.index("typedef struct vb200_config {"):text.index("} vb200_config;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    declared = re.findall(r"\b(?:int32_t|float|uint8_t)\s+([a-z_0-9]+)\s*(?:\[[^\]]*\])?\s*;", body)
    assert declared == [name for name, _ in Config._fields_]


def _cfg(cfg, batch=None, world=1):
    c = Config()
    c.n_sizes = len(cfg.layers)
    for i, v in enumerate(cfg.layers):
        c.layers[i] = v
    c.activation = ACTIVATIONS[cfg.activation]
    c.optimizer = OPTIMIZERS[cfg.optimizer]
    c.batch = (batch or cfg.batch) // world
    c.global_batch = batch or cfg.batch
    c.world_size = world
    return c


def _plan(c):
    lib = load_library()
    total, unshared = C.c_int64(), C.c_int64()
    report = C.create_string_buffer(1 << 16)
    rc = lib.volta_b200_plan(C.byref(c), C.byref(total), C.byref(unshared), report, len(report))
    assert rc == 0, lib.volta_b200_last_error(None)
    bufs = []
    for line in report.value.decode().splitlines():
        name, off, size, first, last, pers = line.split()
        bufs.append((name, int(off), int(size), int(first), int(last), int(pers)))
    return total.value, unshared.value, bufs


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_memory_plan_has_no_live_overlap(name):
    total, unshared, bufs = _plan(_cfg(CONFIGS[name]))
    assert total <= unshared
    for i, a in enumerate(bufs):
        assert a[1] % 1024 == 0 and a[1] + a[2] <= total
        for b in bufs[i + 1:]:
            live = a[5] or b[5] or (a[3] <= b[4] and b[3] <= a[4])
            if live:
                assert a[1] + a[2] <= b[1] or b[1] + b[2] <= a[1], (a, b)


def test_memory_plan_reuses_temporaries_and_fits_one_gpu():
    total, unshared, bufs = _plan(_cfg(CONFIGS["c5"]))
    assert total < unshared            # deltas and activations share storage
    assert total < 170e9               # the largest configuration fits one 180 GB GPU
    temps = [b for b in bufs if not b[5]]
    assert any(a[1] == b[1] for i, a in enumerate(temps) for b in temps[i + 1:])
    # sharded over 8 ranks the activations shrink 8x, parameters do not
    total8, _, _ = _plan(_cfg(CONFIGS["c5"], world=8))
    assert total8 < total


def _check_no_live_overlap(total, bufs):
    for i, a in enumerate(bufs):
        assert a[1] % 1024 == 0 and a[1] + a[2] <= total
        for b in bufs[i + 1:]:
            if a[5] or b[5] or (a[3] <= b[4] and b[3] <= a[4]):
                assert a[1] + a[2] <= b[1] or b[1] + b[2] <= a[1], (a, b)


def test_memory_plan_of_the_copy_exchange_holds_one_receive_slot_per_rank():
    """dp_exchange = copy: the arena (the one allocation the peers map) also holds world x (parameters + loss slot)
    floats for the peers' pushes, persistent and overlapping nothing; the other exchanges plan no such region."""
    world = 4
    c = _cfg(CONFIGS["c4"], world=world)
    base_total, _, base = _plan(c)
    assert not any(b[0] == "dp_receive_slots" for b in base)
    c.dp_exchange = 2
    total, _, bufs = _plan(c)
    _check_no_live_overlap(total, bufs)
    recv = [b for b in bufs if b[0] == "dp_receive_slots"]
    assert len(recv) == 1 and recv[0][5] == 1
    L = list(CONFIGS["c4"].layers)
    pad64 = lambda v: (v + 63) // 64 * 64
    P = sum(pad64(r * k) for r, k in zip(L[:-1], L[1:])) + sum(pad64(k) for k in L[1:])   # the flat parameter layout
    assert world * (P + 64) * 4 <= recv[0][2] < world * (P + 64) * 4 + 1024
    assert total >= base_total + recv[0][2]
    c.dp_exchange = 3
    lib = load_library()
    t, u = C.c_int64(), C.c_int64()
    assert lib.volta_b200_plan(C.byref(c), C.byref(t), C.byref(u), None, 0) != 0   # unknown exchange refused


def test_memory_plan_with_the_optional_stages():
    """Dropout masks (one byte per hidden element), the LayerNorm parameters and 1/sigma rows, and
    pre-activations for relu once the stored output is no longer the activation's own; the clip keeps
    every activation and delta alive until the dW sweep at the end of the step."""
    c = _cfg(CONFIGS["c2"])
    n, B, L = c.n_sizes - 1, c.batch, list(c.layers[:c.n_sizes])
    base_total, _, base = _plan(c)
    assert not any(b[0].startswith(("pre", "mask", "ln_", "layernorm")) for b in base)
    c.dropout_p, c.use_layernorm = 0.5, 1
    total, _, bufs = _plan(c)
    _check_no_live_overlap(total, bufs)
    by = {b[0]: b for b in bufs}
    for k in range(n - 1):
        assert by["mask%d" % k][2] == B * L[k + 1] and by["pre%d" % k][2] == 4 * B * L[k + 1]
        assert 4 * B <= by["ln_invstd%d" % k][2] <= 4 * B + 1023
        # alive from the layer's forward position to the backward position of its own delta
        assert by["mask%d" % k][3] == k and by["mask%d" % k][4] == n + 1 + (n - 1 - k)
        assert by["act%d" % (k + 1)][4] == by["mask%d" % k][4]
    assert by["layernorm_params"][5] == 1 and by["layernorm_params"][2] >= 4 * 2 * sum(L[1:n])
    assert total > base_total
    c.clip_grad = 1.0
    total_clip, _, bufs = _plan(c)
    _check_no_live_overlap(total_clip, bufs)
    end = 2 * n + 1
    assert all(b[4] == end for b in bufs if b[0].startswith("delta") or (b[0].startswith("act") and b[0] != "act%d" % n))
    assert total_clip >= total
    c.dropout_p = 1.0
    assert load_library().volta_b200_plan(C.byref(c), None, None, None, 0) == 1


def test_plan_holds_the_split_k_slabs_where_a_gemm_needs_them():
    """c4's 4096 x 4096 weight-gradient GEMMs (256 pair tiles on 74 SM pairs) split K in two: the step's GEMM
    scratch holds two output slabs.  c5's GEMMs fill their waves: no slabs beyond what the small-shape path wants."""
    by = {b[0]: b for b in _plan(_cfg(CONFIGS["c4"]))[2]}
    assert by["gemm_splitk_scratch"][2] >= 2 * 4096 * 4096 * 4
    by5 = {b[0]: b for b in _plan(_cfg(CONFIGS["c5"]))[2]}
    assert by5["gemm_splitk_scratch"][2] < 4096 * 4096 * 4


def test_plan_rejects_bad_configs():
    lib = load_library()
    c = _cfg(CONFIGS["c1"])
    c.n_sizes = 1
    assert lib.volta_b200_plan(C.byref(c), None, None, None, 0) != 0
    c = _cfg(CONFIGS["c1"])
    c.optimizer = 17       # e.g. RMSprop: outside the generated step's list (executor.rs:3147-3189)
    assert lib.volta_b200_plan(C.byref(c), None, None, None, 0) == 6
    c = _cfg(CONFIGS["c1"])
    c.batch = 0
    assert lib.volta_b200_plan(C.byref(c), None, None, None, 0) == 1


def test_unsupported_names_are_rejected_before_the_library_is_called():
    with pytest.raises(VoltaB200Error):
        TrainHandle([4, 4, 1], "relu", "rmsprop", 2)
    with pytest.raises(VoltaB200Error):
        TrainHandle([4, 4, 1], "softplus", "sgd", 2)


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_create_fails_loudly_without_a_gpu():
    with pytest.raises(VoltaB200Error) as e:
        TrainHandle([4, 4, 1], "relu", "sgd", 2)
    assert "no CPU fallback" in str(e.value)


def _train_symbols():
    text = open(os.path.join(ROOT, "include", "volta_train.h")).read()
    return sorted(set(re.findall(r"\b(volta_train_[a-z_]+)\s*\(", text)))


def test_codegen_emits_a_library_with_the_reference_symbols(tmp_path):
    from volta_b200 import codegen
    out = codegen.compile_model([512, 1024, 1024, 512, 256, 1], "relu", "adam", str(tmp_path / "m.train_cuda.so"))
    lib = C.CDLL(out)
    syms = _train_symbols()
    assert syms == ["volta_train_free", "volta_train_get_params", "volta_train_init", "volta_train_loss",
                    "volta_train_set_params", "volta_train_step"]
    for s in syms:
        assert hasattr(lib, s)
    src = open(out + ".shim.c").read()
    assert "512, 1024, 1024, 512, 256, 1" in src


def test_codegen_rejects_what_the_reference_rejects(tmp_path):
    # tests/cli_smoke.rs:207-379: compile-train refuses RMSprop on the Rust path and non-MLP input
    from volta_b200 import codegen
    with pytest.raises(codegen.CodegenError, match="does not support optimizer"):
        codegen.compile_model([4, 4, 1], "relu", "rmsprop", str(tmp_path / "a.so"))
    with pytest.raises(codegen.CodegenError, match="need >= 2 layer sizes"):
        codegen.compile_model([4], "relu", "sgd", str(tmp_path / "b.so"))
    with pytest.raises(codegen.CodegenError, match="does not support activation"):
        codegen.compile_model([4, 4, 1], "mish", "sgd", str(tmp_path / "c.so"))
    with pytest.raises(codegen.CodegenError, match="--dropout must lie"):
        codegen.compile_model([4, 4, 1], "relu", "sgd", str(tmp_path / "d.so"), dropout_p=1.5)


def test_codegen_compiles_the_topology_switches_in(tmp_path):
    """MlpTopology's dropout_p / use_layernorm / clip_grad (mlp_train_rust_codegen.rs:34-38) and the
    softmax activation end up in the emitted init function."""
    from volta_b200 import codegen
    out = codegen.compile_model([8, 16, 4], "softmax", "sgd", str(tmp_path / "o.so"), emit_only=True,
                                dropout_p=0.25, use_layernorm=True, clip_grad=1.5)
    src = open(out).read()
    assert "cfg.activation = 6;" in src and "cfg.use_layernorm = 1;" in src
    assert "cfg.dropout_p = (float)0.25;" in src and "cfg.clip_grad = (float)1.5;" in src
    plain = open(codegen.compile_model([8, 16, 4], "relu", "sgd", str(tmp_path / "p.so"), emit_only=True)).read()
    assert "cfg.use_layernorm = 0;" in plain and "cfg.dropout_p = (float)0;" in plain


def test_codegen_emits_an_inference_library_with_the_checkpoint_embedded(tmp_path):
    """--infer: one exported function, volta_infer (include/volta_infer.h; the reference's
    src/engine/ir/codegen/inner.rs:194-198), the checkpoint file's bytes inside the image."""
    import numpy as np
    from volta_b200 import codegen
    from volta_b200.checkpoint import Checkpoint
    ck = Checkpoint()
    marker = np.arange(32, dtype=np.float32).reshape(8, 4) + np.float32(0.123)
    ck.add("layer0.weight", marker)
    ck.save(tmp_path / "m.ckpt", 2)
    out = codegen.compile_model([8, 4], "relu", "sgd", str(tmp_path / "m.infer.so"), infer=True,
                                checkpoint=str(tmp_path / "m.ckpt"))
    lib = C.CDLL(out)
    assert hasattr(lib, "volta_infer") and not hasattr(lib, "volta_train_init")
    assert marker.tobytes() in open(out, "rb").read()
    header = open(os.path.join(ROOT, "include", "volta_infer.h")).read()
    assert re.findall(r"\b(volta_infer)\s*\(", header)
    with pytest.raises(codegen.CodegenError, match="cannot read checkpoint"):
        codegen.compile_model([8, 4], "relu", "sgd", str(tmp_path / "n.so"), infer=True, checkpoint=str(tmp_path / "nope"))
    with pytest.raises(codegen.CodegenError, match="goes with --infer"):
        codegen.compile_model([8, 4], "relu", "sgd", str(tmp_path / "n.so"), checkpoint=str(tmp_path / "m.ckpt"))
