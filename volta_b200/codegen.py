"""Per-model training libraries for the CUDA target.

`compile_model` plays the part of the reference's compile_mlp_train_rust_dll
(src/engine/ir/codegen/mlp_train_rust_codegen.rs:143-247): given an MLP topology it
produces one shared object exporting volta_train_init/_step/_loss/_get_params/_set_params/
_free.  The work is done by the native tool volta-b200-codegen (codegen_src/main.cpp).
"""
from __future__ import annotations

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
TOOL = os.path.join(HERE, "volta-b200-codegen")
SRC = os.path.join(HERE, "codegen_src", "main.cpp")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")


class CodegenError(RuntimeError):
    pass


def build_tool(force: bool = False) -> str:
    if force or not os.path.exists(TOOL) or os.path.getmtime(TOOL) < os.path.getmtime(SRC):
        r = subprocess.run(["g++", "-O2", "-std=c++17", SRC, "-o", TOOL], capture_output=True, text=True)
        if r.returncode != 0:
            raise CodegenError("building volta-b200-codegen failed:\n" + r.stderr)
    return TOOL


def compile_model(layers, activation: str, optimizer: str, out_path: str, emit_only: bool = False, *,
                  dropout_p: float = 0.0, use_layernorm: bool = False, clip_grad: float = 0.0,
                  infer: bool = False, checkpoint: str | None = None) -> str:
    """Emit (and link) the training library for one model; returns the path produced."""
    tool = build_tool()
    cmd = [tool, "--layers", ",".join(str(int(x)) for x in layers), "--activation", activation, "--optimizer",
           optimizer, "-o", out_path, "--libdir", HERE, "--include", INCLUDE]
    if dropout_p:
        cmd += ["--dropout", repr(float(dropout_p))]
    if use_layernorm:
        cmd.append("--layernorm")
    if clip_grad:
        cmd += ["--clip-grad", repr(float(clip_grad))]
    if infer:
        cmd.append("--infer")
    if checkpoint:
        cmd += ["--checkpoint", str(checkpoint)]
    if emit_only:
        cmd.append("--emit-only")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise CodegenError(r.stderr.strip() or "volta-b200-codegen failed")
    return r.stdout.strip().splitlines()[-1]
