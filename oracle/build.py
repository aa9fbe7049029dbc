"""Build recipe for the CPU oracle (test infrastructure, never shipped).

Produces, next to this file:
  _build/liboracle_f32.so   golden fp32 restatement (strict IEEE, no contraction)
  _build/liboracle_f64.so   fp64 shadow of the same source
  _ref/libgemm_shim_<flavour>.so
      the reference's own src/engine/ir/codegen/gemm_shim.c compiled, unmodified and
      from where it lies, with the reference's flags (-O3 -ffast-math -funroll-loops,
      cpu_target.rs:33-38).  -fopenmp, which mlp_train_codegen.rs:76-81 adds only when
      it finds an OpenMP runtime, is left out on purpose: the shim's OpenMP branch packs
      A inside "#pragma omp single" into the executing thread's private buffer while
      the other threads read their own, never-filled buffers (gemm_shim.c:104-131), so
      with more than one thread it returns wrong products (observed here: the loss of
      a 5-step run doubled).  The single-threaded build is the reference's "no OpenMP
      found" configuration.  Built only where the reference checkout is present; the prebuilt
      objects travel with the working tree.  Flavours: "native" (-march=native, usable
      only on a CPU with at least the build host's ISA flags, recorded in
      _ref/native.cpuflags) and "v3" (-march=x86-64-v3, any AVX2 server).
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD = os.path.join(HERE, "_build")
REF = os.path.join(HERE, "_ref")
# The reference checkout: $VOLTA_REFERENCE_ROOT, else a directory named "reference" beside this repository.
REFERENCE_ROOT = os.environ.get("VOLTA_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
SHIM_SRC = os.path.join(REFERENCE_ROOT, "src", "engine", "ir", "codegen", "gemm_shim.c")

STRICT = ["-O3", "-mavx2", "-fPIC", "-shared", "-std=c11", "-ffp-contract=off", "-fno-fast-math",
          "-fno-unsafe-math-optimizations", "-Wall", "-Wno-unused-function"]


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources if os.path.exists(s))


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("oracle build failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))


def _cpuflags() -> set:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def build_oracle(force: bool = False) -> dict:
    os.makedirs(BUILD, exist_ok=True)
    src = os.path.join(HERE, "volta_oracle.c")
    out = {}
    for name, real in (("f32", "float"), ("f64", "double")):
        so = os.path.join(BUILD, "liboracle_%s.so" % name)
        if force or not _newer(so, src, __file__):
            _run(["gcc", *STRICT, "-DORACLE_REAL=%s" % real, src, "-o", so, "-lm"])
        out[name] = so
    return out


def build_ref(force: bool = False) -> dict:
    """Compile the reference's gemm_shim.c where the reference checkout exists."""
    out = {}
    if not os.path.exists(SHIM_SRC):
        for flavour in ("native", "v3"):
            so = os.path.join(REF, "libgemm_shim_%s.so" % flavour)
            if os.path.exists(so):
                out[flavour] = so
        return out
    os.makedirs(REF, exist_ok=True)
    base = ["gcc", "-O3", "-ffast-math", "-funroll-loops", "-fPIC", "-shared"]
    for flavour, march in (("native", "-march=native"), ("v3", "-march=x86-64-v3")):
        so = os.path.join(REF, "libgemm_shim_%s.so" % flavour)
        if force or not _newer(so, SHIM_SRC, __file__):
            _run([*base, march, SHIM_SRC, "-o", so])
        out[flavour] = so
    with open(os.path.join(REF, "native.cpuflags"), "w") as f:
        f.write(" ".join(sorted(_cpuflags())))
    return out


def pick_ref_shim() -> tuple[str, str] | None:
    """Return (flavour, path) of a prebuilt reference GEMM shim this CPU can run."""
    native = os.path.join(REF, "libgemm_shim_native.so")
    flags_file = os.path.join(REF, "native.cpuflags")
    if os.path.exists(native) and os.path.exists(flags_file):
        with open(flags_file) as f:
            need = {x for x in f.read().split() if x.startswith(("avx", "fma", "bmi", "sse", "f16c"))}
        if need <= _cpuflags():
            return "native", native
    v3 = os.path.join(REF, "libgemm_shim_v3.so")
    if os.path.exists(v3) and {"avx2", "fma"} <= _cpuflags():
        return "v3", v3
    return None


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
