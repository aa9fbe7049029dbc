"""volta_b200 — B200 (sm_100a) implementation of Volta's compiled MLP training step.

The product is libvolta_b200.so (C ABI, include/volta_b200.h).  This package is the thin
host side around it: the loader (lib.py), a handle class mirroring the six volta_train_*
entry points of the reference's generated library (train.py), the per-model shim emitter
(codegen.py), the benchmark configurations (configs.py) and the seeded input generator
(synth.py).  There is no CPU or PyTorch fallback: without the compiled library, or without
a CUDA device, creating a handle raises.
"""
from .lib import load_library, library_path, VoltaB200Error  # noqa: F401
from .train import TrainHandle, ACTIVATIONS, OPTIMIZERS  # noqa: F401
from .configs import CONFIGS, MlpConfig  # noqa: F401

__all__ = ["load_library", "library_path", "VoltaB200Error", "TrainHandle", "ACTIVATIONS", "OPTIMIZERS",
           "CONFIGS", "MlpConfig"]
