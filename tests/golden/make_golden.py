"""Regenerate tests/golden/mlp_parity.json by importing the reference's own PyTorch
parity script (examples/pytorch_parity.py) from a checkout of the reference.

The reference's Rust parity tests (tests/pytorch_parity.rs:1949-2417) shell out to that
script and compare against what it prints; this captures the same values, together with
the fixture inputs (dataset, initial parameters, learning rates) defined in the script
(examples/pytorch_parity.py:613-857), so that the oracle can be pinned where no
checkout is available.

Usage:  python tests/golden/make_golden.py /path/to/reference
"""
import importlib.util
import json
import os
import sys

import torch

if len(sys.argv) < 2:
    sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
ref_root = sys.argv[1]
spec = importlib.util.spec_from_file_location("pytorch_parity", os.path.join(ref_root, "examples", "pytorch_parity.py"))
pp = importlib.util.module_from_spec(spec)
spec.loader.exec_module(pp)

torch.manual_seed(0)
torch.set_num_threads(1)

w1, b1, w2, b2 = pp.mlp_train_parameters()
dataset = pp.mlp_train_dataset()
out = {
    "source": "examples/pytorch_parity.py (mlp_train_* cases), torch %s" % torch.__version__,
    "layers": [3, 4, 2],
    "activation": "relu",
    "batch": 2,
    "init": {
        "w1": w1.detach().reshape(-1).tolist(), "b1": b1.detach().reshape(-1).tolist(),
        "w2": w2.detach().reshape(-1).tolist(), "b2": b2.detach().reshape(-1).tolist(),
    },
    "dataset": [{"x": x.reshape(-1).tolist(), "y": y.reshape(-1).tolist()} for x, y in dataset],
    # learning rates / epochs as set in mlp_train_loop_case (examples/pytorch_parity.py:725-760)
    "hyper": {
        "sgd": {"lr": 0.05, "epochs": 3}, "adam": {"lr": 0.01, "epochs": 3}, "adamw": {"lr": 0.01, "epochs": 3},
        "adagrad": {"lr": 0.1, "epochs": 3}, "long_sgd": {"lr": 0.05, "epochs": 24},
        "long_adam": {"lr": 0.01, "epochs": 24}, "long_adamw": {"lr": 0.01, "epochs": 24},
    },
    "cases": {
        "mlp_train_sgd": pp.mlp_train_sgd_case(),
        "mlp_train_loop_sgd": pp.mlp_train_loop_sgd_case(),
        "mlp_train_loop_adam": pp.mlp_train_loop_adam_case(),
        "mlp_train_loop_adamw": pp.mlp_train_loop_adamw_case(),
        "mlp_train_loop_adagrad": pp.mlp_train_loop_adagrad_case(),
        "mlp_train_loop_long_sgd": pp.mlp_train_loop_long_sgd_case(),
        "mlp_train_loop_long_adam": pp.mlp_train_loop_long_adam_case(),
        "mlp_train_loop_long_adamw": pp.mlp_train_loop_long_adamw_case(),
    },
}
dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "mlp_parity.json")
with open(dst, "w") as f:
    json.dump(out, f, indent=1)
print("wrote", dst)
