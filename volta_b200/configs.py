"""The benchmark configurations (layers, activation, optimizer, batch, steps, input
distributions).  C1-C3 are single-GPU, C4/C5 shard the global batch over the ranks."""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class MlpConfig:
    name: str
    layers: tuple
    activation: str
    optimizer: str
    lr: float
    batch: int            # global batch
    steps: int
    x_dist: str = "normal"   # "normal" N(0,1) or "uniform" U(-1,1)
    y_dist: str = "normal"
    sharded: bool = False
    note: str = ""

    @property
    def n_params(self) -> int:
        return sum(r * c + c for r, c in zip(self.layers[:-1], self.layers[1:]))

    def flops_per_step(self, batch: int | None = None) -> float:
        """Logical fp32 flops of one step: forward + dW for every layer, dX for layers >= 1."""
        b = self.batch if batch is None else batch
        rc = [r * c for r, c in zip(self.layers[:-1], self.layers[1:])]
        return 2.0 * b * (2 * sum(rc) + sum(rc[1:]))

    def optimizer_bytes_per_param(self) -> int:
        return {"sgd": 12, "adam": 28, "adamw": 28, "adagrad": 20, "sgd_momentum": 20}[self.optimizer]


CONFIGS = {
    "c1": MlpConfig("c1", (256, 512, 512, 256, 1), "relu", "sgd", 0.01, 64, 50),
    "c2": MlpConfig("c2", (512, 1024, 1024, 512, 256, 1), "relu", "adam", 1e-3, 64, 50),
    "c3_b64": MlpConfig("c3_b64", (512, 2048, 2048, 512, 1), "gelu", "adamw", 1e-3, 64, 50),
    "c3_b1024": MlpConfig("c3_b1024", (512, 2048, 2048, 512, 1), "gelu", "adamw", 1e-3, 1024, 50),
    "c4": MlpConfig("c4", (1024, 4096, 4096, 4096, 1024, 1), "silu", "sgd_momentum", 0.01, 65536, 20,
                    x_dist="uniform", sharded=True, note="lr is not given by the configuration; 0.01 is used"),
    "c5": MlpConfig("c5", (4096, 16384, 16384, 4096, 1), "relu", "adam", 1e-3, 131072, 10, sharded=True),
}
