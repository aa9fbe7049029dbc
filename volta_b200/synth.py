"""Seeded synthetic inputs and weights, identical on every rank and for the oracle.

A counter-based generator (SplitMix64 of seed + index) so that any row range can be
produced independently: rank k of N generates rows [k*B/N, (k+1)*B/N) of the same global
tensor without materialising the rest.  Normal variates come from Box-Muller on two
uniform draws per element (element index i uses counters 2i and 2i+1).
Seeds: 42 weights, 1234 inputs, 4321 targets.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = x + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _u01(seed: int, counters: np.ndarray) -> np.ndarray:
    """Uniform doubles in (0, 1) from 53 random bits of SplitMix64(seed-mixed counter)."""
    with np.errstate(over="ignore"):
        base = _splitmix64(np.array([seed], dtype=np.uint64))[0]
        bits = _splitmix64(counters ^ base)
    return ((bits >> np.uint64(11)).astype(np.float64) + 0.5) * (1.0 / 9007199254740992.0)


def uniform(seed: int, start: int, count: int, lo=-1.0, hi=1.0, chunk=1 << 22) -> np.ndarray:
    out = np.empty(count, dtype=np.float32)
    for a in range(0, count, chunk):
        b = min(count, a + chunk)
        idx = np.arange(start + a, start + b, dtype=np.uint64)
        out[a:b] = (lo + (hi - lo) * _u01(seed, idx)).astype(np.float32)
    return out


def normal(seed: int, start: int, count: int, chunk=1 << 22) -> np.ndarray:
    out = np.empty(count, dtype=np.float32)
    for a in range(0, count, chunk):
        b = min(count, a + chunk)
        idx = np.arange(start + a, start + b, dtype=np.uint64)
        u1 = _u01(seed, idx * np.uint64(2))
        u2 = _u01(seed, idx * np.uint64(2) + np.uint64(1))
        out[a:b] = (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)
    return out


def rows(dist: str, seed: int, row0: int, nrows: int, width: int) -> np.ndarray:
    """Rows [row0, row0+nrows) of a global [*, width] tensor."""
    fn = normal if dist == "normal" else uniform
    return fn(seed, row0 * width, nrows * width).reshape(nrows, width)


def kaiming_uniform_weights(layers, seed: int = 42):
    """U(-sqrt(6/fan_in), +sqrt(6/fan_in)) per layer from one stream in layer order
    (ReLU gain sqrt(2), fan_in = rows of W[in x out]); biases zero."""
    ws, bs, start = [], [], 0
    for r, c in zip(layers[:-1], layers[1:]):
        lim = float(np.sqrt(6.0 / r))
        ws.append(uniform(seed, start, r * c, -lim, lim).reshape(r, c))
        bs.append(np.zeros(c, dtype=np.float32))
        start += r * c
    return ws, bs


# ---------------------------------------------------------------------------------------------
# The same kind of tensors generated ON the GPU, for configurations whose inputs and weights are
# too large to draw with numpy in reasonable time (configuration 5: 2.1 GB of inputs, 1.6 GB of
# weights).  Blocks of 4096 rows (of 2^22 elements for weights) are seeded by (seed, block index), so
# any rank generates exactly its rows of the same global tensor; values differ from the numpy
# generator above (another bit source), distributions and shapes are the same.
# ---------------------------------------------------------------------------------------------
_DEV_BLOCK_ROWS = 4096


def rows_cuda(dist: str, seed: int, row0: int, nrows: int, width: int, device=None):
    """Rows [row0, row0+nrows) of a global [*, width] tensor as a CUDA tensor; row0 and nrows must be
    multiples of 4096 or lie inside one block."""
    import torch
    device = device or torch.device("cuda", torch.cuda.current_device())
    out = torch.empty((nrows, width), dtype=torch.float32, device=device)
    gen = torch.Generator(device=device)
    r = row0
    while r < row0 + nrows:
        blk = r // _DEV_BLOCK_ROWS
        lo, hi = blk * _DEV_BLOCK_ROWS, (blk + 1) * _DEV_BLOCK_ROWS
        gen.manual_seed((seed << 20) + blk)
        full = torch.empty((_DEV_BLOCK_ROWS, width), dtype=torch.float32, device=device)
        full.normal_(generator=gen) if dist == "normal" else full.uniform_(-1.0, 1.0, generator=gen)
        a, b = r, min(hi, row0 + nrows)
        out[a - row0:b - row0] = full[a - lo:b - lo]
        r = b
    return out


def kaiming_uniform_weights_cuda(layers, seed: int = 42, device=None):
    """U(-sqrt(6/fan_in), +sqrt(6/fan_in)) per layer as CUDA tensors, one generator seed per layer; biases zero."""
    import torch
    device = device or torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=device)
    ws, bs = [], []
    for i, (r, c) in enumerate(zip(layers[:-1], layers[1:])):
        lim = float(np.sqrt(6.0 / r))
        gen.manual_seed((seed << 20) + i)
        ws.append(torch.empty((r, c), dtype=torch.float32, device=device).uniform_(-lim, lim, generator=gen))
        bs.append(torch.zeros(c, dtype=torch.float32, device=device))
    return ws, bs
