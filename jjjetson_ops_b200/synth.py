"""Seeded synthetic inputs for the five benchmark configurations.

No dataset is involved: every tensor is drawn from ``numpy.random.Generator(PCG64(seed))`` in a
fixed order, so that the CPU oracle, the GPU tests and the benchmark all see the same bits.

Draw order for a linear ``(N, K)`` with ``M`` activation rows: the fp32 weights
``[N, K] ~ N(0, sigma_w)`` first, then the activations ``[M_max, K] ~ N(0, 1)`` (callers slice the
first ``M`` rows, so M = 1, 2, 4, 8 share their leading rows), then, where the configuration asks
for outliers, ``round(0.01 * K)`` distinct channel indices whose activations are multiplied by 20
in every row.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import numpy as np


@dataclass(frozen=True)
class LinearSpec:
    name: str
    K: int
    N: int
    sigma_w: float = 0.02


@dataclass(frozen=True)
class ConfigSpec:
    index: int
    name: str
    seed: int
    linears: Tuple[LinearSpec, ...]
    Ms: Tuple[int, ...]
    outliers: bool = False


CONFIGS = {
    1: ConfigSpec(1, "cfg1 decode GEMV 4096x4096", 0, (LinearSpec("gemv", 4096, 4096),), (1,)),
    2: ConfigSpec(2, "cfg2 decode-batch GEMV 4096->11008", 1, (LinearSpec("ffn_up", 4096, 11008),), (1, 2, 4, 8), True),
    3: ConfigSpec(3, "cfg3 prefill GEMM 512x4096x4096", 2, (LinearSpec("prefill", 4096, 4096),), (512,)),
    4: ConfigSpec(4, "cfg4 sharded 8192->28672", 3, (LinearSpec("ffn70b", 8192, 28672, 0.015),), (1, 2048)),
    5: ConfigSpec(
        5, "cfg5 Llama-7B layer chain", 4,
        (
            LinearSpec("qkv", 4096, 12288), LinearSpec("o", 4096, 4096), LinearSpec("gate", 4096, 11008),
            LinearSpec("up", 4096, 11008), LinearSpec("down", 11008, 4096),
        ),
        (1, 128),
    ),
}


def make_weights(rng: np.random.Generator, spec: LinearSpec, rows: Optional[int] = None) -> np.ndarray:
    """fp32 ``[N, K]``; ``rows`` limits how many rows are materialised (the draws of the rest are
    still consumed so that later tensors do not depend on it)."""
    n = spec.N if rows is None else min(rows, spec.N)
    w = rng.standard_normal((spec.N, spec.K), dtype=np.float32)
    w *= np.float32(spec.sigma_w)
    return w[:n]


def make_activations(rng: np.random.Generator, K: int, M: int, outliers: bool) -> np.ndarray:
    x = rng.standard_normal((M, K), dtype=np.float32)
    if outliers:
        idx = rng.choice(K, size=int(round(0.01 * K)), replace=False)
        x[:, idx] *= np.float32(20.0)
    return x


def make_linear_case(cfg: int, linear: int = 0, M: Optional[int] = None, rows: Optional[int] = None):
    """-> ``(W fp32 [N or rows, K], X fp32 [M, K], spec)`` for one linear of configuration ``cfg``.

    For cfg5 every linear draws from its own generator ``PCG64(seed * 100 + linear)`` and takes a
    fresh ``N(0, 1)`` input (the configuration fixes this for ``down``; using it for every step
    keeps the five multiplies independent and individually checkable).
    """
    spec = CONFIGS[cfg]
    lin = spec.linears[linear]
    seed = spec.seed if len(spec.linears) == 1 else spec.seed * 100 + linear
    rng = np.random.default_rng(np.random.PCG64(seed))
    w = make_weights(rng, lin, rows)
    m_max = max(spec.Ms)
    x = make_activations(rng, lin.K, m_max, spec.outliers)
    if M is not None:
        x = np.ascontiguousarray(x[:M])
    return w, x, lin


def shard_rows(N: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous N-shard ``[begin, end)`` of rank ``rank``; sizes differ by at most one 32-row unit."""
    units = (N + 31) // 32
    b = (units * rank // world) * 32
    e = min(N, (units * (rank + 1) // world) * 32)
    return min(b, N), e


def algorithmic_bytes(K: int, N: int, M: int, fused_quantize: bool = True) -> int:
    """Bytes one linear must move: weights once, activations once, outputs once.

    With the quantizer fused the activations are read as fp32 (``M*K*4``); otherwise as Q8_1 blocks
    (``M*K/128*144``)."""
    w = N * (K // 32) * 18
    x = M * K * 4 if fused_quantize else M * (K // 128) * 144
    return w + x + M * N * 4


def ops(K: int, N: int, M: int) -> int:
    return 2 * M * N * K
