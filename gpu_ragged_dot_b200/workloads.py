"""Seeded synthetic workloads with the shapes and value distributions of the benchmark
configurations (MoE expert GEMMs).  No dataset is involved: the reference's own tests and
tuner also draw random normals (tests.py:51-71, tuning.py:31-45).

group_sizes always come from NumPy's ``default_rng(seed)`` on the host so they are identical
on every machine; the large tensors are drawn with torch on whichever device is asked for.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch


@dataclass(frozen=True)
class Shape:
    name: str
    m: int
    k: int
    n: int
    g: int


SMALL = Shape("small_m512_k256_n384_g8", 512, 256, 384, 8)
MIXTRAL = Shape("mixtral8x7b_up_m8192_k4096_n14336_g8", 8192, 4096, 14336, 8)
DEEPSEEK_V3 = Shape("deepseekv3_m32768_k7168_n2048_g256", 32768, 7168, 2048, 256)
# a quarter of the DeepSeek-V3 shape (same k, n and mean rows per expert): small enough for a
# profiler capture, still 1.9 GB of weights
DEEPSEEK_QUARTER = Shape("deepseekv3_quarter_m8192_k7168_n2048_g64", 8192, 7168, 2048, 64)
EP_PREFILL = Shape("ep_prefill_m32768_k4096_n1536_g64", 32768, 4096, 1536, 64)
EP_DECODE = Shape("ep_decode_m256_k4096_n1536_g64", 256, 4096, 1536, 64)


def group_sizes_small(seed: int = 0) -> np.ndarray:
    """multinomial(512, Dirichlet(1)) over 8 groups, forced to contain an empty group."""
    rng = np.random.default_rng(seed)
    gs = rng.multinomial(SMALL.m, rng.dirichlet(np.ones(SMALL.g))).astype(np.int32)
    if not (gs == 0).any():
        lo, hi = int(np.argmin(gs)), int(np.argmax(gs))
        gs[hi] += gs[lo]
        gs[lo] = 0
    return gs


def group_sizes_mixtral(seed: int = 0) -> np.ndarray:
    """multinomial(8192, Dirichlet(2)) over 8 experts."""
    rng = np.random.default_rng(seed)
    return rng.multinomial(MIXTRAL.m, rng.dirichlet(2.0 * np.ones(MIXTRAL.g))).astype(np.int32)


def group_sizes_mixtral_ragged(seed: int = 0) -> np.ndarray:
    """The Mixtral sizes with every group moved to a random offset mod 128 (sum kept at m)."""
    gs = group_sizes_mixtral(seed).astype(np.int64)
    rng = np.random.default_rng(seed + 1)
    r = rng.integers(1, 128, size=gs.size)
    gs = 128 * (gs // 128) + r
    gs[-1] += MIXTRAL.m - gs.sum()
    assert gs.min() >= 0 and gs.sum() == MIXTRAL.m
    return gs.astype(np.int32)


def group_sizes_deepseek(seed: int = 0) -> np.ndarray:
    """Heavy-tailed multinomial(32768, Dirichlet(0.3)) over 256 experts (~20% empty)."""
    rng = np.random.default_rng(seed)
    p = rng.dirichlet(0.3 * np.ones(DEEPSEEK_V3.g))
    return rng.multinomial(DEEPSEEK_V3.m, p).astype(np.int32)


def group_sizes_deepseek_quarter(seed: int = 0) -> np.ndarray:
    """multinomial(8192, Dirichlet(0.3)) over 64 experts: the DeepSeek draw at a quarter of the size."""
    rng = np.random.default_rng(seed)
    p = rng.dirichlet(0.3 * np.ones(DEEPSEEK_QUARTER.g))
    return rng.multinomial(DEEPSEEK_QUARTER.m, p).astype(np.int32)


def topk_routing(tokens: int, experts: int, top_k: int, seed: int) -> np.ndarray:
    """[tokens, top_k] distinct expert ids per token, uniform at random."""
    rng = np.random.default_rng(seed)
    perm = rng.permuted(np.tile(np.arange(experts, dtype=np.int32), (tokens, 1)), axis=1)
    return np.ascontiguousarray(perm[:, :top_k])


def group_sizes_from_routing(routing: np.ndarray, experts: int) -> np.ndarray:
    return np.bincount(routing.reshape(-1), minlength=experts).astype(np.int32)


def normal_tensor(shape, std: float, seed: int, device, dtype=torch.bfloat16,
                  chunk_rows: Optional[int] = None) -> torch.Tensor:
    """N(0, std^2) drawn in fp32 on `device` with a seeded generator, rounded to `dtype`."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = torch.empty(shape, dtype=dtype, device=device)
    flat = out.view(-1)
    step = 1 << 26
    for lo in range(0, flat.numel(), step):
        hi = min(lo + step, flat.numel())
        flat[lo:hi] = (torch.randn(hi - lo, generator=gen, device=device, dtype=torch.float32) * std).to(dtype)
    return out


def make_inputs(shape: Shape, device, seed: int = 0, dtype=torch.bfloat16, with_dout: bool = True):
    """x ~ N(0,1) [m,k];  A ~ N(0,1/k) [g,k,n];  dout ~ N(0,1) [m,n]."""
    x = normal_tensor((shape.m, shape.k), 1.0, seed * 3 + 11, device, dtype)
    A = normal_tensor((shape.g, shape.k, shape.n), shape.k ** -0.5, seed * 3 + 12, device, dtype)
    dout = normal_tensor((shape.m, shape.n), 1.0, seed * 3 + 13, device, dtype) if with_dout else None
    return x, A, dout
