"""Seeded synthetic inputs with the shapes and value distributions of the five
benchmark configurations (stand-ins: the reference measures on no public dataset).

By default everything is drawn on the CPU in float32 from
``torch.Generator().manual_seed(k)`` and rounded to bf16 afterwards, so every machine
sees identical bits (what the parity tests use).  ``device="cuda"`` draws the same
distributions with the CUDA generator instead (what the benchmark uses: the values
differ from the CPU stream, the shapes and distributions do not).  ``scale`` shrinks
a configuration (rows and columns divided, distributions kept).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class Config:
    name: str
    rows: int
    cols: int
    dtype: torch.dtype
    seed: int
    what: str


CONFIGS = {
    1: Config("per_tensor_e4m3_4096x4096", 4096, 4096, torch.bfloat16, 0,
              "N(0,1); scale = 448/amax; E4M3 RNE cast and dequantize"),
    2: Config("per_channel_8192x8192", 8192, 8192, torch.bfloat16, 1,
              "N(0, 0.02^2), row r times 10^U(-2,2); per-row E4M3 and E5M2"),
    3: Config("mx_1x32_16384x8192", 16384, 8192, torch.bfloat16, 2,
              "0.5 * Student-t(3) with 0.1% entries set to +-1000; 1x32 groups, E8M0 scales, E4M3 and E2M3"),
    4: Config("mor_128x128_32768x8192", 32768, 8192, torch.bfloat16, 3,
              "128x128 blocks alternating N(0,1), Laplace(0,1e-3), log-uniform 1e-6..1e4; MoR choice"),
    5: Config("sharded_fp32_131072x16384", 131072, 16384, torch.float32, 4,
              "N(0,1) float32, 8 GiB; global amax then per-tensor / block-scaled E4M3"),
}


def _gen(seed: int, device="cpu") -> torch.Generator:
    return torch.Generator(device=device).manual_seed(seed)


def config1(scale: int = 1, device="cpu") -> torch.Tensor:
    c = CONFIGS[1]
    return torch.randn(c.rows // scale, c.cols // scale, generator=_gen(c.seed, device), device=device).to(torch.bfloat16)


def config2(scale: int = 1, device="cpu") -> torch.Tensor:
    c = CONFIGS[2]
    g = _gen(c.seed, device)
    rows, cols = c.rows // scale, c.cols // scale
    x = torch.randn(rows, cols, generator=g, device=device) * 0.02
    f = 10.0 ** (torch.rand(rows, generator=g, device=device) * 4.0 - 2.0)
    return (x * f[:, None]).to(torch.bfloat16)


def config3(scale: int = 1, device="cpu") -> torch.Tensor:
    c = CONFIGS[3]
    g = _gen(c.seed, device)
    rows, cols = c.rows // scale, c.cols // scale
    z = torch.randn(rows, cols, generator=g, device=device)
    chi = torch.zeros(rows, cols, device=device)
    for _ in range(3):
        chi += torch.randn(rows, cols, generator=g, device=device) ** 2
    x = 0.5 * z / torch.sqrt(chi / 3.0)
    del z, chi
    m = torch.rand(rows, cols, generator=g, device=device) < 0.001
    sign = torch.where(torch.rand(rows, cols, generator=g, device=device) < 0.5, -1.0, 1.0)
    x = torch.where(m, 1000.0 * sign, x)
    return x.to(torch.bfloat16)


def config4(scale: int = 1, block: int = 128, device="cpu") -> torch.Tensor:
    """Block (bi, bj) has kind (bi * blocks_per_row + bj) mod 3: 0 N(0,1), 1 Laplace(0, 1e-3),
    2 sign * 10^U(-6, 4).  Drawn whole-tensor three times and selected per block, so the
    bits do not depend on how the tensor is later sharded."""
    c = CONFIGS[4]
    g = _gen(c.seed, device)
    rows, cols = c.rows // scale, c.cols // scale
    nbx = cols // block
    bi = torch.arange(rows, device=device)[:, None] // block
    bj = torch.arange(cols, device=device)[None, :] // block
    kind = (bi * nbx + bj) % 3
    out = torch.randn(rows, cols, generator=g, device=device)
    u = torch.rand(rows, cols, generator=g, device=device) - 0.5
    lap = -1e-3 * torch.sign(u) * torch.log1p(-2.0 * u.abs().clamp(max=0.49999997))  # rand() == 0 would give inf
    out = torch.where(kind == 1, lap, out)
    del u, lap
    mag = 10.0 ** (torch.rand(rows, cols, generator=g, device=device) * 10.0 - 6.0)
    sgn = torch.where(torch.rand(rows, cols, generator=g, device=device) < 0.5, -1.0, 1.0)
    out = torch.where(kind == 2, mag * sgn, out)
    return out.to(torch.bfloat16)


SLAB_ROWS_5 = 16384  # 1 GiB of float32 at 16384 columns


def config5_slab(slab: int, scale: int = 1, device="cpu") -> torch.Tensor:
    """Row slab `slab` (0-based) of configuration 5: SLAB_ROWS_5 // scale rows of N(0,1)
    float32 from seed 4000 + slab, so shards can be produced independently."""
    c = CONFIGS[5]
    return torch.randn(SLAB_ROWS_5 // scale, c.cols // scale, generator=_gen(c.seed * 1000 + slab, device),
                       device=device)


def config5(scale: int = 1) -> torch.Tensor:
    c = CONFIGS[5]
    n_slabs = c.rows // SLAB_ROWS_5
    return torch.cat([config5_slab(s, scale) for s in range(n_slabs)], dim=0)
