"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

All tensors are generated on the CPU with an explicit generator in fp32 and cast last, so that the GPU path and
the CPU oracle see identical bits.
"""

from __future__ import annotations

import torch


def normal_with_outliers(rows: int, cols: int, seed: int = 0) -> torch.Tensor:
    """N(0,1) with 0.1 % of the entries replaced by N(0,1)*100 (fp32)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    m = torch.rand(rows, cols, generator=g) < 1e-3
    return torch.where(m, torch.randn(rows, cols, generator=g) * 100, x)


def student_t3(rows: int, cols: int, seed: int = 1, scale: float = 0.02, dtype=torch.bfloat16) -> torch.Tensor:
    """Student-t with 3 degrees of freedom times `scale`: z / sqrt(chi2_3 / 3) from seeded normals."""
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(rows, cols, generator=g)
    chi = torch.zeros(rows, cols)
    for _ in range(3):
        chi += torch.randn(rows, cols, generator=g) ** 2
    return (z / (chi / 3).sqrt() * scale).to(dtype)


def linear_operands(m: int, k: int = 4096, n: int = 4096, seed: int = 2, dtype=torch.bfloat16):
    """W[n,k] ~ N(0, 0.02); x[m,k] ~ N(0,1) with 1 % of the k channels scaled by 50."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.02
    ch = torch.rand(k, generator=g) < 0.01
    x = torch.randn(m, k, generator=g)
    x = torch.where(ch.view(1, -1), x * 50, x)
    return x.to(dtype), w.to(dtype)


def device_student_t3(rows: int, cols: int, seed: int, device, dtype=torch.bfloat16, scale: float = 0.02):
    """The same distribution generated directly on a CUDA device (for tensors too large to stage on the host)."""
    g = torch.Generator(device=device).manual_seed(seed)
    out = torch.empty(rows, cols, dtype=dtype, device=device)
    step = max(1, (1 << 26) // cols)
    for r0 in range(0, rows, step):
        r1 = min(rows, r0 + step)
        z = torch.randn(r1 - r0, cols, generator=g, device=device)
        chi = torch.zeros_like(z)
        for _ in range(3):
            chi += torch.randn(r1 - r0, cols, generator=g, device=device) ** 2
        out[r0:r1] = (z / (chi / 3).sqrt() * scale).to(dtype)
    return out
