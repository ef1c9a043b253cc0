"""Seeded synthetic Q/K/V with the shapes of a video diffusion transformer layer.

Real activations of the model are not available offline, so the tests and the
benchmark use a *3D locality mixture*: tokens lie on a (T, Y, X) latent grid in
row-major order; every head draws 512 centres ~ N(0, 1) in R^128; each grid
block of 1 x 4 x 4 tokens (edge blocks truncated) picks one centre uniformly;
K_i = centre + 0.3 eps_i, Q_i = centre + 0.3 eps'_i with independent noise, and
V ~ N(0, 1).  Everything is generated on the CPU from `torch.Generator` seeds
(`seed + head`), so every device sees identical bits.
"""
from __future__ import annotations

import torch

GRIDS = {
    "cpu": (4, 32, 32),        # N = 4,096
    "480p": (21, 30, 52),      # N = 32,760
    "720p": (21, 45, 80),      # N = 75,600
}


def grid_tokens(grid) -> int:
    t, y, x = grid
    return t * y * x


def locality_mixture(H: int, grid, *, D: int = 128, seed: int = 1234, centres: int = 512,
                     noise: float = 0.3, dtype=torch.bfloat16, heads=None):
    """Returns q, k, v of shape [H, N, D] in `dtype` on the CPU.

    `heads` (optional) lists the global head indices to generate, so that a
    rank holding heads [a, b) of a larger layer gets exactly the tensors the
    single-GPU run would give those heads."""
    T, Y, X = grid
    N = T * Y * X
    heads = list(range(H)) if heads is None else list(heads)
    t = torch.arange(T)[:, None, None].expand(T, Y, X)
    y = torch.arange(Y)[None, :, None].expand(T, Y, X)
    x = torch.arange(X)[None, None, :].expand(T, Y, X)
    by, bx = (Y + 3) // 4, (X + 3) // 4
    block = ((t * by + y // 4) * bx + x // 4).reshape(N)
    nblocks = T * by * bx
    q = torch.empty(len(heads), N, D, dtype=dtype)
    k = torch.empty(len(heads), N, D, dtype=dtype)
    v = torch.empty(len(heads), N, D, dtype=dtype)
    for i, h in enumerate(heads):
        g = torch.Generator(device="cpu").manual_seed(seed + h)
        cen = torch.randn(centres, D, generator=g)
        pick = torch.randint(0, centres, (nblocks,), generator=g)
        base = cen[pick[block]]
        k[i] = (base + noise * torch.randn(N, D, generator=g)).to(dtype)
        q[i] = (base + noise * torch.randn(N, D, generator=g)).to(dtype)
        v[i] = torch.randn(N, D, generator=g).to(dtype)
    return q, k, v
