"""Lloyd-Max codebook for coordinates of a rotated unit vector, x ~ N(0, 1/d).

Same interface and iteration as the reference (turboquant/core/codebook.py:17-79):
uniform start on [-6 sigma, 6 sigma], 100 Lloyd iterations, boundaries are
midpoints of neighbouring centroids.  The reference integrates the Gaussian
numerically; the cell mass and first moment have closed forms (erf / pdf
differences), which are used here, so construction needs no scipy and takes
microseconds.  Construction is host-side Python by design: kernels receive the
centroid and boundary tensors, never constants.
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def _cell_moments(a: float, b: float, sigma: float) -> tuple[float, float]:
    """(int_a^b x pdf(x) dx, int_a^b pdf(x) dx) for N(0, sigma^2)."""
    k = 1.0 / (sigma * math.sqrt(2.0 * math.pi))
    pa = k * math.exp(-a * a / (2.0 * sigma * sigma))
    pb = k * math.exp(-b * b / (2.0 * sigma * sigma))
    root2 = sigma * math.sqrt(2.0)
    mass = 0.5 * (math.erf(b / root2) - math.erf(a / root2))
    return sigma * sigma * (pa - pb), mass


def solve_codebook(d: int, bits: int) -> tuple[list[float], list[float]]:
    """Return (centroids[2**bits], boundaries[2**bits - 1]) as Python floats."""
    levels = 2 ** bits
    sigma = 1.0 / math.sqrt(d)
    lo, hi = -6.0 * sigma, 6.0 * sigma
    boundaries = [lo + (hi - lo) * i / levels for i in range(1, levels)]
    centroids = [0.0] * levels
    for _ in range(100):
        edges = [lo, *boundaries, hi]
        for i in range(levels):
            first, mass = _cell_moments(edges[i], edges[i + 1], sigma)
            centroids[i] = first / max(mass, 1e-30)
        # N(0, sigma^2) is symmetric, so the optimum is: remove the last-bit asymmetry the start grid
        # leaves, which makes the middle boundary exactly 0.0 (as in the reference's tables).
        centroids = [0.5 * (centroids[i] - centroids[levels - 1 - i]) for i in range(levels)]
        boundaries = [0.5 * (centroids[i] + centroids[i + 1]) for i in range(levels - 1)]
    return centroids, boundaries


def make_codebook(
    d: int = 128,
    bits: int = 3,
    device: Optional[torch.device] = None,
    dtype: torch.dtype = torch.float32,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Codebook as tensors: centroids [2**bits], boundaries [2**bits - 1]."""
    centroids, boundaries = solve_codebook(d, bits)
    return (
        torch.tensor(centroids, dtype=dtype, device=device),
        torch.tensor(boundaries, dtype=dtype, device=device),
    )
