"""Walsh-Hadamard rotation matrix (turboquant/core/rotation.py:28-44 of the reference).

The kernels never multiply by this matrix: compression and query rotation use
an in-register fast WHT.  The matrix is kept for callers that want the
explicit operator (x_rot = x @ H, H @ H = I) and as the definition the fast
transform must agree with: every entry is +-2**-3.5 with the Sylvester sign
pattern sign(H[i, j]) = (-1)**popcount(i & j).
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def make_wht_matrix(d: int, device: Optional[torch.device] = None) -> torch.Tensor:
    """Normalised Sylvester Hadamard matrix [d, d] in fp32 (d a power of two)."""
    H = torch.ones(1, 1, device=device)
    while H.shape[0] < d:
        top = torch.cat([H, H], dim=1)
        bottom = torch.cat([H, -H], dim=1)
        H = torch.cat([top, bottom], dim=0) / math.sqrt(2)
    return H[:d, :d]
