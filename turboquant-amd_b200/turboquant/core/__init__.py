"""Codebook, rotation and quantizer entry points (turboquant/core/__init__.py:3-14 of the reference)."""

from turboquant.core.codebook import solve_codebook, make_codebook
from turboquant.core.rotation import make_wht_matrix
from turboquant.core.quantizer import PolarQuantConfig, polarquant_compress, polarquant_decompress

__all__ = [
    "solve_codebook",
    "make_codebook",
    "make_wht_matrix",
    "PolarQuantConfig",
    "polarquant_compress",
    "polarquant_decompress",
]
