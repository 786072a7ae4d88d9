"""PolarQuant configuration and the compress entry point.

Interface of turboquant/core/quantizer.py:26-201 in the reference.  The
arithmetic (rotate, norm of the rotated vector, divide by norm + 1e-8, count
of boundaries strictly below each coordinate, residual signs with zero -> +1)
runs in one CUDA kernel; this module only validates arguments and shapes the
result dictionary.  There is no CPU implementation here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class PolarQuantConfig:
    """Bit widths and layer gating for PolarQuant compression.

    `bits` is the key bit width (2, 3 or 4); `v_bits` the value bit width
    (None means "same as keys").  `use_qjl` adds one residual sign bit per key
    coordinate.  With `protect_boundary_layers`, the first and last
    `num_protected_layers` of `num_layers` layers are left uncompressed.
    """

    head_dim: int = 128
    bits: int = 3
    v_bits: Optional[int] = None
    use_qjl: bool = True
    protect_boundary_layers: bool = True
    num_protected_layers: int = 2
    num_layers: int = 0

    @property
    def k_bits(self) -> int:
        return self.bits

    @property
    def effective_v_bits(self) -> int:
        return self.bits if self.v_bits is None else self.v_bits

    @property
    def is_asymmetric(self) -> bool:
        return self.v_bits is not None and self.v_bits != self.bits

    @property
    def n_centroids(self) -> int:
        return 1 << self.bits

    def should_compress(self, layer_idx: int) -> bool:
        """False for protected boundary layers; True when the depth is unknown (num_layers == 0)."""
        if not self.protect_boundary_layers or self.num_layers == 0:
            return True
        first_ok = self.num_protected_layers
        last_ok = self.num_layers - self.num_protected_layers
        return first_ok <= layer_idx < last_ok

    def _compression_ratio_for_bits(self, bits: int) -> float:
        # Same accounting as the reference (quantizer.py:102-108): widths up to
        # 3 bits carry a sign bit per coordinate, every vector one fp16 norm.
        payload = bits * self.head_dim + 16
        if bits <= 3:
            payload += self.head_dim
        return (16 * self.head_dim) / payload

    @property
    def compression_ratio(self) -> float:
        return self._compression_ratio_for_bits(self.bits)

    @property
    def k_compression_ratio(self) -> float:
        return self._compression_ratio_for_bits(self.k_bits)

    @property
    def v_compression_ratio(self) -> float:
        return self._compression_ratio_for_bits(self.effective_v_bits)

    @property
    def combined_compression_ratio(self) -> float:
        return 2.0 / (1.0 / self.k_compression_ratio + 1.0 / self.v_compression_ratio)


def polarquant_compress(
    x: torch.Tensor,
    centroids: torch.Tensor,
    boundaries: torch.Tensor,
    config: PolarQuantConfig,
    rotation_matrix: Optional[torch.Tensor] = None,
) -> dict:
    """Compress vectors; same arguments and result keys as the reference.

    x [N, D] or [B, H, D] on a CUDA device, D = 128.  `rotation_matrix` must be
    None (x is already rotated) or the Walsh-Hadamard matrix of
    `make_wht_matrix(D)`; the kernel applies that rotation as a fast transform,
    it does not read the matrix.  Returns indices (int64), norms, k_mse_rot
    and, with `config.use_qjl`, signs (+-1) and rot_residual_norm, all fp32.
    """
    from turboquant.kernels import _native

    if not x.is_cuda:
        raise RuntimeError(
            "turboquant (B200 build) has no CPU path: polarquant_compress needs a CUDA tensor")
    orig_shape = x.shape
    if x.dim() == 3:
        x2 = x.reshape(-1, x.shape[-1])
    elif x.dim() == 2:
        x2 = x
    else:
        raise ValueError(f"x must be [N, D] or [B, H, D], got {tuple(x.shape)}")
    rotate = rotation_matrix is not None
    if rotate:
        _native.check_is_wht(rotation_matrix, x2.shape[-1])
    res = _native.polarquant(x2, centroids, boundaries, config.bits, config.use_qjl, rotate)
    if len(orig_shape) == 3:
        for key in ("k_mse_rot", "indices", "signs"):
            if key in res:
                res[key] = res[key].reshape(orig_shape)
    return res


def polarquant_decompress(compressed: dict, centroids: torch.Tensor, config: PolarQuantConfig) -> torch.Tensor:
    """MSE reconstruction in rotated space: the `k_mse_rot` entry, unchanged."""
    return compressed["k_mse_rot"]
