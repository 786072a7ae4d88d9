"""Per-layer TurboQuant state and layer gating for a paged-cache serving engine.

Mirrors the hook objects of the reference's turboquant/integration/vllm_backend.py
(TurboQuantFP8State :64-176, turbo4_fp8_compress_and_scatter :179-230,
TurboQuantFP8Config :237-289, get_tq_fp8_config :295-337) with one change of
substance: the cache holds TurboQuant's own packed pages (indices, norms, QJL
signs) instead of FP8 re-encodings of the dequantised values, so decode reads
118 / 132 bytes per token-head instead of 256 and runs in this package's CUDA
kernel rather than in AITER's FP8 paged attention.

Names of the reference (TurboQuantFP8Config, TurboQuantFP8State, get_tq_fp8_config)
are kept as aliases so existing call sites and tests import unchanged.
"""
from __future__ import annotations

from typing import Optional

import torch

from turboquant.core.codebook import make_codebook
from turboquant.core.rotation import make_wht_matrix
from turboquant.kernels.paged import CacheFormat, Codebooks


class TurboQuantState:
    """Codebooks and rotation helpers of one compressed layer.

    k_bits / v_bits may differ (asymmetric K/V); with equal widths K and V share
    the codebook tensors.  QJL signs are stored for 2- and 3-bit keys unless
    use_qjl says otherwise (turbo2/turbo3 vs turbo4).
    """

    def __init__(self, head_size: int, layer_idx: int, device, k_bits: int = 4, v_bits: Optional[int] = None,
                 use_qjl: Optional[bool] = None):
        if head_size != 128:
            raise ValueError("the B200 kernels are built for head_size 128")
        self.head_size = head_size
        self.layer_idx = layer_idx
        self.device = torch.device(device)
        self.k_bits = k_bits
        self.v_bits = k_bits if v_bits is None else v_bits
        self.use_qjl = (k_bits <= 3) if use_qjl is None else use_qjl
        self.format = CacheFormat(self.k_bits, self.v_bits, self.use_qjl)
        kc, kb = make_codebook(head_size, self.k_bits, device=self.device)
        self.k_centroids, self.k_boundaries = kc, kb
        if self.v_bits == self.k_bits:
            self.v_centroids, self.v_boundaries = kc, kb
        else:
            self.v_centroids, self.v_boundaries = make_codebook(head_size, self.v_bits, device=self.device)
        self.centroids, self.boundaries = self.k_centroids, self.k_boundaries   # names kept from the reference
        self._books: Optional[Codebooks] = None
        self._wht: Optional[torch.Tensor] = None

    @property
    def books(self) -> Codebooks:
        if self._books is None:
            self._books = Codebooks(self.format, self.device, (self.k_centroids, self.k_boundaries),
                                    (self.v_centroids, self.v_boundaries))
        return self._books

    @property
    def wht(self) -> torch.Tensor:
        """The rotation as an explicit matrix (the kernels never read it)."""
        if self._wht is None:
            self._wht = make_wht_matrix(self.head_size, self.device)
        return self._wht

    def rotate_query(self, q: torch.Tensor) -> torch.Tensor:
        """q [..., 128] -> q @ H, by the fast transform."""
        from turboquant.kernels import _native
        return _native.wht_rows(q)

    def rotate_output(self, out: torch.Tensor) -> torch.Tensor:
        """Attention output in rotated space -> original space (H is its own inverse)."""
        from turboquant.kernels import _native
        return _native.wht_rows(out)


def turbo_compress_and_scatter(key: torch.Tensor, value: torch.Tensor, kv_cache: torch.Tensor,
                               slot_mapping: torch.Tensor, state: TurboQuantState, block_size: int = 16) -> None:
    """Compress this step's K/V [T, Hkv, 128] and write them at their slots of the packed paged cache."""
    from turboquant.kernels.paged import compress_and_scatter
    compress_and_scatter(key, value, kv_cache, slot_mapping, state.books, block_size)


class TurboQuantConfig:
    """Which layers are compressed, and their per-layer state.

    With protect_boundary_layers, the first and last num_protected_layers of
    num_layers layers keep the engine's ordinary KV cache (get_state returns
    None for them); num_layers == 0 means "depth unknown": compress all.
    """

    def __init__(self, head_size: int = 128, num_layers: int = 0, protect_boundary_layers: bool = True,
                 num_protected_layers: int = 2, k_bits: int = 4, v_bits: Optional[int] = None,
                 use_qjl: Optional[bool] = None):
        self.head_size = head_size
        self.num_layers = num_layers
        self.protect_boundary_layers = protect_boundary_layers
        self.num_protected_layers = num_protected_layers
        self.k_bits = k_bits
        self.v_bits = v_bits
        self.use_qjl = use_qjl
        self.layer_states: dict[int, TurboQuantState] = {}

    def should_compress(self, layer_idx: int) -> bool:
        if not self.protect_boundary_layers or self.num_layers == 0:
            return True
        return self.num_protected_layers <= layer_idx < self.num_layers - self.num_protected_layers

    def get_state(self, layer_idx: int, device) -> Optional[TurboQuantState]:
        if not self.should_compress(layer_idx):
            return None
        st = self.layer_states.get(layer_idx)
        if st is None:
            st = TurboQuantState(self.head_size, layer_idx, device, k_bits=self.k_bits, v_bits=self.v_bits,
                                 use_qjl=self.use_qjl)
            self.layer_states[layer_idx] = st
        return st


_config: Optional[TurboQuantConfig] = None


def get_tq_config(head_size: int = 128, num_layers: int = 0, protect_boundary_layers: bool = True,
                  num_protected_layers: int = 2, k_bits: int = 4, v_bits: Optional[int] = None,
                  use_qjl: Optional[bool] = None) -> TurboQuantConfig:
    """Process-wide configuration, created on first call (later calls return the same object)."""
    global _config
    if _config is None:
        _config = TurboQuantConfig(head_size, num_layers, protect_boundary_layers, num_protected_layers, k_bits,
                                   v_bits, use_qjl)
    return _config


# names of the reference
TurboQuantFP8Config = TurboQuantConfig
TurboQuantFP8State = TurboQuantState
get_tq_fp8_config = get_tq_config
