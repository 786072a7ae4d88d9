"""vLLM attention backend over the packed TurboQuant paged cache (B200).

Shape of the reference's only complete vLLM backend,
turboquant/integration/tq_fp4_backend.py (TurboQuantFP4Backend :650-733,
TurboQuantFP4Impl :389-648): the cache update is separate from forward
(`forward_includes_kv_cache_update = False`), decode runs the native kernel,
prefill runs ordinary attention on the raw K/V of the step.  Differences:
  * registered through vLLM's extension point
    `register_backend(AttentionBackendEnum.CUSTOM, ...)` instead of patching
    the backend selector (tq_fp4_backend.py:805-819);
  * the cache tensor is uint8 [num_blocks, num_kv_heads, block_size/16 * page_bytes]
    (TurboQuant packed pages), not FP4 nibbles plus side buffers of scales.

The classes are built on first use so that importing this module does not import vLLM.
Status: written against vLLM 0.22's v1 interface.  `do_kv_cache_update` and `forward` are exercised
on a GPU with hand-built layer and metadata objects (decode, fresh prefill and steps that mix both);
they have not been run inside a vLLM engine.  A step may mix decode rows (one new token over cached
context) with fresh prefills; a prefill chunk that continues cached context (an "extend") raises.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from turboquant.integration.vllm_backend import TurboQuantConfig, get_tq_config, turbo_compress_and_scatter
from turboquant.kernels.paged import CacheFormat, paged_decode_attention

BACKEND_PATH = "turboquant.integration.tq_b200_backend.TurboQuantB200Backend"
_FORMATS = {"turbo2": CacheFormat(2, 2, True), "turbo3": CacheFormat(3, 3, True), "turbo4": CacheFormat(4, 4, False)}


def cache_format_from_env() -> CacheFormat:
    """TQ_B200_FORMAT = turbo2 | turbo3 | turbo4 (default turbo4, the reference's serving default)."""
    return _FORMATS[os.environ.get("TQ_B200_FORMAT", "turbo4")]


def kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                   fmt: Optional[CacheFormat] = None) -> tuple[int, int, int]:
    """uint8 cache shape for a format (the role of get_kv_cache_shape, tq_fp4_backend.py:699-722)."""
    if head_size != 128:
        raise ValueError("head_size must be 128")
    if block_size not in (16, 32):
        raise ValueError("block_size must be 16 or 32")
    return (fmt or cache_format_from_env()).cache_shape(num_blocks, block_size, num_kv_heads)


def split_batch(query_start_loc: list, seq_lens: list) -> tuple[list, list]:
    """Sort the requests of one step into decode rows and fresh prefills.

    query_start_loc [n + 1] and seq_lens [n] are host lists.  Request i owns query tokens
    query_start_loc[i] .. query_start_loc[i + 1]; it is a decode when it has one query token (its sequence
    length counts that token), a fresh prefill when its query tokens are its whole sequence.  Returns
    (decodes, prefills): decodes = [(request, token_row)], prefills = [(request, first_row, end_row)].
    Anything else continues cached context with more than one token and raises NotImplementedError
    (the reference serves those through its extend branch, tq_fp4_backend.py:555-601).  Requests without
    query tokens (padding) are dropped.
    """
    decodes, prefills = [], []
    for i in range(len(query_start_loc) - 1):
        a, b = int(query_start_loc[i]), int(query_start_loc[i + 1])
        n, total = b - a, int(seq_lens[i])
        if n <= 0:
            continue
        if n == total:
            prefills.append((i, a, b))       # includes a one-token sequence: attention over itself
        elif n == 1:
            decodes.append((i, a))
        else:
            raise NotImplementedError("chunked prefill over cached context is not supported")
    return decodes, prefills


_classes = None


def _build_classes():
    global _classes
    if _classes is not None:
        return _classes
    from vllm.v1.attention.backend import AttentionBackend, AttentionImpl, AttentionType
    from vllm.v1.attention.backends.flash_attn import FlashAttentionMetadataBuilder

    class TurboQuantB200Impl(AttentionImpl):
        def __init__(self, num_heads: int, head_size: int, scale: float, num_kv_heads: int,
                     alibi_slopes: Optional[list] = None, sliding_window: Optional[int] = None,
                     kv_cache_dtype: str = "auto", logits_soft_cap: Optional[float] = None,
                     attn_type: str = AttentionType.DECODER, kv_sharing_target_layer_name: Optional[str] = None,
                     **_ignored) -> None:
            if alibi_slopes is not None or sliding_window is not None or logits_soft_cap is not None:
                raise NotImplementedError("TurboQuant B200 backend: no ALiBi, sliding window or soft cap")
            if attn_type != AttentionType.DECODER:
                raise NotImplementedError("TurboQuant B200 backend: decoder self-attention only")
            self.num_heads, self.head_size, self.scale, self.num_kv_heads = num_heads, head_size, float(scale), num_kv_heads
            self.kv_cache_dtype = "turboquant"
            self.format = cache_format_from_env()
            self.config: TurboQuantConfig = get_tq_config(head_size, k_bits=self.format.k_bits,
                                                          v_bits=self.format.v_bits, use_qjl=self.format.use_qjl)
            self._layer_idx: Optional[int] = None

        def _state(self, layer, device):
            if self._layer_idx is None:
                name = getattr(layer, "layer_name", "") or ""
                digits = [int(t) for t in name.replace(".", " ").split() if t.isdigit()]
                self._layer_idx = digits[0] if digits else 0
            state = self.config.get_state(self._layer_idx, device)
            if state is None:
                raise NotImplementedError(
                    "protected boundary layers keep the engine's own KV cache; give them another backend")
            return state

        def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
            """Compress the step's K/V into the packed cache (tq_fp4_backend.py:456-484)."""
            state = self._state(layer, key.device)
            block_size = kv_cache.shape[2] // self.format.page_bytes * 16
            turbo_compress_and_scatter(key, value, kv_cache, slot_mapping[:key.shape[0]], state, block_size)

        def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None, output_scale=None,
                    output_block_scale=None):
            assert output is not None, "accept_output_buffer: the engine provides the output tensor"
            if output_scale is not None or output_block_scale is not None:
                raise NotImplementedError("fused output quantisation is not supported")
            if attn_metadata is None:
                return output.fill_(0)
            n = attn_metadata.num_actual_tokens
            q = query[:n].view(n, self.num_heads, self.head_size)
            out = output[:n].view(n, self.num_heads, self.head_size)
            max_seq_len = int(getattr(attn_metadata, "max_seq_len", 0) or 0)
            if attn_metadata.max_query_len == 1:
                # decode: one token per sequence, attention over the packed cache (tq_fp4_backend.py:604-641)
                state = self._state(layer, q.device)
                block_size = kv_cache.shape[2] // self.format.page_bytes * 16
                res = paged_decode_attention(q.contiguous(), kv_cache, attn_metadata.block_table[:n],
                                             attn_metadata.seq_lens[:n], state.books, block_size,
                                             sm_scale=self.scale, rotate_q=True, derotate_out=True,
                                             max_seq_len=max_seq_len)
                out.copy_(res)
                return output
            # A step with prefills: sort the requests on the host (the reference's metadata carries
            # num_decodes / num_prefills for this, tq_fp4_backend.py:517-530).
            decodes, prefills = split_batch(attn_metadata.query_start_loc.tolist(), attn_metadata.seq_lens.tolist())
            if decodes:
                state = self._state(layer, q.device)
                block_size = kv_cache.shape[2] // self.format.page_bytes * 16
                req = torch.tensor([r for r, _ in decodes], dtype=torch.long, device=q.device)
                rows = torch.tensor([t for _, t in decodes], dtype=torch.long, device=q.device)
                res = paged_decode_attention(q[rows].contiguous(), kv_cache, attn_metadata.block_table[req].contiguous(),
                                             attn_metadata.seq_lens[req].contiguous(), state.books, block_size,
                                             sm_scale=self.scale, rotate_q=True, derotate_out=True,
                                             max_seq_len=max_seq_len)
                out[rows] = res
            # prefill on the raw K/V of this step (tq_fp4_backend.py:532-553)
            g = self.num_heads // self.num_kv_heads
            for _, a, b in prefills:
                qs = q[a:b].transpose(0, 1).unsqueeze(0)
                ks = key[a:b].view(b - a, self.num_kv_heads, self.head_size).repeat_interleave(g, 1).transpose(0, 1).unsqueeze(0)
                vs = value[a:b].view(b - a, self.num_kv_heads, self.head_size).repeat_interleave(g, 1).transpose(0, 1).unsqueeze(0)
                o = torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True, scale=self.scale)
                out[a:b].copy_(o.squeeze(0).transpose(0, 1))
            return output

        def fused_rope_kvcache_supported(self):
            return False

    class TurboQuantB200Backend(AttentionBackend):
        accept_output_buffer: bool = True
        forward_includes_kv_cache_update: bool = False
        supported_dtypes = [torch.float16, torch.bfloat16]
        supported_kv_cache_dtypes = ["auto"]

        @staticmethod
        def get_name() -> str:
            return "CUSTOM"

        @staticmethod
        def get_impl_cls():
            return TurboQuantB200Impl

        @staticmethod
        def get_builder_cls():
            return FlashAttentionMetadataBuilder

        @staticmethod
        def get_supported_kernel_block_sizes():
            return [16, 32]

        @classmethod
        def get_supported_head_sizes(cls):
            return [128]

        @staticmethod
        def get_kv_cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
                               cache_dtype_str: str = "auto"):
            return kv_cache_shape(num_blocks, block_size, num_kv_heads, head_size)

    _classes = (TurboQuantB200Backend, TurboQuantB200Impl)
    return _classes


def __getattr__(name: str):
    if name == "TurboQuantB200Backend":
        return _build_classes()[0]
    if name == "TurboQuantB200Impl":
        return _build_classes()[1]
    raise AttributeError(name)


def register() -> None:
    """Make `--attention-backend CUSTOM` (AttentionBackendEnum.CUSTOM) resolve to this backend."""
    from vllm.v1.attention.backends.registry import AttentionBackendEnum, register_backend
    register_backend(AttentionBackendEnum.CUSTOM, BACKEND_PATH)
