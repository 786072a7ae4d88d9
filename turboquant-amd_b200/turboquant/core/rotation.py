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


# ---- weight fusion: fold the rotation into projection weights at model-load time ------------------
# Same three entry points as the reference (turboquant/core/rotation.py:47-140).  With the rotation
# folded into the projections, Q, K and V leave the QKV projection already rotated and the output
# projection undoes the rotation, so serving needs neither the query rotation nor the output
# de-rotation step.  H is symmetric, so "H^T @ W" per head is one batched matmul over all heads.

def _rotate_head_rows(weight: torch.Tensor, n_heads: int, head_size: int, H: torch.Tensor) -> torch.Tensor:
    """weight [n_heads * head_size, hidden]: left-multiply every head's [head_size, hidden] block by H^T."""
    blocks = weight.reshape(n_heads, head_size, -1)
    return torch.matmul(H.T.to(weight.dtype), blocks).reshape(n_heads * head_size, -1)


def fuse_rotation_into_qkv_proj(qkv_weight: torch.Tensor, num_heads: int, num_kv_heads: int,
                                head_size: int) -> torch.Tensor:
    """Packed [Q | K | V] projection weight [(nh + 2 nkv) * D, hidden] -> the same with every head rotated."""
    H = make_wht_matrix(head_size, device=qkv_weight.device)
    total = num_heads + 2 * num_kv_heads
    if qkv_weight.shape[0] != total * head_size:
        raise ValueError("qkv_weight rows do not match (num_heads + 2 * num_kv_heads) * head_size")
    return _rotate_head_rows(qkv_weight, total, head_size, H)


def fuse_rotation_into_o_proj(o_weight: torch.Tensor, num_heads: int, head_size: int) -> torch.Tensor:
    """Output projection [hidden, nh * D]: right-multiply every head's column block by H^T (= H)."""
    H = make_wht_matrix(head_size, device=o_weight.device).to(o_weight.dtype)
    hidden = o_weight.shape[0]
    blocks = o_weight.reshape(hidden, num_heads, head_size)
    return torch.matmul(blocks, H.T).reshape(hidden, num_heads * head_size)


def apply_weight_fusion(model_state_dict: dict, num_heads: int, num_kv_heads: int, head_size: int) -> dict:
    """Fuse every `qkv_proj.weight` and `o_proj.weight` entry of a state dict in place; returns the dict."""
    for key in list(model_state_dict.keys()):
        if "qkv_proj.weight" in key:
            model_state_dict[key] = fuse_rotation_into_qkv_proj(model_state_dict[key], num_heads, num_kv_heads, head_size)
        elif "o_proj.weight" in key:
            model_state_dict[key] = fuse_rotation_into_o_proj(model_state_dict[key], num_heads, head_size)
    return model_state_dict
