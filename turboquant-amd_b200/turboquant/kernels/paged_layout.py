"""Byte layout of one 16-token page of the paged TurboQuant cache, and pure-torch pack/unpack.

The decode kernel feeds tensor-core fragments straight from the packed bits, so
the physical order of bits inside a page follows the fragment ownership of
`mma.m16n8k16`, not dimension order.  This module is the single written
definition of that order (the CUDA kernels implement the same formulas) and
provides slow, exact packers/unpackers used for inspection and tests; it is
not on the hot path.

Cache tensor: uint8 [num_blocks, num_kv_heads, block_size // 16 * page_bytes].
A block of 32 tokens is two consecutive 16-token pages.

Page = K part, then V part (both multiples of 16 bytes):

K part
  token t in 0..15 owns a record of RK = 16 * (k_bits + qjl) bytes at t * RK,
  made of 4 sub-records (one per dim quarter q = d >> 5), each k_bits index
  words followed by one sign word when QJL is on.  Inside a quarter, dim
  d = 32 q + 4 c + e (c in 0..7, e in 0..3):
    4-bit: word c >> 1, bits (c & 1) * 16 + 4 e + [0..3]
    3-bit: c < 6 : word c >> 1, bits (c & 1) * 16 + 4 e + [0..2]
           c >= 6: bit b of the index sits in word b at (c - 6) * 16 + 4 e + 3
                   (the spare top bit of each nibble)
    2-bit: word c >> 2, bits (c & 1) * 16 + 4 e + ((c >> 1) & 1) * 2 + [0..1]
    sign : sign word, bit 4 c + e (= d & 31); 1 means residual >= 0
  then fp16 norms at 16 * RK in the order slot(t) = (t & 7) * 2 + (t >> 3),
  and, with QJL, fp16 residual norms in the same order.

V part
  dim d = 16 g + 4 u + e (g in 0..7, u in 0..3, e in 0..3); tokens are paired,
  p = t >> 1, and each 32-bit word holds the same 16-bit field of both tokens
  (token parity selects the half).  Word j of (p, g) is at ((j * 8 + p) * 8 + g) * 4:
    4-bit: j = u, bits 4 e + [0..3]
    3-bit: u < 3 : j = u, bits 4 e + [0..2];  u == 3: bit b in word b at 4 e + 3
    2-bit: j = u >> 1, bits 4 e + (u & 1) * 2 + [0..1]
  then fp16 norms in slot(t) order.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache

import torch

PAGE_TOKENS = 16
HEAD_DIM = 128


@dataclass(frozen=True)
class PageLayout:
    k_bits: int
    v_bits: int
    use_qjl: bool

    @property
    def k_record_bytes(self) -> int:
        return 16 * (self.k_bits + int(self.use_qjl))

    @property
    def k_norm_offset(self) -> int:
        return PAGE_TOKENS * self.k_record_bytes

    @property
    def k_rnorm_offset(self) -> int:
        return self.k_norm_offset + 32

    @property
    def k_part_bytes(self) -> int:
        return self.k_norm_offset + 32 + (32 if self.use_qjl else 0)

    @property
    def v_offset(self) -> int:
        return self.k_part_bytes

    @property
    def v_norm_offset(self) -> int:
        return self.v_offset + 256 * self.v_bits

    @property
    def v_part_bytes(self) -> int:
        return 256 * self.v_bits + 32

    @property
    def page_bytes(self) -> int:
        return self.k_part_bytes + self.v_part_bytes

    @property
    def bytes_per_token(self) -> float:
        return self.page_bytes / PAGE_TOKENS


def page_bytes(k_bits: int, v_bits: int, use_qjl: bool) -> int:
    return PageLayout(k_bits, v_bits, use_qjl).page_bytes


def cache_shape(num_blocks: int, block_size: int, num_kv_heads: int, k_bits: int, v_bits: int,
                use_qjl: bool) -> tuple[int, int, int]:
    if block_size % PAGE_TOKENS:
        raise ValueError("block_size must be a multiple of 16")
    return (num_blocks, num_kv_heads, block_size // PAGE_TOKENS * page_bytes(k_bits, v_bits, use_qjl))


def _norm_slot(t: int) -> int:
    return (t & 7) * 2 + (t >> 3)


def _k_bit_position(bits: int, rk: int, t: int, d: int, b: int) -> int:
    q, c, e = d >> 5, (d >> 2) & 7, d & 3
    base = (t * rk + q * (rk // 4)) * 8
    if bits == 4:
        return base + (c >> 1) * 32 + (c & 1) * 16 + 4 * e + b
    if bits == 3:
        if c < 6:
            return base + (c >> 1) * 32 + (c & 1) * 16 + 4 * e + b
        return base + b * 32 + (c - 6) * 16 + 4 * e + 3
    if bits == 2:
        return base + (c >> 2) * 32 + (c & 1) * 16 + 4 * e + ((c >> 1) & 1) * 2 + b
    raise ValueError(bits)


def _k_sign_position(bits: int, rk: int, t: int, d: int) -> int:
    q, c, e = d >> 5, (d >> 2) & 7, d & 3
    base = (t * rk + q * (rk // 4)) * 8 + bits * 32
    return base + 4 * c + e


def _v_bit_position(bits: int, voff: int, t: int, d: int, b: int) -> int:
    g, u, e = d >> 4, (d >> 2) & 3, d & 3
    p, h = t >> 1, t & 1
    if bits == 4:
        j, pos = u, 4 * e + b
    elif bits == 3:
        j, pos = (u, 4 * e + b) if u < 3 else (b, 4 * e + 3)
    elif bits == 2:
        j, pos = u >> 1, 4 * e + (u & 1) * 2 + b
    else:
        raise ValueError(bits)
    return (voff + ((j * 8 + p) * 8 + g) * 4) * 8 + h * 16 + pos


@lru_cache(maxsize=None)
def _tables(k_bits: int, v_bits: int, use_qjl: bool):
    """Absolute bit positions inside a page for every logical bit (int64 tensors on CPU)."""
    L = PageLayout(k_bits, v_bits, use_qjl)
    rk = L.k_record_bytes
    kpos = torch.empty(PAGE_TOKENS, HEAD_DIM, k_bits, dtype=torch.int64)
    vpos = torch.empty(PAGE_TOKENS, HEAD_DIM, v_bits, dtype=torch.int64)
    spos = torch.empty(PAGE_TOKENS, HEAD_DIM, dtype=torch.int64)
    for t in range(PAGE_TOKENS):
        for d in range(HEAD_DIM):
            for b in range(k_bits):
                kpos[t, d, b] = _k_bit_position(k_bits, rk, t, d, b)
            for b in range(v_bits):
                vpos[t, d, b] = _v_bit_position(v_bits, L.v_offset, t, d, b)
            spos[t, d] = _k_sign_position(k_bits, rk, t, d)
    slots = torch.tensor([_norm_slot(t) for t in range(PAGE_TOKENS)], dtype=torch.int64)
    return L, kpos, vpos, spos, slots


def _bits_of(pages: torch.Tensor) -> torch.Tensor:
    """uint8 [..., B] -> 0/1 uint8 [..., 8 B], little-endian bit order."""
    shifts = torch.arange(8, device=pages.device, dtype=torch.uint8)
    return ((pages.unsqueeze(-1) >> shifts) & 1).reshape(*pages.shape[:-1], pages.shape[-1] * 8)


def _bytes_of(bits: torch.Tensor) -> torch.Tensor:
    w = (1 << torch.arange(8, device=bits.device, dtype=torch.int32))
    b = bits.reshape(*bits.shape[:-1], bits.shape[-1] // 8, 8).to(torch.int32)
    return (b * w).sum(-1).to(torch.uint8)


def unpack_pages(pages: torch.Tensor, k_bits: int, v_bits: int, use_qjl: bool) -> dict:
    """pages uint8 [..., page_bytes] -> logical fields.

    Returns k_idx, v_idx uint8 [..., 16, 128]; k_norm, v_norm fp16 [..., 16];
    with QJL also k_signs uint8 (1 = +) [..., 16, 128] and k_rnorm fp16 [..., 16].
    """
    L, kpos, vpos, spos, slots = _tables(k_bits, v_bits, use_qjl)
    if pages.shape[-1] != L.page_bytes:
        raise ValueError(f"last dim {pages.shape[-1]} != page_bytes {L.page_bytes}")
    dev = pages.device
    bits = _bits_of(pages)
    lead = pages.shape[:-1]

    def gather_idx(pos, nb):
        g = bits[..., pos.to(dev).reshape(-1)].reshape(*lead, PAGE_TOKENS, HEAD_DIM, nb).to(torch.int32)
        return (g << torch.arange(nb, device=dev, dtype=torch.int32)).sum(-1).to(torch.uint8)

    def norms(off):
        raw = pages[..., off:off + 32].contiguous().view(torch.float16)
        return raw[..., slots.to(dev)]

    out = {
        "k_idx": gather_idx(kpos, k_bits),
        "v_idx": gather_idx(vpos, v_bits),
        "k_norm": norms(L.k_norm_offset),
        "v_norm": norms(L.v_norm_offset),
    }
    if use_qjl:
        out["k_signs"] = bits[..., spos.to(dev).reshape(-1)].reshape(*lead, PAGE_TOKENS, HEAD_DIM)
        out["k_rnorm"] = norms(L.k_rnorm_offset)
    return out


def pack_pages(k_idx, k_norm, v_idx, v_norm, k_bits: int, v_bits: int, use_qjl: bool,
               k_signs=None, k_rnorm=None) -> torch.Tensor:
    """Inverse of `unpack_pages`; fields shaped [..., 16, 128] / [..., 16] -> uint8 [..., page_bytes]."""
    L, kpos, vpos, spos, slots = _tables(k_bits, v_bits, use_qjl)
    dev = k_idx.device
    lead = k_idx.shape[:-2]
    bits = torch.zeros(*lead, L.page_bytes * 8, dtype=torch.uint8, device=dev)

    def scatter_idx(idx, pos, nb):
        b = ((idx.to(torch.int32).unsqueeze(-1) >> torch.arange(nb, device=dev, dtype=torch.int32)) & 1)
        bits[..., pos.to(dev).reshape(-1)] = b.reshape(*lead, -1).to(torch.uint8)

    scatter_idx(k_idx, kpos, k_bits)
    scatter_idx(v_idx, vpos, v_bits)
    if use_qjl:
        bits[..., spos.to(dev).reshape(-1)] = k_signs.reshape(*lead, -1).to(torch.uint8)
    pages = _bytes_of(bits)

    def put_norms(off, vals):
        ordered = torch.empty(*lead, PAGE_TOKENS, dtype=torch.float16, device=dev)
        ordered[..., slots.to(dev)] = vals.to(torch.float16)
        pages[..., off:off + 32] = ordered.contiguous().view(torch.uint8)

    put_norms(L.k_norm_offset, k_norm)
    put_norms(L.v_norm_offset, v_norm)
    if use_qjl:
        put_norms(L.k_rnorm_offset, k_rnorm)
    return pages


def unpack_cache(cache: torch.Tensor, block_size: int, k_bits: int, v_bits: int, use_qjl: bool) -> dict:
    """cache uint8 [num_blocks, Hkv, sub * page_bytes] -> fields shaped [num_blocks, block_size, Hkv, ...]."""
    nb, hkv, _ = cache.shape
    sub = block_size // PAGE_TOKENS
    f = unpack_pages(cache.reshape(nb, hkv, sub, -1), k_bits, v_bits, use_qjl)
    out = {}
    for key, val in f.items():
        if val.dim() == 5:    # [nb, hkv, sub, 16, 128]
            out[key] = val.permute(0, 2, 3, 1, 4).reshape(nb, block_size, hkv, HEAD_DIM)
        else:                 # [nb, hkv, sub, 16]
            out[key] = val.permute(0, 2, 3, 1).reshape(nb, block_size, hkv)
    return out


def pack_cache(fields: dict, block_size: int, k_bits: int, v_bits: int, use_qjl: bool) -> torch.Tensor:
    """Inverse of `unpack_cache`."""
    k_idx = fields["k_idx"]
    nb, _, hkv, _ = k_idx.shape
    sub = block_size // PAGE_TOKENS

    def big(x):
        return x.reshape(nb, sub, PAGE_TOKENS, hkv, HEAD_DIM).permute(0, 3, 1, 2, 4)

    def small(x):
        return x.reshape(nb, sub, PAGE_TOKENS, hkv).permute(0, 3, 1, 2)

    pages = pack_pages(big(fields["k_idx"]), small(fields["k_norm"]), big(fields["v_idx"]), small(fields["v_norm"]),
                       k_bits, v_bits, use_qjl,
                       big(fields["k_signs"]) if use_qjl else None,
                       small(fields["k_rnorm"]) if use_qjl else None)
    return pages.reshape(nb, hkv, -1).contiguous()
