"""ctypes binding of libtq_b200.so and its registration as torch custom ops.

The library is the only implementation: if it cannot be loaded, every entry
point raises.  Set TQ_B200_SO to load it from a non-default path (the role
TQ_FP4_PA_SO plays in the reference, turboquant/integration/tq_fp4_backend.py:59-76).

Ops registered (namespace `tq_b200`):
  compress_paged(key, value, cache, slot_mapping, kc, kb, vc, vb, block_size, k_bits, v_bits, use_qjl, prerotated)
  decode_paged(q_rot, q_proj, cache, block_tables, seq_lens, kc, vc, sm_scale, corr_scale, sparse_thresh,
               block_size, k_bits, v_bits, use_qjl, chunk_pages, io_flags, max_seq_len) -> out
  wht_rows(x, scale) -> x @ H * scale
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_DTYPES = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
_ERRORS = {-1: "bad argument", -2: "unsupported configuration", -3: "CUDA launch failed", -4: "workspace too small"}

STATUS_BAD_BLOCK = 1
STATUS_TIMEOUT = 2
STATUS_BAD_SLOT = 4
IO_ROTATE_Q = 0x100        # q is in original space: rotate it inside the decode kernel
IO_DEROTATE_OUT = 0x200    # write the decode output in original space
IO_TCGEN05 = 0x400         # tensor-memory variant of the decode kernel (2- / 3-bit codebooks, no Sparse-V)

_lib: Optional[ctypes.CDLL] = None


def library_path() -> str:
    env = os.environ.get("TQ_B200_SO")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libtq_b200.so")


def lib() -> ctypes.CDLL:
    """Load libtq_b200.so once; raise if it is missing (there is no fallback implementation)."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"libtq_b200.so not found at {path}: build it with `python turboquant-amd_b200/build.py` "
            "or point TQ_B200_SO at it. turboquant (B200 build) has no other implementation.")
    L = ctypes.CDLL(path)
    vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float
    L.tq_version.restype = i32
    L.tq_page_bytes.argtypes = [i32, i32, i32]
    L.tq_compress_paged.argtypes = [vp, vp, i32, i64, i64, i64, i64, vp, i64, i32, vp, vp, vp, vp, vp,
                                    i32, i32, i32, i32, i32, i32, vp, vp]
    L.tq_decode_auto_chunk_pages.argtypes = [i32, i32, i32, i32]
    L.tq_decode_workspace_bytes.argtypes = [i32, i32, i32, i32, i32]
    L.tq_decode_workspace_bytes.restype = i64
    L.tq_decode_paged.argtypes = [vp, vp, vp, i32, vp, i64, i32, vp, i64, vp, vp, vp, f32, f32, f32, vp, i64,
                                  vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp]
    L.tq_decode_paged_static.argtypes = [vp, vp, vp, i32, vp, i64, i32, vp, i64, vp, vp, vp, f32, f32, f32,
                                         vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, vp]
    L.tq_wht_rows.argtypes = [vp, vp, i32, i64, f32, vp]
    L.tq_compress_k.argtypes = [vp, i32, i64, vp, vp, i32, i32, i32, vp, vp, vp, vp, vp]
    L.tq_compress_v.argtypes = [vp, i32, i64, vp, i32, i32, vp, vp, vp]
    L.tq_polarquant_compress.argtypes = [vp, i32, i64, vp, vp, i32, i32, i32, vp, vp, vp, vp, vp, vp]
    L.tq_packed_attention_workspace_bytes.argtypes = [i32, i32]
    L.tq_packed_attention_workspace_bytes.restype = i64
    L.tq_packed_attention_auto_splits.argtypes = [i32, i32]
    L.tq_packed_attention.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, f32, i32, i32, i32, i32, vp, i64, vp, vp]
    for name in ("tq_page_bytes", "tq_compress_paged", "tq_decode_auto_chunk_pages", "tq_decode_paged",
                 "tq_decode_paged_static", "tq_wht_rows", "tq_compress_k", "tq_compress_v", "tq_polarquant_compress",
                 "tq_packed_attention_auto_splits", "tq_packed_attention"):
        getattr(L, name).restype = i32
    _lib = L
    return L


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed: {_ERRORS.get(rc, rc)} (status {rc})")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream(device: torch.device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("turboquant (B200 build) has no CPU path: all tensors must be CUDA tensors")
        if t is not None and t.device != dev:
            raise RuntimeError("all tensors must be on the same CUDA device")
    return dev


def _f32(t: torch.Tensor, device: torch.device) -> torch.Tensor:
    return t.to(device=device, dtype=torch.float32).contiguous()


def check_is_wht(matrix: torch.Tensor, d: int) -> None:
    """Raise unless `matrix` is the normalised Sylvester WHT matrix the fast transform implements."""
    if d != 128 or tuple(matrix.shape) != (128, 128):
        raise ValueError("only head_dim 128 is supported")
    # The verdict is remembered on the tensor object itself (and dropped if it is written to),
    # so a matrix is compared once, not on every call.
    if getattr(matrix, "_tq_is_wht_version", None) == matrix._version:
        return
    from turboquant.core.rotation import make_wht_matrix
    if not torch.allclose(matrix.detach().float().cpu(), make_wht_matrix(128), atol=1e-6, rtol=0):
        raise ValueError("rotation_matrix must be make_wht_matrix(128): the kernels apply that rotation as a "
                         "fast Walsh-Hadamard transform and cannot apply an arbitrary matrix")
    matrix._tq_is_wht_version = matrix._version

# ---- per-device scratch: status word, split-K workspaces --------------------------------------
_status: dict = {}
_workspaces: dict = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Device int32[1] the kernels OR their TQ_STATUS_* bits into."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    if device not in _status:
        _status[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status[device]


def read_status(device, reset: bool = True) -> int:
    """Synchronising read of the status word (for tests and debugging)."""
    w = status_word(device)
    val = int(w.item())
    if reset:
        w.zero_()
    return val


def workspace(device: torch.device, nbytes: int, tag: str = "decode") -> torch.Tensor:
    """A cached uint8 workspace of at least nbytes; grows geometrically, never shrinks."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (device, tag)
    cur = _workspaces.get(key)
    if cur is None or cur.numel() < nbytes:
        cur = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = cur
    return cur


# ---- thin checked wrappers -----------------------------------------------------------------
def page_bytes(k_bits: int, v_bits: int, use_qjl: bool) -> int:
    rc = lib().tq_page_bytes(k_bits, v_bits, int(use_qjl))
    if rc < 0:
        _check(rc, "tq_page_bytes")
    return rc


COMPRESS_TCGEN05 = 2       # flag in tq_compress_paged's `prerotated` argument: tensor-memory rotation kernel


def _compress_paged_impl(key, value, cache, slot_mapping, kc, kb, vc, vb, block_size, k_bits, v_bits, use_qjl,
                         prerotated, tcgen05: bool = False) -> None:
    dev = _require_cuda(key, value, cache, slot_mapping, kc, kb, vc, vb)
    if key.dim() != 3 or key.shape[-1] != 128 or value.shape != key.shape:
        raise ValueError("key/value must be [tokens, kv_heads, 128]")
    if key.dtype not in _DTYPES or value.dtype != key.dtype:
        raise ValueError("key/value must share a dtype of fp16, bf16 or fp32")
    if key.stride(-1) != 1 or value.stride(-1) != 1:
        raise ValueError("the head dimension must be contiguous")
    if cache.dtype != torch.uint8 or cache.dim() != 3 or not cache.is_contiguous():
        raise ValueError("cache must be a contiguous uint8 [num_blocks, kv_heads, bytes] tensor")
    T, H, _ = key.shape
    sub = block_size // 16
    if block_size % 16 or cache.shape[1] != H or cache.shape[2] != sub * page_bytes(k_bits, v_bits, use_qjl):
        raise ValueError("cache shape does not match (kv_heads, block_size, format): the last dimension must be "
                         f"block_size/16 * page_bytes = {sub * page_bytes(k_bits, v_bits, use_qjl)}")
    if slot_mapping.dtype != torch.int64 or slot_mapping.numel() < T or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be contiguous int64 with at least one entry per token")
    for name, t, n in (("k_centroids", kc, 1 << k_bits), ("k_boundaries", kb, (1 << k_bits) - 1),
                       ("v_boundaries", vb, (1 << v_bits) - 1)):
        if t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous fp32 with {n} entries")
    with torch.cuda.device(dev):
        rc = lib().tq_compress_paged(
            _ptr(key), _ptr(value), _DTYPES[key.dtype], key.stride(0), key.stride(1), value.stride(0), value.stride(1),
            _ptr(cache), cache.shape[0], block_size, _ptr(slot_mapping), _ptr(kc), _ptr(kb), _ptr(vc), _ptr(vb),
            T, H, k_bits, v_bits, int(use_qjl), int(bool(prerotated)) | (COMPRESS_TCGEN05 if tcgen05 else 0),
            _ptr(status_word(dev)), _stream(dev))
    _check(rc, "tq_compress_paged")


def decode_chunk_pages(num_seqs: int, num_kv_heads: int, num_q_heads: int, max_pages: int) -> int:
    return lib().tq_decode_auto_chunk_pages(num_seqs, num_kv_heads, num_q_heads, max(max_pages, 1))


def _decode_paged_impl(out, q_rot, q_proj, cache, block_tables, seq_lens, kc, vc, sm_scale, corr_scale,
                       sparse_thresh, block_size, k_bits, v_bits, use_qjl, chunk_pages, skip_stats=None,
                       io_flags: int = 0, max_seq_len: int = 0, static_scratch: bool = False) -> None:
    """Checked call of tq_decode_paged (or, with static_scratch, of tq_decode_paged_static, which keeps the
    split-K partials in the library's fixed device array and allocates nothing).

    max_seq_len > 0 is the longest sequence of this step as the host knows it: grid, chunk size and workspace are
    then sized for it instead of for the width of the block table (an engine hands over a table as wide as its
    maximum model length).  Lengths beyond it are cut by the kernel and flagged STATUS_BAD_BLOCK."""
    dev = _require_cuda(out, q_rot, cache, block_tables, seq_lens, kc, vc)
    if q_rot.dim() != 3 or q_rot.shape[-1] != 128 or not q_rot.is_contiguous():
        raise ValueError("q must be contiguous [num_seqs, q_heads, 128]")
    if q_rot.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("q must be fp16 or bf16")
    if out.shape != q_rot.shape or out.dtype != q_rot.dtype or not out.is_contiguous():
        raise ValueError("out must match q in shape and dtype and be contiguous")
    if q_proj is not None and (q_proj.shape != q_rot.shape or q_proj.dtype != q_rot.dtype or not q_proj.is_contiguous()):
        raise ValueError("q_proj must match q in shape and dtype and be contiguous")
    if cache.dtype != torch.uint8 or cache.dim() != 3 or not cache.is_contiguous():
        raise ValueError("cache must be a contiguous uint8 [num_blocks, kv_heads, bytes] tensor")
    ns, Hq, _ = q_rot.shape
    nb, Hkv, row = cache.shape
    sub = block_size // 16
    # The kernel's idea of the block size must be the cache's (the mismatch behind the reference's
    # intermittent Sparse-V fault, docs/MI355X_BLOCKSIZE_FIX.md:18-21 of the reference).
    if block_size % 16 or row != sub * page_bytes(k_bits, v_bits, use_qjl):
        raise ValueError(f"cache row of {row} bytes does not match block_size {block_size} and the format "
                         f"({sub * page_bytes(k_bits, v_bits, use_qjl)} expected)")
    if Hq % Hkv:
        raise ValueError("q heads must be a multiple of kv heads")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or block_tables.stride(1) != 1:
        raise ValueError("block_tables must be int32 [num_seqs, max_blocks] with contiguous rows")
    if seq_lens.dtype != torch.int32 or not seq_lens.is_contiguous() or seq_lens.numel() < ns:
        raise ValueError("seq_lens must be contiguous int32 [num_seqs]")
    if block_tables.shape[0] < ns:
        raise ValueError("block_tables has fewer rows than sequences")
    for name, t, n in (("k_centroids", kc, 1 << k_bits), ("v_centroids", vc, 1 << v_bits)):
        if t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous fp32 with {n} entries")
    max_pages = block_tables.shape[1] * sub
    if max_seq_len > 0:
        max_pages = max(1, min(max_pages, (int(max_seq_len) + 15) // 16))
    L = lib()
    if chunk_pages <= 0:
        chunk_pages = L.tq_decode_auto_chunk_pages(ns, Hkv, Hq, max_pages)
    common_tail = (_ptr(status_word(dev)), _ptr(skip_stats), ns, Hq, Hkv, max_pages, k_bits, v_bits, int(use_qjl),
                   chunk_pages, _stream(dev))
    head = (_ptr(out), _ptr(q_rot), _ptr(q_proj), _DTYPES[q_rot.dtype] | int(io_flags), _ptr(cache), nb, block_size,
            _ptr(block_tables), block_tables.stride(0), _ptr(seq_lens), _ptr(kc), _ptr(vc),
            float(sm_scale), float(corr_scale), float(sparse_thresh))
    with torch.cuda.device(dev):
        if static_scratch:
            rc = L.tq_decode_paged_static(*head, *common_tail)
        else:
            need = L.tq_decode_workspace_bytes(ns, Hq, Hkv, max_pages, chunk_pages)
            ws = workspace(dev, need)
            rc = L.tq_decode_paged(*head, _ptr(ws), ws.numel(), *common_tail)
    _check(rc, "tq_decode_paged_static" if static_scratch else "tq_decode_paged")


def wht_rows(x: torch.Tensor, scale: float = 1.0, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [..., 128] -> scale * (x @ H) with the fast transform; same dtype."""
    dev = _require_cuda(x)
    if x.shape[-1] != 128 or x.dtype not in _DTYPES:
        raise ValueError("x must be [..., 128] in fp16, bf16 or fp32")
    x = x.contiguous()
    if out is None:
        out = torch.empty_like(x)
    with torch.cuda.device(dev):
        rc = lib().tq_wht_rows(_ptr(x), _ptr(out), _DTYPES[x.dtype], x.numel() // 128, float(scale), _stream(dev))
    _check(rc, "tq_wht_rows")
    return out


def polarquant(x: torch.Tensor, centroids, boundaries, bits: int, use_qjl: bool, rotate: bool) -> dict:
    dev = _require_cuda(x)
    if x.shape[-1] != 128:
        raise ValueError("only head_dim 128 is supported")
    if x.dtype not in _DTYPES:
        x = x.float()
    x = x.contiguous()
    n = x.shape[0]
    c, b = _f32(centroids, dev), _f32(boundaries, dev)
    if c.numel() != 1 << bits or b.numel() != (1 << bits) - 1:
        raise ValueError("codebook size does not match config.bits")
    res = {
        "indices": torch.empty(n, 128, dtype=torch.int64, device=dev),
        "norms": torch.empty(n, dtype=torch.float32, device=dev),
        "k_mse_rot": torch.empty(n, 128, dtype=torch.float32, device=dev),
    }
    if use_qjl:
        res["signs"] = torch.empty(n, 128, dtype=torch.float32, device=dev)
        res["rot_residual_norm"] = torch.empty(n, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = lib().tq_polarquant_compress(
            _ptr(x), _DTYPES[x.dtype], n, _ptr(c), _ptr(b), bits, int(use_qjl), int(not rotate),
            _ptr(res["indices"]), _ptr(res["norms"]), _ptr(res["k_mse_rot"]), _ptr(res.get("signs")),
            _ptr(res.get("rot_residual_norm")), _stream(dev))
    _check(rc, "tq_polarquant_compress")
    return res


# ---- torch custom ops --------------------------------------------------------------------------
@torch.library.custom_op("tq_b200::compress_paged", mutates_args=("cache",))
def compress_paged_op(key: torch.Tensor, value: torch.Tensor, cache: torch.Tensor, slot_mapping: torch.Tensor,
                      kc: torch.Tensor, kb: torch.Tensor, vc: torch.Tensor, vb: torch.Tensor, block_size: int,
                      k_bits: int, v_bits: int, use_qjl: bool, prerotated: bool) -> None:
    _compress_paged_impl(key, value, cache, slot_mapping, kc, kb, vc, vb, block_size, k_bits, v_bits, use_qjl,
                         prerotated)


@compress_paged_op.register_fake
def _(key, value, cache, slot_mapping, kc, kb, vc, vb, block_size, k_bits, v_bits, use_qjl, prerotated) -> None:
    return None


@torch.library.custom_op("tq_b200::decode_paged", mutates_args=())
def decode_paged_op(q_rot: torch.Tensor, q_proj: Optional[torch.Tensor], cache: torch.Tensor,
                    block_tables: torch.Tensor, seq_lens: torch.Tensor, kc: torch.Tensor, vc: torch.Tensor,
                    sm_scale: float, corr_scale: float, sparse_thresh: float, block_size: int, k_bits: int,
                    v_bits: int, use_qjl: bool, chunk_pages: int, io_flags: int = 0,
                    max_seq_len: int = 0) -> torch.Tensor:
    out = torch.empty_like(q_rot)
    _decode_paged_impl(out, q_rot, q_proj, cache, block_tables, seq_lens, kc, vc, sm_scale, corr_scale,
                       sparse_thresh, block_size, k_bits, v_bits, use_qjl, chunk_pages, io_flags=io_flags,
                       max_seq_len=max_seq_len)
    return out


@decode_paged_op.register_fake
def _(q_rot, q_proj, cache, block_tables, seq_lens, kc, vc, sm_scale, corr_scale, sparse_thresh, block_size,
      k_bits, v_bits, use_qjl, chunk_pages, io_flags=0, max_seq_len=0):
    return torch.empty_like(q_rot)


@torch.library.custom_op("tq_b200::wht_rows", mutates_args=())
def wht_rows_op(x: torch.Tensor, scale: float) -> torch.Tensor:
    return wht_rows(x, scale)


@wht_rows_op.register_fake
def _(x, scale):
    return torch.empty_like(x)
