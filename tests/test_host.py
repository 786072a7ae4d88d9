"""Host-side logic of the product package: config, codebook, rotation matrix, pack helpers, page layout, C ABI.
No GPU is used; compute entry points are only checked to exist and to refuse CPU tensors."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from turboquant.core import (PolarQuantConfig, make_codebook, make_wht_matrix, polarquant_compress,
                             polarquant_decompress, solve_codebook)
from turboquant.kernels import _native, packed_compress, paged_layout
from turboquant.kernels.paged import CacheFormat

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ---- PolarQuantConfig (turboquant/core/quantizer.py:26-108) ----------------------------------
def test_config_rows_match_reference(golden):
    for row in golden["config_rows"]:
        bits, vb = int(row[0]), int(row[1])
        cfg = PolarQuantConfig(head_dim=128, bits=bits, v_bits=None if vb < 0 else vb)
        got = [cfg.k_bits, cfg.effective_v_bits, int(cfg.is_asymmetric), cfg.n_centroids, cfg.compression_ratio,
               cfg.k_compression_ratio, cfg.v_compression_ratio, cfg.combined_compression_ratio]
        np.testing.assert_allclose(got, row[2:], rtol=1e-12)


def test_config_should_compress(golden):
    cfg = PolarQuantConfig(num_layers=40, protect_boundary_layers=True, num_protected_layers=2)
    assert [cfg.should_compress(i) for i in range(40)] == list(golden["config_should_compress_40"])
    cfg = PolarQuantConfig(num_layers=0)
    assert [cfg.should_compress(i) for i in range(8)] == list(golden["config_should_compress_0"])
    cfg = PolarQuantConfig(num_layers=40, protect_boundary_layers=False)
    assert all(cfg.should_compress(i) for i in range(40))


def test_config_defaults():
    cfg = PolarQuantConfig()
    assert (cfg.head_dim, cfg.bits, cfg.v_bits, cfg.use_qjl) == (128, 3, None, True)
    assert (cfg.protect_boundary_layers, cfg.num_protected_layers, cfg.num_layers) == (True, 2, 0)


# ---- codebook / rotation (stay Python) ------------------------------------------------------
@pytest.mark.parametrize("d", [64, 128, 256])
@pytest.mark.parametrize("bits", [1, 2, 3, 4])
def test_codebook_fp32_identical_to_reference(golden, d, bits):
    c, b = make_codebook(d, bits)
    assert torch.equal(c, torch.from_numpy(golden[f"codebook_d{d}_b{bits}_c"]).float())
    assert torch.equal(b, torch.from_numpy(golden[f"codebook_d{d}_b{bits}_b"]).float())
    cl, bl = solve_codebook(d, bits)
    assert len(cl) == 2 ** bits and len(bl) == 2 ** bits - 1
    assert all(x < y for x, y in zip(cl, cl[1:])) and all(cl[i] < bl[i] < cl[i + 1] for i in range(len(bl)))


def test_codebook_dtype_and_symmetry():
    c, b = make_codebook(128, 3, dtype=torch.float16)
    assert c.dtype == torch.float16 and b.dtype == torch.float16 and c.shape == (8,) and b.shape == (7,)
    c, _ = solve_codebook(128, 3)
    assert all(abs(c[i] + c[7 - i]) < 1e-6 for i in range(8))
    c64, _ = solve_codebook(64, 2)
    c256, _ = solve_codebook(256, 2)
    assert 1.8 < abs(c64[-1] / c256[-1]) < 2.2


@pytest.mark.parametrize("d", [8, 128])
def test_wht_matrix_identical_to_reference(golden, d):
    assert torch.equal(make_wht_matrix(d), torch.from_numpy(golden[f"wht_d{d}"]))


@pytest.mark.parametrize("d", [2, 16, 128])
def test_wht_orthogonal_self_inverse(d):
    H = make_wht_matrix(d)
    eye = torch.eye(d)
    assert (H @ H.T - eye).abs().max() < 1e-5 and (H @ H - eye).abs().max() < 1e-5


# ---- pack helpers (turboquant/kernels/packed_compress.py:145-216) ---------------------------
def test_unpack_and_permute_match_reference(golden):
    pk = torch.from_numpy(golden["pack_idx_bytes"])
    sg = torch.from_numpy(golden["pack_sign_bytes"])
    assert torch.equal(packed_compress.unpack_2bit(pk, 128), torch.from_numpy(golden["unpack_2bit"]))
    assert torch.equal(packed_compress.unpack_1bit(sg, 128), torch.from_numpy(golden["unpack_1bit"]))
    assert torch.equal(packed_compress.permute_signs_for_chunked(sg), torch.from_numpy(golden["permute_signs"]))


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_unpackers_invert_oracle_packers(bits):
    from oracle import tq_oracle as O
    idx = np.random.default_rng(1).integers(0, 1 << bits, (19, 128))
    got = packed_compress.unpack_indices(torch.from_numpy(O.pack_indices(idx, bits)), bits)
    assert np.array_equal(got.numpy(), idx)


# ---- page layout ---------------------------------------------------------------------------
@pytest.mark.parametrize("kb,vb,qjl,per_token", [(2, 2, True, 86), (3, 3, True, 118), (4, 4, False, 132),
                                                 (4, 2, False, 100), (3, 3, False, 100), (4, 4, True, 150)])
def test_page_sizes(kb, vb, qjl, per_token):
    L = paged_layout.PageLayout(kb, vb, qjl)
    assert L.page_bytes == 16 * per_token
    assert L.k_part_bytes % 16 == 0 and L.v_part_bytes % 16 == 0      # bulk-copy granularity
    assert _native.page_bytes(kb, vb, qjl) == L.page_bytes            # the library agrees with the Python definition
    assert CacheFormat(kb, vb, qjl).cache_shape(7, 32, 3) == (7, 3, 2 * L.page_bytes)


@pytest.mark.parametrize("kb,vb,qjl", [(2, 2, True), (3, 3, True), (4, 4, False), (4, 2, True), (2, 4, False), (3, 2, True)])
def test_layout_is_a_bijection(kb, vb, qjl):
    L, kpos, vpos, spos, slots = paged_layout._tables(kb, vb, qjl)
    used = torch.cat([kpos.reshape(-1), vpos.reshape(-1)] + ([spos.reshape(-1)] if qjl else []))
    assert used.unique().numel() == used.numel()                      # no two logical bits share a position
    norm_bytes = 32 * (2 + int(qjl)) * 8
    assert used.numel() + norm_bytes == L.page_bytes * 8              # and no bit of the page is wasted
    assert used.min() >= 0 and used.max() < L.page_bytes * 8
    assert sorted(slots.tolist()) == list(range(16))


@pytest.mark.parametrize("kb,vb,qjl", [(2, 2, True), (3, 3, True), (4, 4, False), (4, 3, True)])
def test_pack_unpack_cache_roundtrip(kb, vb, qjl):
    g = torch.Generator().manual_seed(kb * 10 + vb)
    nb, bs, hkv = 3, 32, 2
    f = {"k_idx": torch.randint(0, 1 << kb, (nb, bs, hkv, 128), generator=g, dtype=torch.uint8),
         "v_idx": torch.randint(0, 1 << vb, (nb, bs, hkv, 128), generator=g, dtype=torch.uint8),
         "k_norm": torch.rand(nb, bs, hkv, generator=g).half(), "v_norm": torch.rand(nb, bs, hkv, generator=g).half()}
    if qjl:
        f["k_signs"] = torch.randint(0, 2, (nb, bs, hkv, 128), generator=g, dtype=torch.uint8)
        f["k_rnorm"] = torch.rand(nb, bs, hkv, generator=g).half()
    cache = paged_layout.pack_cache(f, bs, kb, vb, qjl)
    assert cache.shape == CacheFormat(kb, vb, qjl).cache_shape(nb, bs, hkv) and cache.dtype == torch.uint8
    back = paged_layout.unpack_cache(cache, bs, kb, vb, qjl)
    for key, val in f.items():
        assert torch.equal(back[key], val), key


# ---- C ABI -----------------------------------------------------------------------------------
def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared_symbols()
    assert len(names) >= 12
    L = ctypes.CDLL(_native.library_path())
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/tq_b200.h but not exported"


def test_host_only_entry_points():
    L = _native.lib()
    assert L.tq_version() >= 1
    assert L.tq_page_bytes(5, 3, 1) == -2 and L.tq_page_bytes(3, 1, 0) == -2
    cp = L.tq_decode_auto_chunk_pages(64, 8, 64, 512)
    assert cp == 256
    assert L.tq_decode_workspace_bytes(64, 64, 8, 512, cp) == 64 * 8 * ((512 + cp - 1) // cp) * 8 * 130 * 4
    assert L.tq_decode_auto_chunk_pages(1, 8, 32, 1) == 1
    assert L.tq_decode_auto_chunk_pages(64, 1, 8, 512) == 57          # one KV head per GPU: 9 chunks fill the 592 CTA slots
    assert L.tq_decode_auto_chunk_pages(1, 8, 32, 256) == 16         # a single sequence: small chunks fill the GPU
    assert L.tq_decode_auto_chunk_pages(256, 8, 32, 4096) == 256     # skewed long sequences: capped
    assert L.tq_packed_attention_auto_splits(64, 32768) >= 1
    assert L.tq_packed_attention_workspace_bytes(8, 16) == 8 * 16 * 130 * 4


def test_launchers_validate_arguments_without_touching_a_gpu():
    L = _native.lib()
    null = ctypes.c_void_p(0)
    assert L.tq_compress_k(null, 0, 4, null, null, 3, 0, 1, null, null, null, null, null) == -1
    assert L.tq_compress_v(null, 0, 0, null, 3, 0, null, null, null) == 0        # zero rows: nothing to do
    assert L.tq_wht_rows(null, null, 0, 8, 1.0, null) == -1
    assert L.tq_decode_paged(null, null, null, 0, null, 1, 16, null, 1, null, null, null, 1.0, 1.0, 0.0, null, 0,
                             null, null, 0, 8, 8, 1, 3, 3, 1, 0, null) == 0          # zero sequences
    assert L.tq_decode_paged(null, null, null, 0, null, 1, 16, null, 1, null, null, null, 1.0, 1.0, 0.0, null, 0,
                             null, null, 2, 8, 8, 1, 3, 3, 1, 0, null) == -1


def test_head_counts_that_form_no_query_group_are_refused_on_the_host():
    """Fewer query heads than KV heads (or a non-multiple) used to make the chunk-size search loop for ever."""
    L = _native.lib()
    null = ctypes.c_void_p(0)
    assert L.tq_decode_auto_chunk_pages(4, 8, 4, 100) == -1
    assert L.tq_decode_auto_chunk_pages(4, 8, 12, 100) == -1
    assert L.tq_decode_workspace_bytes(4, 4, 8, 100, 0) == -1
    assert L.tq_decode_workspace_bytes(4, 12, 8, 100, 16) == -1
    assert L.tq_decode_paged_static(null, null, null, 0, null, 1, 16, null, 1, null, null, null, 1.0, 1.0, 0.0,
                                    null, null, 2, 4, 8, 100, 3, 3, 1, 0, null) == -1
    assert L.tq_decode_paged_static(null, null, null, 0, null, 1, 16, null, 1, null, null, null, 1.0, 1.0, 0.0,
                                    null, null, 0, 4, 8, 100, 3, 3, 1, 0, null) == 0      # zero sequences


def test_no_cpu_fallback():
    x = torch.randn(4, 128)
    c, b = make_codebook(128, 3)
    with pytest.raises(RuntimeError, match="no CPU path"):
        polarquant_compress(x, c, b, PolarQuantConfig(bits=3), None)
    with pytest.raises(RuntimeError, match="no CPU path"):
        packed_compress.compress_v(x, None, c, b)
    assert torch.equal(polarquant_decompress({"k_mse_rot": x}, c, PolarQuantConfig()), x)


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setenv("TQ_B200_SO", "/nonexistent/libtq_b200.so")
    monkeypatch.setattr(_native, "_lib", None)
    with pytest.raises(RuntimeError, match="not found"):
        _native.lib()


# ---- weight fusion (turboquant/core/rotation.py:47-140; the reference's tests/test_rotation.py:73-126) ----
def test_weight_fusion_equals_explicit_rotation():
    from turboquant.core.rotation import apply_weight_fusion, fuse_rotation_into_o_proj, fuse_rotation_into_qkv_proj
    nh, nkv, D, hid = 4, 2, 128, 512
    torch.manual_seed(42)
    H = make_wht_matrix(D)
    qkv = torch.randn((nh + 2 * nkv) * D, hid)
    x = torch.randn(2, hid)
    out = x @ qkv.T
    fused = x @ fuse_rotation_into_qkv_proj(qkv.clone(), nh, nkv, D).T
    for lo, n in ((0, nh), (nh * D, nkv), ((nh + nkv) * D, nkv)):
        a = out[:, lo:lo + n * D].view(2, n, D) @ H
        assert (a - fused[:, lo:lo + n * D].view(2, n, D)).abs().max() < 1e-3
    o_w = torch.randn(hid, nh * D)
    attn_rot = torch.randn(2, nh, D)
    want = (attn_rot @ H).reshape(2, -1) @ o_w.T
    got = attn_rot.reshape(2, -1) @ fuse_rotation_into_o_proj(o_w.clone(), nh, D).T
    assert torch.nn.functional.cosine_similarity(want.reshape(1, -1), got.reshape(1, -1)).item() > 0.9999
    sd = {"layers.0.qkv_proj.weight": qkv.clone(), "layers.0.o_proj.weight": o_w.clone(), "other": torch.ones(2)}
    sd2 = apply_weight_fusion(sd, nh, nkv, D)
    assert sd2 is sd and torch.equal(sd["other"], torch.ones(2))
    assert torch.allclose(sd["layers.0.qkv_proj.weight"], fuse_rotation_into_qkv_proj(qkv, nh, nkv, D))
