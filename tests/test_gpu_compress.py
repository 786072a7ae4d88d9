"""CUDA compression kernels against the CPU oracle and the reference's golden vectors (through the C ABI)."""
import numpy as np
import pytest
import torch

from oracle import tq_oracle as O
from turboquant.core import PolarQuantConfig, make_codebook, make_wht_matrix, polarquant_compress
from turboquant.kernels import _native, packed_compress, paged_layout
from turboquant.kernels.paged import CacheFormat, Codebooks, allocate_cache, compress_and_scatter

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(n, seed=0, outliers=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, 128, generator=g)
    if outliers:
        x[:, [3, 40, 77, 120]] *= 10.0
    return x


def _half_ulp_close(got_h: torch.Tensor, want_f32: np.ndarray, max_ulp=1):
    """fp16 values within max_ulp units in the last place of the fp16 rounding of want."""
    want_h = torch.from_numpy(want_f32.astype(np.float16))
    a = got_h.cpu().view(torch.int16).to(torch.int32)
    b = want_h.view(torch.int16).to(torch.int32)
    return (a - b).abs().max().item() <= max_ulp


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_polarquant_prerotated_bit_exact_vs_golden(golden, bits):
    """Identical fp32 rotated inputs -> indices and signs equal to the reference's own outputs."""
    x = torch.from_numpy(golden["pq_x"]).to(DEV)
    c, b = make_codebook(128, bits)
    r = polarquant_compress(x, c.to(DEV), b.to(DEV), PolarQuantConfig(bits=bits, use_qjl=True), None)
    p = f"pq_b{bits}_pre_"
    idx = r["indices"].cpu().numpy()
    ref_idx = golden[p + "indices"].astype(np.int64)
    signs = (r["signs"].cpu().numpy() > 0)
    ref_signs = np.unpackbits(golden[p + "signs"], axis=1, bitorder="little").astype(bool)
    assert r["indices"].dtype == torch.int64
    assert (idx != ref_idx).mean() <= 1e-4 and np.abs(idx - ref_idx).max() <= 1
    assert (signs != ref_signs).mean() <= 1e-4
    assert set(np.unique(r["signs"].cpu().numpy())) <= {-1.0, 1.0}
    np.testing.assert_allclose(r["norms"].cpu().numpy(), golden[p + "norms"], rtol=3e-7)
    np.testing.assert_allclose(r["rot_residual_norm"].cpu().numpy(), golden[p + "rnorm"], rtol=2e-5, atol=1e-7)
    np.testing.assert_allclose(r["k_mse_rot"][:8].cpu().numpy(), golden[p + "k_mse_rot"], rtol=3e-7, atol=1e-9)
    # the all-zero row: norm 0, ties at boundary 0 go to the lower centroid, every sign +
    assert r["norms"][5] == 0 and (r["signs"][5] == 1).all()
    assert (r["indices"][5] == (1 << bits) // 2 - 1).all()


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_polarquant_rotated_vs_golden(golden, bits):
    """In-kernel fast WHT instead of x @ H: at most 1e-4 of coordinates move, and only by one centroid."""
    x = torch.from_numpy(golden["pq_x"]).to(DEV)
    c, b = make_codebook(128, bits)
    H = make_wht_matrix(128).to(DEV)
    r = polarquant_compress(x, c.to(DEV), b.to(DEV), PolarQuantConfig(bits=bits), H)
    p = f"pq_b{bits}_rot_"
    idx = r["indices"].cpu().numpy()
    ref_idx = golden[p + "indices"].astype(np.int64)
    assert (idx != ref_idx).mean() <= 1e-4 and np.abs(idx - ref_idx).max() <= 1
    ref_signs = np.unpackbits(golden[p + "signs"], axis=1, bitorder="little").astype(bool)
    assert ((r["signs"].cpu().numpy() > 0) != ref_signs).mean() <= 1e-4
    np.testing.assert_allclose(r["norms"].cpu().numpy(), golden[p + "norms"], rtol=2e-6)


def test_polarquant_dict_contract():
    c, b = make_codebook(128, 3)
    x = _inputs(32).to(DEV)
    r = polarquant_compress(x, c.to(DEV), b.to(DEV), PolarQuantConfig(bits=3, use_qjl=False), make_wht_matrix(128).to(DEV))
    assert sorted(r) == ["indices", "k_mse_rot", "norms"]
    x3 = _inputs(32).reshape(4, 8, 128).to(DEV)
    r3 = polarquant_compress(x3, c.to(DEV), b.to(DEV), PolarQuantConfig(bits=3), make_wht_matrix(128).to(DEV))
    assert r3["indices"].shape == (4, 8, 128) and r3["k_mse_rot"].shape == (4, 8, 128) and r3["signs"].shape == (4, 8, 128)
    assert r3["norms"].shape == (32,) and (r3["norms"] >= 0).all()
    assert 0 <= r3["indices"].min() and r3["indices"].max() < 8
    cos = torch.nn.functional.cosine_similarity(x3.reshape(-1, 128) @ make_wht_matrix(128).to(DEV), r3["k_mse_rot"].reshape(-1, 128), dim=-1)
    assert cos.mean() > 0.95
    with pytest.raises(ValueError):
        polarquant_compress(x, c.to(DEV), b.to(DEV), PolarQuantConfig(bits=3), torch.eye(128, device=DEV))


@pytest.mark.parametrize("n", [4099, 33189])   # generic kernel / persistent table-driven kernel (more than 32768 rows); both ragged
@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_compress_k_v_contiguous_vs_oracle(bits, dtype, n):
    x = _inputs(n, seed=bits).to(dtype)
    c, b = make_codebook(128, bits)
    H = make_wht_matrix(128)
    xin = x.float().numpy()                    # the oracle sees the same rounded inputs
    for rotate in (False, True):
        rot = O.make_wht_matrix(128) if rotate else None
        o_idx, o_sg, o_rn, o_n = O.compress_k_packed(xin, c.numpy(), b.numpy(), bits, rot, permuted=False)
        o_sgp = O.permute_signs_for_chunked(o_sg)
        PiT = H.to(DEV) if rotate else None
        k_idx, k_sg, k_rn, k_n = packed_compress.compress_k(x.to(DEV), PiT, None, c.to(DEV), b.to(DEV))
        _, k_sgp, _, _ = packed_compress.compress_k_permuted(x.to(DEV), PiT, None, c.to(DEV), b.to(DEV))
        assert k_idx.dtype == torch.uint8 and k_idx.shape == (n, 16 * bits) and k_sg.shape == (n, 16)
        assert k_rn.dtype == torch.float16 and k_n.dtype == torch.float16
        got = packed_compress.unpack_indices(k_idx.cpu(), bits).numpy()
        want = O.unpack_indices(o_idx, bits)
        mism = (got != want)
        assert mism.mean() <= (0.0 if not rotate else 1e-4) + 1e-4 and np.abs(got.astype(int) - want).max() <= 1
        if not rotate:
            assert mism.sum() <= 2                                   # exact ties only
            assert (np.unpackbits(k_sg.cpu().numpy(), axis=1) != np.unpackbits(o_sg, axis=1)).mean() <= 1e-5
            assert (np.unpackbits(k_sgp.cpu().numpy(), axis=1) != np.unpackbits(o_sgp, axis=1)).mean() <= 1e-5
        else:
            assert (np.unpackbits(k_sg.cpu().numpy(), axis=1) != np.unpackbits(o_sg, axis=1)).mean() <= 1e-4
        # permuted output is the reference's permutation of the sequential one
        assert torch.equal(packed_compress.permute_signs_for_chunked(k_sg.cpu()), k_sgp.cpu())
        assert _half_ulp_close(k_n, o_n.astype(np.float32)) and _half_ulp_close(k_rn, o_rn.astype(np.float32))
        v_idx, v_n = packed_compress.compress_v(x.to(DEV), PiT, c.to(DEV), b.to(DEV))
        ov_idx, ov_n = O.compress_v_packed(xin, c.numpy(), b.numpy(), bits, rot)
        gotv = packed_compress.unpack_indices(v_idx.cpu(), bits).numpy()
        assert (gotv != O.unpack_indices(ov_idx, bits)).mean() <= 1e-4
        assert torch.equal(v_idx, k_idx) and torch.equal(v_n, k_n)   # V is the K computation without the residual


@pytest.mark.parametrize("rotate", [False, True])
def test_compress_contiguous_large_tight_codebook_and_nonfinite_rows(rotate):
    """More than 32768 rows take the persistent kernel.  A codebook with two boundaries closer than 1/64 makes it fall
    back to the binary search inside the kernel; a NaN / Inf row spoils only itself."""
    n = 33189
    x = _inputs(n, seed=5).half()
    x[17, 5] = float("nan")
    x[n - 1, 100] = float("inf")
    rot = O.make_wht_matrix(128) if rotate else None
    PiT = make_wht_matrix(128).to(DEV) if rotate else None
    for tight in (False, True):
        c, b = make_codebook(128, 3)
        if tight:
            b = b.clone()
            b[3] = b[2] + 1e-3
        k_idx, k_sg, k_rn, k_n = packed_compress.compress_k(x.to(DEV), PiT, None, c.to(DEV), b.to(DEV))
        good = np.ones(n, dtype=bool)
        good[[17, n - 1]] = False
        o_idx, o_sg, o_rn, o_n = O.compress_k_packed(x.float().numpy()[good], c.numpy(), b.numpy(), 3, rot, permuted=False)
        got = packed_compress.unpack_indices(k_idx.cpu(), 3).numpy()[good]
        want = O.unpack_indices(o_idx, 3)
        assert (got != want).mean() <= (1e-4 if rotate else 1e-6) and np.abs(got.astype(int) - want).max() <= 1
        assert (np.unpackbits(k_sg.cpu().numpy()[good], axis=1) != np.unpackbits(o_sg, axis=1)).mean() <= (1e-4 if rotate else 1e-5)
        assert _half_ulp_close(k_n.cpu()[torch.from_numpy(good)], o_n.astype(np.float32))
        assert not torch.isfinite(k_n[17].float()) and not torch.isfinite(k_n[n - 1].float())


def test_compress_k_v_general_rotation_and_projection_matrices():
    """The reference's own demo (packed_compress.py:247-275) passes a QR-orthogonal Pi and PiST = Pi S^T with a
    Gaussian S.  Such matrices take the composed path (matrix products around the same quantizer kernels): indices
    within the 1e-4 allowance of a differently rounded rotation, projected signs equal except where the projection is
    within rounding of zero."""
    n = 3001
    x = _inputs(n, seed=11)
    c, b = make_codebook(128, 2)
    g = torch.Generator().manual_seed(3)
    Pi, _ = torch.linalg.qr(torch.randn(128, 128, generator=g))
    S = torch.randn(128, 128, generator=g)
    PiT, PiST = Pi.T.contiguous(), (Pi @ S.T).contiguous()
    for pit, pist in ((PiT, PiST), (PiT, None), (make_wht_matrix(128), PiST), (None, PiST)):
        rot = None if pit is None else pit.numpy()
        o_idx, o_sg, o_rn, o_n = O.compress_k_packed(x.numpy(), c.numpy(), b.numpy(), 2, rot, permuted=False,
                                                     sign_projection=None if pist is None else pist.numpy())
        k_idx, k_sg, k_rn, k_n = packed_compress.compress_k(x.to(DEV), None if pit is None else pit.to(DEV),
                                                            None if pist is None else pist.to(DEV), c.to(DEV), b.to(DEV))
        got = packed_compress.unpack_indices(k_idx.cpu(), 2).numpy()
        want = O.unpack_indices(o_idx, 2)
        assert (got != want).mean() <= 1e-4 and np.abs(got.astype(int) - want).max() <= 1
        assert (np.unpackbits(k_sg.cpu().numpy(), axis=1) != np.unpackbits(o_sg, axis=1)).mean() <= 2e-4
        assert _half_ulp_close(k_n, o_n.astype(np.float32)) and _half_ulp_close(k_rn, o_rn.astype(np.float32), max_ulp=2)
        _, k_sgp, _, _ = packed_compress.compress_k_permuted(x.to(DEV), None if pit is None else pit.to(DEV),
                                                            None if pist is None else pist.to(DEV), c.to(DEV), b.to(DEV))
        assert torch.equal(packed_compress.permute_signs_for_chunked(k_sg.cpu()), k_sgp.cpu())
    v_idx, v_n = packed_compress.compress_v(x.to(DEV), PiT.to(DEV), c.to(DEV), b.to(DEV))
    ov_idx, ov_n = O.compress_v_packed(x.numpy(), c.numpy(), b.numpy(), 2, PiT.numpy())
    assert (packed_compress.unpack_indices(v_idx.cpu(), 2).numpy() != O.unpack_indices(ov_idx, 2)).mean() <= 1e-4
    assert _half_ulp_close(v_n, ov_n.astype(np.float32))
    with pytest.raises(ValueError):
        packed_compress.compress_v(x.to(DEV), (2 * PiT).to(DEV), c.to(DEV), b.to(DEV))      # not orthogonal


def test_compress_empty_and_single():
    c, b = make_codebook(128, 3)
    e = torch.empty(0, 128, device=DEV)
    k_idx, k_sg, k_rn, k_n = packed_compress.compress_k(e, None, None, c.to(DEV), b.to(DEV))
    assert k_idx.shape == (0, 48) and k_n.shape == (0,)
    one = _inputs(1).to(DEV)
    k_idx, _, _, k_n = packed_compress.compress_k(one, None, None, c.to(DEV), b.to(DEV))
    r = O.polarquant_compress(one.cpu().numpy(), c.numpy(), b.numpy(), 3, True, None)
    assert np.array_equal(packed_compress.unpack_indices(k_idx.cpu(), 3).numpy(), r["indices"])


@pytest.mark.parametrize("fmt_name,block_size", [("turbo2", 16), ("turbo3", 16), ("turbo4", 16), ("turbo3", 32)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_compress_paged_fields_vs_oracle(fmt_name, block_size, dtype):
    fmt = CacheFormat.named(fmt_name)
    books = Codebooks(fmt, DEV)
    T, Hkv, nb = 150, 3, 16
    g = torch.Generator().manual_seed(7)
    key = torch.randn(T, Hkv, 128, generator=g)
    val = torch.randn(T, Hkv, 128, generator=g)
    key[..., [3, 40, 77, 120]] *= 10
    key, val = key.to(dtype), val.to(dtype)
    slots = torch.randperm(nb * block_size, generator=g)[:T]
    cache = allocate_cache(nb, block_size, Hkv, fmt, DEV)
    cache.fill_(0xA5)                                                 # stale bytes must be fully overwritten
    compress_and_scatter(key.to(DEV), val.to(DEV), cache, slots.to(DEV), books, block_size)
    assert _native.read_status(DEV) == 0
    f = paged_layout.unpack_cache(cache.cpu(), block_size, fmt.k_bits, fmt.v_bits, fmt.use_qjl)
    blk, off = slots // block_size, slots % block_size
    H = O.make_wht_matrix(128)
    ok = O.polarquant_compress(key.float().numpy().reshape(-1, 128), books.kc.cpu().numpy(), books.kb.cpu().numpy(),
                               fmt.k_bits, fmt.use_qjl, H)
    ov = O.polarquant_compress(val.float().numpy().reshape(-1, 128), books.vc.cpu().numpy(), books.vb.cpu().numpy(),
                               fmt.v_bits, False, H)
    got_k = f["k_idx"][blk, off].numpy().reshape(-1, 128)
    got_v = f["v_idx"][blk, off].numpy().reshape(-1, 128)
    assert (got_k != ok["indices"]).mean() <= 1e-4 and (got_v != ov["indices"]).mean() <= 1e-4
    assert _half_ulp_close(f["k_norm"][blk, off].reshape(-1), ok["norms"])
    assert _half_ulp_close(f["v_norm"][blk, off].reshape(-1), ov["norms"])
    if fmt.use_qjl:
        got_s = f["k_signs"][blk, off].numpy().reshape(-1, 128)
        assert (got_s != (ok["signs"] > 0)).mean() <= 1e-4
        assert _half_ulp_close(f["k_rnorm"][blk, off].reshape(-1), ok["rot_residual_norm"])
    # slots that were not written keep their old bytes
    untouched = torch.ones(nb * block_size, dtype=torch.bool)
    untouched[slots] = False
    raw = paged_layout.unpack_cache(torch.full_like(cache.cpu(), 0xA5), block_size, fmt.k_bits, fmt.v_bits, fmt.use_qjl)
    ub, uo = torch.nonzero(untouched).squeeze(1) // block_size, torch.nonzero(untouched).squeeze(1) % block_size
    assert torch.equal(f["k_idx"][ub, uo], raw["k_idx"][ub, uo]) and torch.equal(f["v_idx"][ub, uo], raw["v_idx"][ub, uo])


def test_compress_paged_prerotated_strided_and_bad_slots():
    fmt = CacheFormat.named("turbo3")
    books = Codebooks(fmt, DEV)
    T, Hkv, nb, bs = 20, 2, 4, 16
    g = torch.Generator().manual_seed(9)
    qkv = torch.randn(T, 3 * Hkv, 128, generator=g).half().to(DEV)      # K and V as strided views of one buffer
    key, val = qkv[:, Hkv:2 * Hkv], qkv[:, 2 * Hkv:]
    slots = torch.arange(T, dtype=torch.int64)
    slots[3] = -1                                                       # padding slot -> clamped to 0 (like the reference)
    slots[0] = 45                                                       # so slot 0 is written by token 3 only
    slots[7] = nb * bs + 3                                              # beyond the cache -> skipped and flagged
    cache = allocate_cache(nb, bs, Hkv, fmt, DEV)
    compress_and_scatter(key, val, cache, slots.to(DEV), books, bs, prerotated=True)
    assert _native.read_status(DEV) == _native.STATUS_BAD_SLOT
    f = paged_layout.unpack_cache(cache.cpu(), bs, 3, 3, True)
    ok = O.polarquant_compress(key.float().cpu().numpy().reshape(-1, 128), books.kc.cpu().numpy(),
                               books.kb.cpu().numpy(), 3, True, None)
    want = ok["indices"].reshape(T, Hkv, 128)
    assert np.array_equal(f["k_idx"][0, 0].numpy(), want[3])            # token 3 landed in slot 0
    assert np.array_equal(f["k_idx"][2, 13].numpy(), want[0])           # slot 45 = block 2, offset 13
    assert np.array_equal(f["k_idx"][0, 9].numpy(), want[9])
    assert (f["k_idx"][0, 7] == 0).all()                                # token 7 was skipped; slot 7 untouched (zeros)
    with pytest.raises(ValueError):
        compress_and_scatter(key, val, cache[:, :, :-16], slots.to(DEV), books, bs)


def test_wht_rows_matches_matrix():
    x = _inputs(257, seed=5)
    H = make_wht_matrix(128)
    for dtype, tol in ((torch.float32, 2e-5), (torch.float16, 4e-2), (torch.bfloat16, 3e-1)):
        xin = x.to(dtype)
        y = _native.wht_rows(xin.to(DEV), 0.5)
        assert y.dtype == dtype
        ref = (xin.float() @ H) * 0.5
        assert (y.float().cpu() - ref).abs().max() <= tol
    y = _native.wht_rows(_native.wht_rows(x.to(DEV)))                  # H is its own inverse
    assert (y.cpu() - x).abs().max() < 1e-4


def test_full_size_properties():
    """1M vectors: scale invariance of indices and signs, norm homogeneity, idempotent re-compression."""
    n = 1 << 20
    g = torch.Generator(device=DEV).manual_seed(11)
    x = torch.randn(n, 128, generator=g, device=DEV, dtype=torch.float16)
    c, b = make_codebook(128, 3)
    H = make_wht_matrix(128).to(DEV)
    i1, s1, rn1, n1 = packed_compress.compress_k(x, H, None, c.to(DEV), b.to(DEV))
    i2, s2, rn2, n2 = packed_compress.compress_k(x * 2, H, None, c.to(DEV), b.to(DEV))   # exact power-of-two scaling
    assert torch.equal(i1, i2) and torch.equal(s1, s2)
    assert torch.equal(n2.float(), (n1.float() * 2)) and torch.equal(rn2.float(), rn1.float() * 2)
    # index histogram is the Lloyd-Max cell mass of a Gaussian (all 8 cells used, symmetric)
    idx = packed_compress.unpack_indices(i1[:65536].cpu(), 3).long()
    hist = torch.bincount(idx.reshape(-1), minlength=8).float()
    hist /= hist.sum()
    assert (hist - hist.flip(0)).abs().max() < 2e-3 and hist.min() > 0.02
    # checksum of checksums is reproducible run to run
    assert torch.equal(i1.sum(dtype=torch.int64), packed_compress.compress_k(x, H, None, c.to(DEV), b.to(DEV))[0].sum(dtype=torch.int64))


def test_compress_paged_no_tokens_and_fp32_input():
    fmt = CacheFormat.named("turbo2")
    books = Codebooks(fmt, DEV)
    cache = allocate_cache(2, 16, 2, fmt, DEV)
    before = cache.clone()
    compress_and_scatter(torch.empty(0, 2, 128, device=DEV), torch.empty(0, 2, 128, device=DEV), cache,
                         torch.empty(0, dtype=torch.int64, device=DEV), books, 16)
    assert torch.equal(cache, before)
    g = torch.Generator().manual_seed(3)
    K = torch.randn(5, 2, 128, generator=g)
    V = torch.randn(5, 2, 128, generator=g)
    slots = torch.tensor([31, 0, 7, 16, 8])
    compress_and_scatter(K.to(DEV), V.to(DEV), cache, slots.to(DEV), books, 16)
    assert _native.read_status(DEV) == 0
    f = paged_layout.unpack_cache(cache.cpu(), 16, 2, 2, True)
    ok = O.polarquant_compress(K.numpy().reshape(-1, 128), books.kc.cpu().numpy(), books.kb.cpu().numpy(), 2, True,
                               O.make_wht_matrix(128))
    got = f["k_idx"][slots // 16, slots % 16].numpy().reshape(-1, 128)
    assert (got != ok["indices"]).mean() <= 1e-4


def test_compress_paged_tight_codebook_takes_generic_path():
    """Boundaries closer than the table's cell width: the kernel falls back to the binary search."""
    fmt = CacheFormat.named("turbo3")
    b = torch.tensor([-0.03, -0.02, -0.01, 0.0, 0.01, 0.02, 0.03])
    c = torch.tensor([-0.05, -0.025, -0.015, -0.005, 0.005, 0.015, 0.025, 0.05])
    books = Codebooks(fmt, DEV, k_codebook=(c, b), v_codebook=(c, b))
    T, Hkv, bs = 40, 2, 16
    g = torch.Generator().manual_seed(21)
    key = torch.randn(T, Hkv, 128, generator=g).half()
    val = torch.randn(T, Hkv, 128, generator=g).half()
    slots = torch.randperm(4 * bs, generator=g)[:T]
    for prerotated in (False, True):
        cache = allocate_cache(4, bs, Hkv, fmt, DEV)
        compress_and_scatter(key.to(DEV), val.to(DEV), cache, slots.to(DEV), books, bs, prerotated=prerotated)
        assert _native.read_status(DEV) == 0
        f = paged_layout.unpack_cache(cache.cpu(), bs, 3, 3, True)
        H = None if prerotated else O.make_wht_matrix(128)
        ok = O.polarquant_compress(key.float().numpy().reshape(-1, 128), c.numpy(), b.numpy(), 3, True, H)
        ov = O.polarquant_compress(val.float().numpy().reshape(-1, 128), c.numpy(), b.numpy(), 3, False, H)
        got_k = f["k_idx"][slots // bs, slots % bs].numpy().reshape(-1, 128)
        got_v = f["v_idx"][slots // bs, slots % bs].numpy().reshape(-1, 128)
        got_s = f["k_signs"][slots // bs, slots % bs].numpy().reshape(-1, 128)
        if prerotated:
            assert np.array_equal(got_k, ok["indices"]) and np.array_equal(got_v, ov["indices"])
            assert np.array_equal(got_s, ok["signs"] > 0)
        else:
            assert (got_k != ok["indices"]).mean() <= 1e-3 and (got_v != ov["indices"]).mean() <= 1e-3


@pytest.mark.parametrize("dtype,prerotated", [(torch.float16, False), (torch.bfloat16, False), (torch.float16, True),
                                              (torch.float32, False)])
def test_compress_paged_nonfinite_rows_do_not_disturb_others(dtype, prerotated):
    """A NaN or an infinity inside one vector only spoils that vector (its norm shows it)."""
    fmt = CacheFormat.named("turbo3")
    books = Codebooks(fmt, DEV)
    T, Hkv, bs = 24, 2, 16
    g = torch.Generator().manual_seed(23)
    key = torch.randn(T, Hkv, 128, generator=g).to(dtype)
    val = torch.randn(T, Hkv, 128, generator=g).to(dtype)
    slots = torch.arange(T, dtype=torch.int64)
    clean = allocate_cache(2, bs, Hkv, fmt, DEV)
    compress_and_scatter(key.to(DEV), val.to(DEV), clean, slots.to(DEV), books, bs, prerotated=prerotated)
    bad_k, bad_v = key.clone(), val.clone()
    bad_k[3, 1, 17] = float("nan")
    bad_k[5, 0, 100] = float("inf")
    bad_v[7, 1, 0] = float("-inf")
    dirty = allocate_cache(2, bs, Hkv, fmt, DEV)
    compress_and_scatter(bad_k.to(DEV), bad_v.to(DEV), dirty, slots.to(DEV), books, bs, prerotated=prerotated)
    torch.cuda.synchronize()
    assert _native.read_status(DEV) == 0
    fc = paged_layout.unpack_cache(clean.cpu(), bs, 3, 3, True)
    fd = paged_layout.unpack_cache(dirty.cpu(), bs, 3, 3, True)
    keep_k = torch.ones(2, bs, Hkv, dtype=torch.bool)
    keep_k[0, 3, 1] = keep_k[0, 5, 0] = False
    keep_v = torch.ones(2, bs, Hkv, dtype=torch.bool)
    keep_v[0, 7, 1] = False
    for name, keep in (("k_idx", keep_k), ("k_signs", keep_k), ("k_norm", keep_k), ("k_rnorm", keep_k),
                       ("v_idx", keep_v), ("v_norm", keep_v)):
        assert torch.equal(fc[name][keep], fd[name][keep]), name
    assert not torch.isfinite(fd["k_norm"][0, 3, 1]) and not torch.isfinite(fd["k_norm"][0, 5, 0])
    assert not torch.isfinite(fd["v_norm"][0, 7, 1])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_compress_paged_strided_rows_match_contiguous(dtype):
    """K and V given as strided views of one fused QKV buffer produce the same cache bytes as contiguous copies."""
    fmt = CacheFormat.named("turbo3")
    books = Codebooks(fmt, DEV)
    T, Hkv, bs = 70, 3, 16
    g = torch.Generator().manual_seed(29)
    qkv = torch.randn(T, 5 * Hkv, 128, generator=g).to(dtype).to(DEV)
    key, val = qkv[:, 2 * Hkv:3 * Hkv], qkv[:, 4 * Hkv:]
    slots = torch.randperm(6 * bs, generator=g)[:T].to(DEV)
    a = allocate_cache(6, bs, Hkv, fmt, DEV)
    b = allocate_cache(6, bs, Hkv, fmt, DEV)
    compress_and_scatter(key, val, a, slots, books, bs)
    compress_and_scatter(key.contiguous(), val.contiguous(), b, slots, books, bs)
    assert _native.read_status(DEV) == 0
    assert torch.equal(a, b)


def test_compress_paged_random_shapes_vs_oracle():
    """Seeded sweep over shapes, formats, dtypes and block sizes: pre-rotated inputs must match the oracle bit for
    bit (indices, signs), rotated ones within the 1e-4 allowance; norms within one fp16 ulp."""
    rng = np.random.default_rng(1234)
    fmts = [CacheFormat.named(n) for n in ("turbo2", "turbo3", "turbo4")] + [CacheFormat(4, 2, True), CacheFormat(2, 4, False)]
    for case in range(24):
        fmt = fmts[case % len(fmts)]
        books = Codebooks(fmt, DEV)
        T = int(rng.integers(1, 200))
        Hkv = int(rng.choice([1, 2, 3, 5, 8]))
        bs = int(rng.choice([16, 32, 64]))
        dtype = [torch.float16, torch.bfloat16, torch.float32][case % 3]
        prerotated = bool(case & 1)
        nb = (T + bs - 1) // bs + 1
        g = torch.Generator().manual_seed(100 + case)
        key = (torch.randn(T, Hkv, 128, generator=g) * float(rng.choice([1e-3, 1.0, 30.0]))).to(dtype)
        val = torch.randn(T, Hkv, 128, generator=g).to(dtype)
        slots = torch.randperm(nb * bs, generator=g)[:T]
        cache = allocate_cache(nb, bs, Hkv, fmt, DEV)
        compress_and_scatter(key.to(DEV), val.to(DEV), cache, slots.to(DEV), books, bs, prerotated=prerotated)
        assert _native.read_status(DEV) == 0, case
        f = paged_layout.unpack_cache(cache.cpu(), bs, fmt.k_bits, fmt.v_bits, fmt.use_qjl)
        H = None if prerotated else O.make_wht_matrix(128)
        ok = O.polarquant_compress(key.float().numpy().reshape(-1, 128), books.kc.cpu().numpy(), books.kb.cpu().numpy(),
                                   fmt.k_bits, fmt.use_qjl, H)
        ov = O.polarquant_compress(val.float().numpy().reshape(-1, 128), books.vc.cpu().numpy(), books.vb.cpu().numpy(),
                                   fmt.v_bits, False, H)
        blk, off = slots // bs, slots % bs
        got_k = f["k_idx"][blk, off].numpy().reshape(-1, 128)
        got_v = f["v_idx"][blk, off].numpy().reshape(-1, 128)
        tol = 0.0 if prerotated else 1e-3          # small cases: one flipped coordinate in 128 T Hkv can exceed 1e-4
        assert (got_k != ok["indices"]).mean() <= tol, (case, "k_idx")
        assert (got_v != ov["indices"]).mean() <= tol, (case, "v_idx")
        assert _half_ulp_close(f["k_norm"][blk, off].reshape(-1), ok["norms"]), (case, "k_norm")
        assert _half_ulp_close(f["v_norm"][blk, off].reshape(-1), ov["norms"]), (case, "v_norm")
        if fmt.use_qjl:
            got_s = f["k_signs"][blk, off].numpy().reshape(-1, 128)
            assert (got_s != (ok["signs"] > 0)).mean() <= tol, (case, "signs")
            assert _half_ulp_close(f["k_rnorm"][blk, off].reshape(-1), ok["rot_residual_norm"], max_ulp=2), (case, "rnorm")
