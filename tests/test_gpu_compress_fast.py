"""The persistent paged compress kernel (`compress_paged_fast_kernel`) field by field against the CPU oracle.

Launches of more than 16384 (token, head) items take the persistent kernel with the table-driven quantizer; every
case here has at least 16800 items so that it is that kernel - tensor-core rotation for fp16 / bf16 rows, the
plain branch for fp32 and for already rotated rows, the in-kernel generic fall-back for tight codebooks - whose
indices, signs and norms are compared with `oracle.polarquant_compress`
(the reference arithmetic: turboquant/core/quantizer.py:141-173; the scatter: turboquant/integration/vllm_backend.py:179-230).
"""
import numpy as np
import pytest
import torch

from oracle import tq_oracle as O
from turboquant.kernels import _native, paged_layout
from turboquant.kernels.paged import CacheFormat, Codebooks, allocate_cache, compress_and_scatter

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
T_BIG, HKV = 2100, 8           # 16800 items: 131 full groups of 128 items and a ragged tail of 32
FAST_MIN_ITEMS = 16384


def _kv(T, Hkv, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    key = torch.randn(T, Hkv, 128, generator=g) * scale
    val = torch.randn(T, Hkv, 128, generator=g)
    key[..., [3, 40, 77, 120]] *= 10
    return key.to(dtype), val.to(dtype)


def _fp16_ulps(got_h: torch.Tensor, want_f32: np.ndarray) -> int:
    want_h = torch.from_numpy(want_f32.astype(np.float16))
    a = got_h.cpu().contiguous().view(torch.int16).to(torch.int32)
    b = want_h.view(torch.int16).to(torch.int32)
    return int((a - b).abs().max())


def _run(key, val, fmt, books, block_size=16, prerotated=False, slots=None, seed=0, tcgen05=False):
    T, Hkv = key.shape[:2]
    assert T * Hkv > FAST_MIN_ITEMS
    nb = (T + block_size - 1) // block_size + 3
    if slots is None:
        slots = torch.randperm(nb * block_size, generator=torch.Generator().manual_seed(seed))[:T]
    cache = allocate_cache(nb, block_size, Hkv, fmt, DEV)
    cache.fill_(0x5A)
    compress_and_scatter(key.to(DEV), val.to(DEV), cache, slots.to(DEV), books, block_size, prerotated=prerotated,
                         tcgen05=tcgen05)
    status = _native.read_status(DEV)
    f = paged_layout.unpack_cache(cache.cpu(), block_size, fmt.k_bits, fmt.v_bits, fmt.use_qjl)
    blk, off = slots // block_size, slots % block_size
    return {n: v[blk, off] for n, v in f.items()}, status, cache


def _oracle(key, val, fmt, books, H):
    ok = O.polarquant_compress(key.float().numpy().reshape(-1, 128), books.kc.cpu().numpy(), books.kb.cpu().numpy(),
                               fmt.k_bits, fmt.use_qjl, H)
    ov = O.polarquant_compress(val.float().numpy().reshape(-1, 128), books.vc.cpu().numpy(), books.vb.cpu().numpy(),
                               fmt.v_bits, False, H)
    return ok, ov


@pytest.mark.parametrize("tcgen05", [False, True])
@pytest.mark.parametrize("fmt_name", ["turbo2", "turbo3", "turbo4"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fast_kernel_tensor_core_rotation_vs_oracle(fmt_name, dtype, tcgen05):
    """fp16 / bf16 rows rotated on the tensor cores (mma.sync kernel, and the opt-in tcgen05 kernel with one thread
    per vector): at most 1e-4 of the coordinates differ from the oracle, never by more than one centroid; norms
    within one fp16 ulp; the ragged last group stores only live items."""
    fmt = CacheFormat.named(fmt_name)
    books = Codebooks(fmt, DEV)
    key, val = _kv(T_BIG, HKV, dtype, seed=41)
    got, status, _ = _run(key, val, fmt, books, tcgen05=tcgen05)
    assert status == 0
    ok, ov = _oracle(key, val, fmt, books, O.make_wht_matrix(128))
    gk, gv = got["k_idx"].numpy().reshape(-1, 128).astype(int), got["v_idx"].numpy().reshape(-1, 128).astype(int)
    assert (gk != ok["indices"]).mean() <= 1e-4 and np.abs(gk - ok["indices"]).max() <= 1
    assert (gv != ov["indices"]).mean() <= 1e-4 and np.abs(gv - ov["indices"]).max() <= 1
    assert _fp16_ulps(got["k_norm"].reshape(-1), ok["norms"]) <= 1
    assert _fp16_ulps(got["v_norm"].reshape(-1), ov["norms"]) <= 1
    if fmt.use_qjl:
        gs = got["k_signs"].numpy().reshape(-1, 128)
        assert (gs != (ok["signs"] > 0)).mean() <= 1e-4
        assert _fp16_ulps(got["k_rnorm"].reshape(-1), ok["rot_residual_norm"]) <= 2


@pytest.mark.parametrize("fmt_name", ["turbo2", "turbo3", "turbo4"])
@pytest.mark.parametrize("dtype,prerotated", [(torch.float32, True), (torch.float16, True), (torch.bfloat16, True)])
def test_fast_kernel_plain_branch_prerotated_bit_exact(fmt_name, dtype, prerotated):
    """Already rotated rows (any dtype) take the plain branch: indices and signs equal the oracle's bit for bit."""
    fmt = CacheFormat.named(fmt_name)
    books = Codebooks(fmt, DEV)
    key, val = _kv(T_BIG, HKV, dtype, seed=43)
    got, status, _ = _run(key, val, fmt, books, prerotated=True)
    assert status == 0
    ok, ov = _oracle(key, val, fmt, books, None)
    assert np.array_equal(got["k_idx"].numpy().reshape(-1, 128), ok["indices"])
    assert np.array_equal(got["v_idx"].numpy().reshape(-1, 128), ov["indices"])
    assert _fp16_ulps(got["k_norm"].reshape(-1), ok["norms"]) <= 1
    assert _fp16_ulps(got["v_norm"].reshape(-1), ov["norms"]) <= 1
    if fmt.use_qjl:
        assert np.array_equal(got["k_signs"].numpy().reshape(-1, 128), ok["signs"] > 0)
        assert _fp16_ulps(got["k_rnorm"].reshape(-1), ok["rot_residual_norm"]) <= 2


@pytest.mark.parametrize("fmt_name", ["turbo3", "turbo4"])
def test_fast_kernel_plain_branch_fp32_rotated(fmt_name):
    """fp32 rows rotated by the in-register butterflies of the plain branch: the 1e-4 allowance of any fast WHT."""
    fmt = CacheFormat.named(fmt_name)
    books = Codebooks(fmt, DEV)
    key, val = _kv(T_BIG, HKV, torch.float32, seed=47, scale=0.05)
    got, status, _ = _run(key, val, fmt, books, block_size=32)
    assert status == 0
    ok, ov = _oracle(key, val, fmt, books, O.make_wht_matrix(128))
    gk, gv = got["k_idx"].numpy().reshape(-1, 128).astype(int), got["v_idx"].numpy().reshape(-1, 128).astype(int)
    assert (gk != ok["indices"]).mean() <= 1e-4 and np.abs(gk - ok["indices"]).max() <= 1
    assert (gv != ov["indices"]).mean() <= 1e-4 and np.abs(gv - ov["indices"]).max() <= 1
    assert _fp16_ulps(got["k_norm"].reshape(-1), ok["norms"]) <= 1
    if fmt.use_qjl:
        assert (got["k_signs"].numpy().reshape(-1, 128) != (ok["signs"] > 0)).mean() <= 1e-4


@pytest.mark.parametrize("prerotated,tcgen05", [(False, False), (True, False), (False, True)])
def test_fast_kernel_tight_codebook_falls_back_inside_the_kernel(prerotated, tcgen05):
    """Two boundaries inside one 1/64 cell: the persistent kernels themselves switch to the binary search."""
    fmt = CacheFormat.named("turbo3")
    b = torch.tensor([-0.03, -0.02, -0.01, 0.0, 0.01, 0.02, 0.03])
    c = torch.tensor([-0.05, -0.025, -0.015, -0.005, 0.005, 0.015, 0.025, 0.05])
    books = Codebooks(fmt, DEV, k_codebook=(c, b), v_codebook=(c, b))
    key, val = _kv(T_BIG, HKV, torch.float16, seed=53)
    got, status, _ = _run(key, val, fmt, books, prerotated=prerotated, tcgen05=tcgen05)
    assert status == 0
    ok, ov = _oracle(key, val, fmt, books, None if prerotated else O.make_wht_matrix(128))
    gk, gv = got["k_idx"].numpy().reshape(-1, 128).astype(int), got["v_idx"].numpy().reshape(-1, 128).astype(int)
    gs = got["k_signs"].numpy().reshape(-1, 128)
    if prerotated:
        assert np.array_equal(gk, ok["indices"]) and np.array_equal(gv, ov["indices"])
        assert np.array_equal(gs, ok["signs"] > 0)
    else:
        # boundaries 0.01 apart: a last-bit difference of the rotation moves more coordinates than with Lloyd-Max cells
        assert (gk != ok["indices"]).mean() <= 1e-3 and np.abs(gk - ok["indices"]).max() <= 1
        assert (gv != ov["indices"]).mean() <= 1e-3
        assert (gs != (ok["signs"] > 0)).mean() <= 1e-3


@pytest.mark.parametrize("dtype,prerotated,tcgen05", [(torch.float16, False, False), (torch.bfloat16, False, False),
                                                      (torch.float32, False, False), (torch.float16, True, False),
                                                      (torch.float16, False, True), (torch.bfloat16, False, True)])
def test_fast_kernel_nonfinite_rows_only_spoil_themselves(dtype, prerotated, tcgen05):
    """NaN / Inf inside a vector: that vector's norm shows it, every other byte of the cache is unchanged."""
    fmt = CacheFormat.named("turbo3")
    books = Codebooks(fmt, DEV)
    key, val = _kv(T_BIG, HKV, dtype, seed=59)
    slots = torch.randperm((T_BIG // 16 + 4) * 16, generator=torch.Generator().manual_seed(5))[:T_BIG]
    clean, s0, _ = _run(key, val, fmt, books, prerotated=prerotated, slots=slots, tcgen05=tcgen05)
    bad_k, bad_v = key.clone(), val.clone()
    bad_k[3, 1, 17] = float("nan")
    bad_k[1500, 0, 100] = float("inf")
    bad_v[2099, 7, 0] = float("-inf")
    dirty, s1, _ = _run(bad_k, bad_v, fmt, books, prerotated=prerotated, slots=slots, tcgen05=tcgen05)
    assert s0 == 0 and s1 == 0
    keep_k = torch.ones(T_BIG, HKV, dtype=torch.bool)
    keep_k[3, 1] = keep_k[1500, 0] = False
    keep_v = torch.ones(T_BIG, HKV, dtype=torch.bool)
    keep_v[2099, 7] = False
    for name, keep in (("k_idx", keep_k), ("k_signs", keep_k), ("k_norm", keep_k), ("k_rnorm", keep_k),
                       ("v_idx", keep_v), ("v_norm", keep_v)):
        assert torch.equal(clean[name][keep], dirty[name][keep]), name
    assert not torch.isfinite(dirty["k_norm"][3, 1]) and not torch.isfinite(dirty["k_norm"][1500, 0])
    assert not torch.isfinite(dirty["v_norm"][2099, 7])


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_fast_kernel_strided_views_and_block_sizes(dtype):
    """K and V as strided views of one fused buffer, block size 64: same cache bytes as contiguous copies, and
    those bytes are the oracle's fields."""
    fmt = CacheFormat.named("turbo3")
    books = Codebooks(fmt, DEV)
    g = torch.Generator().manual_seed(61)
    qkv = torch.randn(T_BIG, 4 * HKV, 128, generator=g).to(dtype)
    key, val = qkv[:, HKV:2 * HKV], qkv[:, 3 * HKV:]
    bs = 64
    nb = T_BIG // bs + 3
    slots = torch.randperm(nb * bs, generator=g)[:T_BIG]
    a = allocate_cache(nb, bs, HKV, fmt, DEV)
    b = allocate_cache(nb, bs, HKV, fmt, DEV)
    qkv_d = qkv.to(DEV)
    compress_and_scatter(qkv_d[:, HKV:2 * HKV], qkv_d[:, 3 * HKV:], a, slots.to(DEV), books, bs)
    compress_and_scatter(key.contiguous().to(DEV), val.contiguous().to(DEV), b, slots.to(DEV), books, bs)
    assert _native.read_status(DEV) == 0
    assert torch.equal(a, b)
    f = paged_layout.unpack_cache(a.cpu(), bs, 3, 3, True)
    ok, ov = _oracle(key, val, fmt, books, O.make_wht_matrix(128))
    gk = f["k_idx"][slots // bs, slots % bs].numpy().reshape(-1, 128)
    gv = f["v_idx"][slots // bs, slots % bs].numpy().reshape(-1, 128)
    assert (gk != ok["indices"]).mean() <= 1e-4 and (gv != ov["indices"]).mean() <= 1e-4


def test_fast_kernel_bad_and_negative_slots():
    """Negative slots are clamped to 0 as the reference does, slots beyond the cache are skipped and flagged."""
    fmt = CacheFormat.named("turbo3")
    books = Codebooks(fmt, DEV)
    key, val = _kv(T_BIG, HKV, torch.float16, seed=67)
    nb = T_BIG // 16 + 3
    slots = torch.arange(T_BIG, dtype=torch.int64) + 16          # slot 0..15 left free
    slots[11] = -1                                                 # -> slot 0
    slots[1234] = nb * 16 + 5                                      # beyond the cache
    got, status, cache = _run(key, val, fmt, books, prerotated=True, slots=slots.clamp(0, nb * 16 - 1))
    _ = got
    cache2 = allocate_cache(nb, 16, HKV, fmt, DEV)
    compress_and_scatter(key.to(DEV), val.to(DEV), cache2, slots.to(DEV), books, 16, prerotated=True)
    assert _native.read_status(DEV) == _native.STATUS_BAD_SLOT
    f = paged_layout.unpack_cache(cache2.cpu(), 16, 3, 3, True)
    ok, _ = _oracle(key, val, fmt, books, None)
    want = ok["indices"].reshape(T_BIG, HKV, 128)
    assert np.array_equal(f["k_idx"][0, 0].numpy(), want[11])                      # clamped to slot 0
    assert np.array_equal(f["k_idx"][(1233 + 16) // 16, (1233 + 16) % 16].numpy(), want[1233])
    assert (f["k_idx"][(1234 + 16) // 16, (1234 + 16) % 16] == 0).all()            # skipped: still zero


def test_fast_kernel_residual_underflow_is_the_only_sign_deviation():
    """Rows so small that their squares underflow have norm 0, so every residual (u - c) * n is +-0.  The
    reference counts -0.0 as + (turboquant/core/quantizer.py:171-172: sign(e), then 0 -> +1); the table-driven
    quantizer reads the sign bit and says -.  That is the one documented deviation: it needs a residual of exactly
    +-0, no other row may show a sign difference, and indices (which do not depend on the residual) stay exact."""
    fmt = CacheFormat.named("turbo3")
    books = Codebooks(fmt, DEV)
    g = torch.Generator().manual_seed(71)
    key = torch.randn(T_BIG, HKV, 128, generator=g)
    val = torch.randn(T_BIG, HKV, 128, generator=g)
    tiny = torch.zeros(T_BIG, dtype=torch.bool)
    tiny[::7] = True
    key[tiny] *= 1e-30                                            # squares ~1e-60 underflow in fp32: norm 0
    got, status, _ = _run(key, val, fmt, books, prerotated=True)
    assert status == 0
    ok, _ = _oracle(key, val, fmt, books, None)
    assert np.array_equal(got["k_idx"].numpy().reshape(-1, 128), ok["indices"])
    # the oracle's residual, recomputed with its own operations
    x = key.numpy().reshape(-1, 128)
    n = ok["norms"][:, None]
    resid = (((x / (n + np.float32(1e-8))).astype(np.float32) - books.kc.cpu().numpy()[ok["indices"]]) * n).astype(np.float32)
    differs = got["k_signs"].numpy().reshape(-1, 128) != (ok["signs"] > 0)
    assert not differs[resid != 0].any()                          # a deviation needs a residual of exactly +-0
    tiny_rows = tiny[:, None].expand(T_BIG, HKV).reshape(-1).numpy()
    assert (ok["norms"][tiny_rows] == 0).all() and not differs[~tiny_rows].any()
    assert differs[tiny_rows].any()                               # the deviation is real: -0.0 read as negative
