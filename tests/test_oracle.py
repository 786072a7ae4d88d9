"""The CPU oracle against the golden vectors made by the reference's own Python code."""
import math

import numpy as np
import pytest

from oracle import tq_oracle as O


@pytest.mark.parametrize("d", [64, 128, 256])
@pytest.mark.parametrize("bits", [1, 2, 3, 4])
def test_codebook_matches_reference(golden, d, bits):
    c, b = O.solve_codebook(d, bits)
    # closed-form moments vs the reference's numeric quadrature
    np.testing.assert_allclose(c, golden[f"codebook_d{d}_b{bits}_c"], rtol=0, atol=2e-9)
    np.testing.assert_allclose(b, golden[f"codebook_d{d}_b{bits}_b"], rtol=0, atol=2e-9)
    # the fp32 tensors kernels receive are identical
    assert np.array_equal(np.asarray(c, np.float32), golden[f"codebook_d{d}_b{bits}_c"].astype(np.float32))
    assert np.array_equal(np.asarray(b, np.float32), golden[f"codebook_d{d}_b{bits}_b"].astype(np.float32))


@pytest.mark.parametrize("d", [8, 128])
def test_wht_matrix_bit_exact(golden, d):
    assert np.array_equal(O.make_wht_matrix(d), golden[f"wht_d{d}"])


def test_wht_entries_are_2_pow_minus_3_5():
    H = O.make_wht_matrix(128)
    assert np.all(np.abs(H) == np.float32(0.08838834764831845))
    i, j = np.meshgrid(np.arange(128), np.arange(128), indexing="ij")
    par = np.array([[bin(a & b).count("1") & 1 for b in range(128)] for a in range(128)])
    assert np.array_equal(H < 0, par == 1)


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("tag", ["pre", "rot"])
def test_polarquant_compress(golden, bits, tag):
    x = golden["pq_x"]
    c, b = O.make_codebook(128, bits)
    H = O.make_wht_matrix(128) if tag == "rot" else None
    r = O.polarquant_compress(x, c, b, bits, True, H)
    p = f"pq_b{bits}_{tag}_"
    ref_idx = golden[p + "indices"].astype(np.int64)
    ref_signs = np.unpackbits(golden[p + "signs"], axis=1, bitorder="little").astype(bool)
    diff = r["indices"] != ref_idx
    if tag == "pre":
        # identical fp32 rotated input: indices and signs bit-exact up to the allowance for ties
        assert diff.mean() <= 1e-4
        assert np.abs(r["indices"] - ref_idx).max() <= 1
        assert ((r["signs"] > 0) != ref_signs).mean() <= 1e-4
    else:
        # numpy and torch order the matmul sums differently: stay inside the 1e-4 allowance
        assert diff.mean() <= 1e-4 and np.abs(r["indices"] - ref_idx).max() <= 1
        assert ((r["signs"] > 0) != ref_signs).mean() <= 1e-4
    np.testing.assert_allclose(r["norms"], golden[p + "norms"], rtol=2e-6)
    np.testing.assert_allclose(r["rot_residual_norm"], golden[p + "rnorm"], rtol=2e-5, atol=1e-7)
    np.testing.assert_allclose(r["k_mse_rot"][:8], golden[p + "k_mse_rot"], rtol=2e-6, atol=1e-7)


def test_zero_vector_edge_case(golden):
    # row 5 of the fixture input is all zero: norm 0, every coordinate ties at boundary 0 -> lower centroid, signs +
    c, b = O.make_codebook(128, 3)
    r = O.polarquant_compress(golden["pq_x"][5:6], c, b, 3, True, None)
    assert r["norms"][0] == 0 and r["rot_residual_norm"][0] == 0
    assert np.all(r["indices"] == 3) and np.all(r["signs"] == 1)
    assert np.array_equal(golden["pq_b3_pre_indices"][5], np.full(128, 3, np.uint8))


def test_3d_input_shape(golden):
    c, b = O.make_codebook(128, 3)
    r = O.polarquant_compress(golden["pq3d_x"], c, b, 3, True, O.make_wht_matrix(128))
    assert r["indices"].shape == (4, 8, 128)
    assert (r["indices"] != golden["pq3d_indices"]).mean() <= 1e-4


def test_pack_helpers(golden):
    assert np.array_equal(O.unpack_2bit(golden["pack_idx_bytes"], 128), golden["unpack_2bit"])
    assert np.array_equal(O.unpack_1bit(golden["pack_sign_bytes"], 128), golden["unpack_1bit"])
    assert np.array_equal(O.permute_signs_for_chunked(golden["pack_sign_bytes"]), golden["permute_signs"])
    # known answers quoted from the reference layout: 0xE4 -> [0,1,2,3]; dim 5 -> permuted byte 4 bit 1
    assert list(O.unpack_2bit(np.array([[0xE4] * 32], np.uint8), 128)[0, :4]) == [0, 1, 2, 3]
    seq = np.zeros((1, 16), np.uint8)
    seq[0, 0] = 1 << 5
    perm = O.permute_signs_for_chunked(seq)
    assert perm[0, 4] == 2 and perm.sum() == 2


@pytest.mark.parametrize("bits", [2, 3, 4])
def test_pack_unpack_roundtrip(bits):
    rng = np.random.default_rng(0)
    idx = rng.integers(0, 1 << bits, size=(37, 128))
    packed = O.pack_indices(idx, bits)
    assert packed.shape == (37, 16 * bits)
    assert np.array_equal(O.unpack_indices(packed, bits, 128), idx)
    sg = rng.integers(0, 2, size=(37, 128))
    assert np.array_equal(O.unpack_1bit(O.pack_1bit(sg), 128), sg)


def test_3bit_stream_is_the_reference_decoder():
    # dim d sits at bit 3d: ((B[3d>>3] | B[(3d>>3)+1] << 8) >> (3d & 7)) & 7
    idx = (np.arange(128) * 5 % 8)[None, :]
    B = O.pack_3bit(idx)[0].astype(np.int64)
    B = np.concatenate([B, [0]])
    for d in range(128):
        assert ((B[3 * d >> 3] | (B[(3 * d >> 3) + 1] << 8)) >> (3 * d & 7)) & 7 == idx[0, d]


def test_attention_unpacked_ref(golden):
    g = golden
    out = O.packed_attention(g["attn_q"], g["attn_qp"], g["attn_k_idx"], g["attn_k_signs_perm"], g["attn_k_rnorm"],
                             g["attn_k_norm"], g["attn_v_idx"], g["attn_v_norm"], g["attn_centroids"],
                             float(g["attn_corr_scale"]), bits=2)
    np.testing.assert_allclose(out, g["attn_ref_out"], rtol=1e-4, atol=2e-6)


def test_config1_roundtrip(golden):
    import torch
    torch.manual_seed(0)
    K = torch.randn(1024, 128)
    V = torch.randn(1024, 128)
    q = torch.randn(1, 128)
    assert np.array_equal(K[:4].numpy(), golden["cfg1_K_head"])      # seeded inputs regenerate
    assert np.array_equal(q.numpy(), golden["cfg1_q"])
    out = O.roundtrip_config1(K.numpy(), V.numpy(), q.numpy(), bits=3)
    err = np.abs(out - golden["cfg1_out"])
    assert err.max() <= 2e-3 and np.linalg.norm(out - golden["cfg1_out"]) <= 1e-2 * np.linalg.norm(golden["cfg1_out"])
    c, b = O.make_codebook(128, 3)
    ck = O.polarquant_compress(K.numpy(), c, b, 3, True, O.make_wht_matrix(128))
    assert (ck["indices"] != golden["cfg1_k_indices"]).mean() <= 1e-4


def test_paged_decode_matches_dense_formula():
    """The paged/GQA walker reproduces attention_unpacked_ref on the same logical data, with and without skip."""
    rng = np.random.default_rng(3)
    ns, Hq, Hkv, bs, D = 3, 8, 2, 16, 128
    lens = np.array([40, 16, 1])
    nblk = 8
    kc, _ = O.make_codebook(128, 3)
    kf = {"idx": rng.integers(0, 8, (nblk, bs, Hkv, D)), "norm": rng.random((nblk, bs, Hkv)).astype(np.float32) + 0.5,
          "signs": rng.integers(0, 2, (nblk, bs, Hkv, D)), "rnorm": rng.random((nblk, bs, Hkv)).astype(np.float32) * 0.1}
    vf = {"idx": rng.integers(0, 8, (nblk, bs, Hkv, D)), "norm": rng.random((nblk, bs, Hkv)).astype(np.float32) + 0.5}
    bt = np.stack([rng.permutation(nblk)[:3] for _ in range(ns)])
    q = rng.standard_normal((ns, Hq, D)).astype(np.float32)
    cs, sm = math.sqrt(math.pi / 2) / 128, 0.7
    out = O.paged_decode(q, q, kf, vf, bt, lens, kc, kc, sm, cs, bs)
    G = Hq // Hkv
    for s in range(ns):
        L = lens[s]
        for h in range(Hq):
            kh = h // G
            blks = bt[s, :(L + bs - 1) // bs]
            gather = lambda a: a[blks, :, kh].reshape(-1, *a.shape[3:])[:L]
            K = kc[gather(kf["idx"])] * gather(kf["norm"])[:, None]
            V = kc[gather(vf["idx"])] * gather(vf["norm"])[:, None]
            ref = O.attention_unpacked_ref(q[s, h][None] * np.float32(sm), q[s, h][None] * np.float32(sm), K[None],
                                           (gather(kf["signs"]) * 2.0 - 1.0)[None], gather(kf["rnorm"])[None], V[None], cs)
            np.testing.assert_allclose(out[s, h], ref[0], rtol=2e-5, atol=2e-6)
    # Sparse-V with a threshold nothing falls under equals dense; a huge threshold drops everything but stays finite
    out0 = O.paged_decode(q, q, kf, vf, bt, lens, kc, kc, sm, cs, bs, sparse_thresh=0.0)
    np.testing.assert_allclose(out0, out, rtol=2e-5, atol=2e-6)
    out1, st = O.paged_decode(q, q, kf, vf, bt, lens, kc, kc, sm, cs, bs, sparse_thresh=1e-6, return_stats=True)
    assert st["positions"] == int(lens.sum()) * Hkv
    assert np.abs(out1 - out).max() <= 1e-4


def test_compress_k_packed_sign_projection():
    """The projected signs (PiST of turboquant/kernels/packed_compress.py:75-77): the identity projection gives the
    residual's own signs, a general projection the signs of residual @ PiST computed from the unpacked fields."""
    rng = np.random.default_rng(5)
    x = rng.standard_normal((64, 128)).astype(np.float32)
    c, b = O.make_codebook(128, 2)
    H = O.make_wht_matrix(128)
    base = O.compress_k_packed(x, c, b, 2, H, permuted=False)
    eye = O.compress_k_packed(x, c, b, 2, H, permuted=False, sign_projection=np.eye(128, dtype=np.float32))
    assert all(np.array_equal(u, v) for u, v in zip(base, eye))
    S = rng.standard_normal((128, 128)).astype(np.float32)
    proj = O.compress_k_packed(x, c, b, 2, H, permuted=False, sign_projection=S)
    r = O.polarquant_compress(x, c, b, 2, True, H)
    resid = (x @ H).astype(np.float32) - r["k_mse_rot"]
    want = (resid @ S) >= 0
    got = np.unpackbits(proj[1], axis=1, bitorder="little").astype(bool)
    assert (got != want).mean() <= 1e-3          # the two residual formulas differ by rounding only
    assert np.array_equal(proj[0], base[0]) and np.array_equal(proj[3], base[3])
