"""CUDA decode-attention kernels against the CPU oracle (through the C ABI).

Tolerance for attention outputs (the one the build is held to), against the fp32 computation on the
same packed data: every element within 2e-3 absolute + 1e-2 relative (|diff| <= 2e-3 + 1e-2 |ref|), and
the whole tensor within 1e-2 relative in norm.  The absolute term alone cannot be met for outputs of
magnitude >= 2: half an fp16 ulp of the output itself is 1e-3 at 2.0 and 2e-3 at 4.0.  Cases whose
outputs stay below 1 in magnitude are additionally held to the bare 2e-3 maximum."""
import math

import numpy as np
import pytest
import torch

from oracle import tq_oracle as O
from turboquant.core import make_codebook
from turboquant.kernels import _native, packed_attention as PA, packed_compress, paged_layout, sparse_v
from turboquant.kernels.paged import (CacheFormat, Codebooks, allocate_cache, compress_and_scatter,
                                      paged_decode_attention)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ATOL, RTOL = 2e-3, 1e-2


def assert_attn_close(got, ref):
    got = np.asarray(got, dtype=np.float32)
    ref = np.asarray(ref, dtype=np.float32)
    assert np.isfinite(got).all()
    d = np.abs(got - ref)
    worst = (d - RTOL * np.abs(ref)).max()
    assert worst <= ATOL, f"max (|diff| - 1e-2 |ref|) = {worst:.3e}, max abs {d.max():.3e}"
    if np.abs(ref).max() < 1.0:
        assert d.max() <= ATOL, f"max abs {d.max():.3e}"
    assert np.linalg.norm(got - ref) <= RTOL * np.linalg.norm(ref) + 1e-6, \
        f"rel {np.linalg.norm(got - ref) / np.linalg.norm(ref):.3e}"


def random_fields(fmt, nb, bs, hkv, seed):
    g = torch.Generator().manual_seed(seed)
    f = {"k_idx": torch.randint(0, 1 << fmt.k_bits, (nb, bs, hkv, 128), generator=g, dtype=torch.uint8),
         "v_idx": torch.randint(0, 1 << fmt.v_bits, (nb, bs, hkv, 128), generator=g, dtype=torch.uint8),
         "k_norm": (torch.rand(nb, bs, hkv, generator=g) * 4 + 8).half(),
         "v_norm": (torch.rand(nb, bs, hkv, generator=g) * 4 + 8).half()}
    if fmt.use_qjl:
        f["k_signs"] = torch.randint(0, 2, (nb, bs, hkv, 128), generator=g, dtype=torch.uint8)
        f["k_rnorm"] = (torch.rand(nb, bs, hkv, generator=g) * 3).half()
    return f


def oracle_decode(q, qp, f, fmt, books, bt, lens, sm, cs, bs, thresh=None):
    kf = {"idx": f["k_idx"].numpy(), "norm": f["k_norm"].float().numpy()}
    if fmt.use_qjl:
        kf["signs"] = f["k_signs"].numpy()
        kf["rnorm"] = f["k_rnorm"].float().numpy()
    vf = {"idx": f["v_idx"].numpy(), "norm": f["v_norm"].float().numpy()}
    return O.paged_decode(q.float().numpy(), (q if qp is None else qp).float().numpy(), kf, vf, bt.numpy(), lens.numpy(),
                          books.kc.cpu().numpy(), books.vc.cpu().numpy(), sm, cs, bs, sparse_thresh=thresh)


def run_case(fmt, lens, Hq, Hkv, bs, seed=0, dtype=torch.float16, chunk_pages=0, thresh=0.0, with_qp=False, qscale=1.0):
    books = Codebooks(fmt, DEV)
    lens = torch.tensor(lens, dtype=torch.int32)
    ns = len(lens)
    max_blocks = max(1, (int(lens.max()) + bs - 1) // bs)
    nb = ns * max_blocks + 3
    g = torch.Generator().manual_seed(seed + 100)
    f = random_fields(fmt, nb, bs, Hkv, seed)
    cache = paged_layout.pack_cache(f, bs, fmt.k_bits, fmt.v_bits, fmt.use_qjl).to(DEV)
    bt = torch.randperm(nb, generator=g)[:ns * max_blocks].reshape(ns, max_blocks).to(torch.int32)
    q = (torch.randn(ns, Hq, 128, generator=g) * qscale).to(dtype)
    qp = (torch.randn(ns, Hq, 128, generator=g) * qscale).to(dtype) if with_qp else None
    sm, cs = 1 / math.sqrt(128), math.sqrt(math.pi / 2) / 128
    out = paged_decode_attention(q.to(DEV), cache, bt.to(DEV), lens.to(DEV), books, bs, sm, cs, sparse_thresh=thresh,
                                 q_proj=None if qp is None else qp.to(DEV), chunk_pages=chunk_pages)
    torch.cuda.synchronize()
    assert _native.read_status(DEV) == 0
    assert out.dtype == dtype and out.shape == (ns, Hq, 128)
    ref = oracle_decode(q, qp, f, fmt, books, bt, lens, sm, cs, bs)
    return out.float().cpu().numpy(), ref


@pytest.mark.parametrize("name", ["turbo2", "turbo3", "turbo4"])
@pytest.mark.parametrize("Hq,Hkv", [(8, 1), (32, 8), (8, 8), (12, 2), (32, 2)])
def test_decode_formats_and_group_sizes(name, Hq, Hkv):
    out, ref = run_case(CacheFormat.named(name), [200, 16, 1, 77], Hq, Hkv, 16, seed=Hq)
    assert_attn_close(out, ref)


@pytest.mark.parametrize("L", [1, 15, 16, 17, 31, 32, 33, 63, 64, 65, 1000])
def test_decode_ragged_lengths(L):
    out, ref = run_case(CacheFormat.named("turbo3"), [L, max(1, L - 1)], 16, 2, 16, seed=L)
    assert_attn_close(out, ref)


@pytest.mark.parametrize("kb,vb,qjl", [(4, 2, False), (4, 3, True), (3, 2, True), (2, 4, False), (3, 3, False), (4, 4, True)])
def test_decode_asymmetric_bits(kb, vb, qjl):
    out, ref = run_case(CacheFormat(kb, vb, qjl), [130, 40], 16, 4, 16, seed=kb * 7 + vb)
    assert_attn_close(out, ref)


def test_decode_block_size_32_bf16_and_separate_qproj():
    out, ref = run_case(CacheFormat.named("turbo3"), [300, 33, 32], 16, 4, 32, seed=1, with_qp=True)
    assert_attn_close(out, ref)
    out, ref = run_case(CacheFormat.named("turbo3"), [300, 33], 16, 4, 16, seed=2, dtype=torch.bfloat16)
    d = np.abs(out - ref)                       # bf16 output rounding (2^-9 relative) is the floor here
    assert d.max() <= 8e-3 and np.linalg.norm(out - ref) <= 1e-2 * np.linalg.norm(ref)


@pytest.mark.parametrize("chunk", [1, 2, 5, 64])
def test_decode_split_k_merge(chunk):
    """Many chunks per sequence (down to one page each), sequences of different chunk counts, an empty one."""
    out, ref = run_case(CacheFormat.named("turbo3"), [700, 90, 0, 16], 8, 2, 16, seed=chunk, chunk_pages=chunk)
    assert_attn_close(out, ref)
    assert (out[2] == 0).all()                  # empty sequence -> zeros


def test_decode_peaked_logits_and_sparse_v():
    """Large queries make the softmax peaked: most V pages fall under the threshold and are skipped."""
    fmt = CacheFormat.named("turbo3")
    for thresh in (1e-6, 1e-2):
        out, ref = run_case(fmt, [2000, 555], 8, 1, 16, seed=3, thresh=thresh, qscale=6.0)
        assert_attn_close(out, ref)             # against the dense (no-skip) fp32 truth
    out_d, _ = run_case(fmt, [2000, 555], 8, 1, 16, seed=3, thresh=0.0, qscale=6.0)
    assert_attn_close(out_d, ref)
    # skip statistics: with a peaked softmax a large share of the pages is skipped
    books = Codebooks(fmt, DEV)
    f = random_fields(fmt, 130, 16, 1, 3)
    cache = paged_layout.pack_cache(f, 16, 3, 3, True).to(DEV)
    bt = torch.arange(125, dtype=torch.int32).reshape(1, 125).to(DEV)
    q = (torch.randn(1, 8, 128, generator=torch.Generator().manual_seed(1)) * 40).half().to(DEV)
    stats = torch.zeros(2, dtype=torch.int32, device=DEV)
    # one chunk, so that every warp streams 32 pages: a warp's first four pages are always fetched whole, after
    # that the V part of a page is only fetched while pages are being used
    paged_decode_attention(q, cache, bt, torch.tensor([2000], dtype=torch.int32, device=DEV), books, 16,
                           sparse_thresh=1e-6, skip_stats=stats, chunk_pages=128)
    seen, skipped = stats.cpu().tolist()
    assert seen == 125 and 0 < skipped < seen


def test_decode_bad_block_table_is_flagged_not_fatal():
    fmt = CacheFormat.named("turbo4")
    books = Codebooks(fmt, DEV)
    cache = allocate_cache(4, 16, 2, fmt, DEV)
    bt = torch.tensor([[1, 99, -5]], dtype=torch.int32, device=DEV)      # two entries outside the cache
    q = torch.randn(1, 8, 128, device=DEV).half()
    out = paged_decode_attention(q, cache, bt, torch.tensor([40], dtype=torch.int32, device=DEV), books, 16)
    torch.cuda.synchronize()
    assert _native.read_status(DEV) == _native.STATUS_BAD_BLOCK
    assert torch.isfinite(out.float()).all()
    with pytest.raises(ValueError):                                       # block size / cache row mismatch is refused
        paged_decode_attention(q, cache, bt, torch.tensor([40], dtype=torch.int32, device=DEV), books, 32)


@pytest.mark.parametrize("chunk", [0, 2])
def test_decode_length_beyond_block_table_is_cut_and_flagged(chunk):
    """A sequence length larger than the block table can describe: the walk stops at the table's width (and the
    chunk count at the workspace's), the status word says so, the result is the attention over the covered part."""
    fmt = CacheFormat.named("turbo3")
    books = Codebooks(fmt, DEV)
    f = random_fields(fmt, 12, 16, 2, 31)
    cache = paged_layout.pack_cache(f, 16, 3, 3, True).to(DEV)
    g = torch.Generator().manual_seed(32)
    bt = torch.randperm(12, generator=g)[:8].reshape(2, 4).to(torch.int32)
    q = torch.randn(2, 8, 128, generator=g).half()
    lens_bad = torch.tensor([4 * 16 + 300, 50], dtype=torch.int32)
    out = paged_decode_attention(q.to(DEV), cache, bt.to(DEV), lens_bad.to(DEV), books, 16, chunk_pages=chunk)
    torch.cuda.synchronize()
    assert _native.read_status(DEV) == _native.STATUS_BAD_BLOCK
    lens_cut = torch.tensor([64, 50], dtype=torch.int32)
    ref = oracle_decode(q, None, f, fmt, books, bt, lens_cut, 1 / math.sqrt(128), math.sqrt(math.pi / 2) / 128, 16)
    assert_attn_close(out.float().cpu().numpy(), ref)
    # the same cut when the host states the longest sequence instead of relying on the table's width
    wide = torch.zeros(2, 40, dtype=torch.int32)
    wide[:, :4] = bt
    out2 = paged_decode_attention(q.to(DEV), cache, wide.to(DEV), lens_cut.to(DEV), books, 16, chunk_pages=chunk,
                                  max_seq_len=64)
    assert _native.read_status(DEV) == 0
    assert_attn_close(out2.float().cpu().numpy(), ref)


def _slice_case(fmt, lens, G, thresh, qscale, seed, bias_pages=0.0, chunk_pages=256):
    """One KV head, `G` query heads, sequences of the given lengths over a shared random page pool."""
    books = Codebooks(fmt, DEV)
    lens_t = torch.tensor(lens, dtype=torch.int32)
    pages = [(n + 15) // 16 for n in lens]
    nb = sum(pages) + 2
    f = random_fields(fmt, nb, 16, 1, seed)
    g = torch.Generator().manual_seed(seed + 1)
    perm = torch.randperm(nb, generator=g)
    bt = torch.zeros(len(lens), max(pages), dtype=torch.int32)
    o = 0
    for i, n in enumerate(pages):
        bt[i, :n] = perm[o:o + n].to(torch.int32)
        o += n
    if bias_pages > 0:
        # a few pages whose keys line up with the query far better than the rest: large norms make their logits peak
        hot = torch.rand(nb, generator=g) < bias_pages
        f["k_norm"][hot] = (f["k_norm"][hot].float() * 5).half()
    cache = paged_layout.pack_cache(f, 16, fmt.k_bits, fmt.v_bits, fmt.use_qjl).to(DEV)
    q = (torch.randn(len(lens), G, 128, generator=g) * qscale).half()
    sm, cs = 1 / math.sqrt(128), math.sqrt(math.pi / 2) / 128
    stats = torch.zeros(2, dtype=torch.int32, device=DEV) if thresh > 0 else None
    # chunks of 256 pages, as the launcher picks for the full batch of this workload (the two-sequence slice alone
    # would get 16-page chunks, where every page is among a warp's first four and is fetched whole)
    out = paged_decode_attention(q.to(DEV), cache, bt.to(DEV), lens_t.to(DEV), books, 16, sm, cs, sparse_thresh=thresh,
                                 skip_stats=stats, chunk_pages=chunk_pages)
    torch.cuda.synchronize()
    assert _native.read_status(DEV) == 0
    ref = oracle_decode(q, None, f, fmt, books, bt, lens_t, sm, cs, 16)        # dense fp32 truth
    return out.float().cpu().numpy(), ref, (None if stats is None else stats.cpu().tolist())


def test_long_sparse_sequence_slice_vs_oracle():
    """The shape of the high-concurrency long-context workload for one (sequence, KV head): 32768 tokens
    (2048 pages, split into chunks), GQA 8, turbo3, Sparse-V threshold 1e-6 with a peaked softmax."""
    out, ref, stats = _slice_case(CacheFormat.named("turbo3"), [32768, 16384 + 5], 8, 1e-6, 3.0, 41, bias_pages=0.02)
    assert_attn_close(out, ref)
    assert stats[0] == 2048 + 1025 and stats[1] > 0                              # pages were really skipped
    out_d, ref_d, _ = _slice_case(CacheFormat.named("turbo3"), [32768, 16384 + 5], 8, 0.0, 3.0, 41, bias_pages=0.02)
    assert_attn_close(out_d, ref_d)


def test_mixed_length_turbo2_slice_vs_oracle():
    """The shape of the mixed-length workload for one KV head: turbo2 (2-bit + QJL), GQA 4, lengths from 128 to
    65536 tokens (4096 pages, 16 chunks) in one batch."""
    out, ref, _ = _slice_case(CacheFormat.named("turbo2"), [65536, 128, 4096, 1500, 9000], 4, 0.0, 1.0, 43)
    assert_attn_close(out, ref)


def test_config2_compress_then_decode():
    """turbo4 single-sequence round trip: 32 query / 8 KV heads, context 4096, block 16, permuted block table,
    fp16 K/V with 4 outlier channels x10, one decode step; compress with the CUDA kernel, then decode."""
    fmt = CacheFormat.named("turbo4")
    books = Codebooks(fmt, DEV)
    T, Hq, Hkv, bs = 4096, 32, 8, 16
    g = torch.Generator().manual_seed(2)
    K = torch.randn(T, Hkv, 128, generator=g)
    V = torch.randn(T, Hkv, 128, generator=g)
    K[..., [5, 50, 90, 127]] *= 10
    V[..., [5, 50, 90, 127]] *= 10
    K, V = K.half(), V.half()
    q = torch.randn(1, Hq, 128, generator=g).half()
    nb = T // bs
    perm = torch.randperm(nb, generator=g)
    slots = (perm[torch.arange(T) // bs] * bs + torch.arange(T) % bs).to(torch.int64)
    cache = allocate_cache(nb, bs, Hkv, fmt, DEV)
    compress_and_scatter(K.to(DEV), V.to(DEV), cache, slots.to(DEV), books, bs)
    out = paged_decode_attention(q.to(DEV), cache, perm.to(torch.int32).reshape(1, nb).to(DEV),
                                 torch.tensor([T], dtype=torch.int32, device=DEV), books, bs,
                                 rotate_q=True, derotate_out=True)
    torch.cuda.synchronize()
    assert _native.read_status(DEV) == 0
    # oracle: reference CPU path on the same inputs (fp32), original space in and out
    H = O.make_wht_matrix(128)
    outs = np.zeros((Hq, 128), np.float32)
    for h in range(Hkv):
        ck = O.polarquant_compress(K[:, h].float().numpy(), books.kc.cpu().numpy(), books.kb.cpu().numpy(), 4, False, H)
        cv = O.polarquant_compress(V[:, h].float().numpy(), books.vc.cpu().numpy(), books.vb.cpu().numpy(), 4, False, H)
        # norms are stored as fp16 in the cache
        Kd = books.kc.cpu().numpy()[ck["indices"]] * ck["norms"].astype(np.float16).astype(np.float32)[:, None]
        Vd = books.vc.cpu().numpy()[cv["indices"]] * cv["norms"].astype(np.float16).astype(np.float32)[:, None]
        for gq in range(Hq // Hkv):
            hq = h * (Hq // Hkv) + gq
            qr = q[0, hq].float().numpy() @ H
            qr = qr.astype(np.float16).astype(np.float32)                   # the rotated query is handed over in fp16
            s = (Kd @ qr) / math.sqrt(128)
            p = np.exp(s - s.max())
            outs[hq] = ((p / p.sum()) @ Vd) @ H
    assert_attn_close(out[0].float().cpu().numpy(), outs)


def test_packed_attention_vs_golden(golden):
    g = golden
    t = lambda k: torch.from_numpy(g[k]).to(DEV)
    out = PA.packed_attention(t("attn_q"), t("attn_qp"), t("attn_k_idx"), t("attn_k_signs_perm"), t("attn_k_rnorm"),
                              t("attn_k_norm"), t("attn_v_idx"), t("attn_v_norm"), t("attn_centroids"),
                              float(g["attn_corr_scale"]))
    assert out.dtype == torch.float16 and out.shape == (4, 128)
    assert_attn_close(out.float().cpu().numpy(), g["attn_ref_out"])       # the reference's own fp32 truth


@pytest.mark.parametrize("bits", [2, 3, 4])
@pytest.mark.parametrize("BH,Sk,splits", [(8, 256, None), (3, 1000, 7), (2, 4096, None), (1, 1, None), (5, 130, 130),
                                          (40, 2500, 9)])   # the last two: more (row, split) items than resident CTAs
def test_packed_attention_vs_oracle(bits, BH, Sk, splits):
    """Random packed bytes as in the reference's self-check (packed_attention.py:371-404), its tolerance tightened
    from cosine > 0.99 to the 2e-3 / 1e-2 bar."""
    gen = torch.Generator().manual_seed(bits * 1000 + Sk)
    c, _ = make_codebook(128, bits)
    k_idx = torch.randint(0, 256, (BH, Sk, 16 * bits), dtype=torch.uint8, generator=gen)
    k_sg = torch.randint(0, 256, (BH, Sk, 16), dtype=torch.uint8, generator=gen)
    v_idx = torch.randint(0, 256, (BH, Sk, 16 * bits), dtype=torch.uint8, generator=gen)
    k_rn = (torch.rand(BH, Sk, generator=gen) * 3).half()
    k_n = (torch.rand(BH, Sk, generator=gen) * 4 + 8).half()
    v_n = (torch.rand(BH, Sk, generator=gen) * 4 + 8).half()
    Q = (torch.randn(BH, 128, generator=gen) / math.sqrt(128)).half()
    Qp = (torch.randn(BH, 128, generator=gen) / math.sqrt(128)).half()
    cs = math.sqrt(math.pi / 2) / math.sqrt(128)
    out = PA.packed_attention(Q.to(DEV), Qp.to(DEV), k_idx.to(DEV), k_sg.to(DEV), k_rn.to(DEV), k_n.to(DEV),
                              v_idx.to(DEV), v_n.to(DEV), c.to(DEV), cs, num_splits=splits, block_sk=16, num_warps=2)
    ref = O.packed_attention(Q.numpy(), Qp.numpy(), k_idx.numpy(), k_sg.numpy(), k_rn.numpy(), k_n.numpy(),
                             v_idx.numpy(), v_n.numpy(), c.numpy(), cs, bits=bits)
    assert_attn_close(out.float().cpu().numpy(), ref)
    assert len(PA._get_config(BH, Sk)) == 4


def test_packed_compress_feeds_packed_attention():
    """compress_k_permuted / compress_v output, reshaped to [BH, Sk, ...], is what packed_attention reads."""
    BH, Sk = 4, 512
    gen = torch.Generator().manual_seed(5)
    c, b = make_codebook(128, 2)
    from turboquant.core import make_wht_matrix
    H = make_wht_matrix(128)
    K = torch.randn(BH * Sk, 128, generator=gen)
    V = torch.randn(BH * Sk, 128, generator=gen)
    q = torch.randn(BH, 128, generator=gen)
    k_idx, k_sgp, k_rn, k_n = packed_compress.compress_k_permuted(K.to(DEV), H.to(DEV), None, c.to(DEV), b.to(DEV))
    v_idx, v_n = packed_compress.compress_v(V.to(DEV), H.to(DEV), c.to(DEV), b.to(DEV))
    Q = ((q @ H) / math.sqrt(128)).half()
    cs = math.sqrt(math.pi / 2) / 128
    out = PA.packed_attention(Q.to(DEV), Q.to(DEV), k_idx.view(BH, Sk, -1), k_sgp.view(BH, Sk, -1), k_rn.view(BH, Sk),
                              k_n.view(BH, Sk), v_idx.view(BH, Sk, -1), v_n.view(BH, Sk), c.to(DEV), cs)
    ref = O.packed_attention(Q.numpy(), Q.numpy(), k_idx.view(BH, Sk, -1).cpu().numpy(), k_sgp.view(BH, Sk, -1).cpu().numpy(),
                             k_rn.view(BH, Sk).cpu().numpy(), k_n.view(BH, Sk).cpu().numpy(),
                             v_idx.view(BH, Sk, -1).cpu().numpy(), v_n.view(BH, Sk).cpu().numpy(), c.numpy(), cs, bits=2)
    assert_attn_close(out.float().cpu().numpy(), ref)


def test_sparse_v_wrapper_on_reference_layout_cache():
    """A cache in the reference's [blocks, 2, block, heads, slot] layout (3-bit stream + fp16 norm at byte 48),
    converted once, gives the dense oracle result; v12 (skip) and v11 (dense) agree within the bar."""
    gen = torch.Generator().manual_seed(8)
    ns, Hkv, G, bs, slot = 3, 2, 6, 32, 64
    Hq = Hkv * G
    lens = torch.tensor([100, 32, 7], dtype=torch.int32)
    nb = 16
    ref_cache = torch.randint(0, 256, (nb, 2, bs, Hkv, slot), dtype=torch.uint8, generator=gen)
    norms = (torch.rand(nb, 2, bs, Hkv, generator=gen) * 0.5 + 0.5).half()
    ref_cache[..., 48:50] = norms.unsqueeze(-1).view(torch.uint8).reshape(nb, 2, bs, Hkv, 2)
    c, _ = make_codebook(128, 3)
    bt = torch.randperm(nb, generator=gen)[:ns * 4].reshape(ns, 4).to(torch.int32)
    q = torch.randn(ns, Hq, 128, generator=gen).half()
    scale = 1 / math.sqrt(128)
    cache = sparse_v.repack_reference_cache(ref_cache, bs).to(DEV)
    out12 = sparse_v.tq_v12_sparse_v(torch.empty_like(q, device=DEV), q.to(DEV), cache, c.to(DEV), bt.to(DEV), lens.to(DEV), scale)
    out11 = sparse_v.tq_v11_dense(torch.empty_like(q, device=DEV), q.to(DEV), cache, c.to(DEV), bt.to(DEV), lens.to(DEV), scale)
    kf = {"idx": O.unpack_3bit(ref_cache[:, 0, ..., :48].reshape(-1, 48).numpy(), 128).reshape(nb, bs, Hkv, 128),
          "norm": norms[:, 0].float().numpy()}
    vf = {"idx": O.unpack_3bit(ref_cache[:, 1, ..., :48].reshape(-1, 48).numpy(), 128).reshape(nb, bs, Hkv, 128),
          "norm": norms[:, 1].float().numpy()}
    ref = O.paged_decode(q.float().numpy(), q.float().numpy(), kf, vf, bt.numpy(), lens.numpy(), c.numpy(), c.numpy(),
                         scale, 0.0, bs)
    assert_attn_close(out11.float().cpu().numpy(), ref)
    assert_attn_close(out12.float().cpu().numpy(), ref)
    assert sparse_v.SPARSE_V_THRESHOLD == 1e-6


def test_full_size_decode_properties():
    """The batched-decode workload at full size for one layer (64 x 8192 tokens, 64q/8kv, turbo3, cache written by the compress
    kernel): results do not depend on the split-K chunking, on where pages sit in the pool, or on a common
    power-of-two scale of V; a slice of the batch matches the oracle."""
    fmt = CacheFormat.named("turbo3")
    books = Codebooks(fmt, DEV)
    B, L, Hq, Hkv, bs = 64, 8192, 64, 8, 16
    nb = B * L // bs
    gd = torch.Generator(device=DEV).manual_seed(21)
    bt = torch.randperm(nb, generator=torch.Generator().manual_seed(22)).to(torch.int32).reshape(B, L // bs).to(DEV)
    cache = allocate_cache(nb, bs, Hkv, fmt, DEV)
    cache2 = allocate_cache(nb, bs, Hkv, fmt, DEV)          # same data, V scaled by 4, different placement
    bt2 = bt.flip(1).contiguous()
    for s0 in range(0, B, 8):
        K = torch.randn(8 * L, Hkv, 128, generator=gd, device=DEV, dtype=torch.float16)
        V = torch.randn(8 * L, Hkv, 128, generator=gd, device=DEV, dtype=torch.float16)
        pos = torch.arange(L, device=DEV)
        slots = (bt[s0:s0 + 8].long().repeat_interleave(bs, dim=1) * bs + pos % bs).reshape(-1)
        compress_and_scatter(K, V, cache, slots, books, bs)
        # the flipped table maps logical page p to physical page bt[., last - p]: re-scatter with the token order kept
        slots2 = (bt2[s0:s0 + 8].long().repeat_interleave(bs, dim=1) * bs + pos % bs).reshape(-1)
        compress_and_scatter(K, V * 4, cache2, slots2, books, bs)
    lens = torch.full((B,), L, dtype=torch.int32, device=DEV)
    q = torch.randn(B, Hq, 128, generator=gd, device=DEV, dtype=torch.float16)
    outs = [paged_decode_attention(q, cache, bt, lens, books, bs, chunk_pages=c).float() for c in (0, 64, 512)]
    torch.cuda.synchronize()
    assert _native.read_status(DEV) == 0
    for o in outs[1:]:
        assert_attn_close(o.cpu().numpy(), outs[0].cpu().numpy())
    o2 = paged_decode_attention(q, cache2, bt2, lens, books, bs).float()
    assert_attn_close((o2 / 4).cpu().numpy(), outs[0].cpu().numpy())
    # oracle on two (sequence, KV head) slices of the full-size cache
    for s, kh in ((3, 0), (60, 7)):
        pages = cache[bt[s].long(), kh].cpu()                                       # [512, page_bytes]
        f = paged_layout.unpack_pages(pages, 3, 3, True)
        kf = {"idx": f["k_idx"].reshape(-1, bs, 1, 128).numpy(), "norm": f["k_norm"].float().reshape(-1, bs, 1).numpy(),
              "signs": f["k_signs"].reshape(-1, bs, 1, 128).numpy(), "rnorm": f["k_rnorm"].float().reshape(-1, bs, 1).numpy()}
        vf = {"idx": f["v_idx"].reshape(-1, bs, 1, 128).numpy(), "norm": f["v_norm"].float().reshape(-1, bs, 1).numpy()}
        qs = q[s:s + 1, kh * 8:(kh + 1) * 8].float().cpu().numpy()
        ref = O.paged_decode(qs, qs, kf, vf, np.arange(L // bs)[None], np.array([L]), books.kc.cpu().numpy(),
                             books.vc.cpu().numpy(), 1 / math.sqrt(128), math.sqrt(math.pi / 2) / 128, bs)
        assert_attn_close(outs[0][s, kh * 8:(kh + 1) * 8].cpu().numpy(), ref[0])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fused_rotations_match_separate_passes(dtype):
    """TQ_IO_ROTATE_Q / TQ_IO_DEROTATE_OUT: rotating inside the decode kernels gives what wht_rows before and
    after the call gives (the fused query is rounded to the io dtype exactly like the separate pass)."""
    fmt = CacheFormat.named("turbo3")
    books = Codebooks(fmt, DEV)
    lens = torch.tensor([700, 90, 16, 0], dtype=torch.int32)      # multi-chunk, single-chunk, one page, empty
    f = random_fields(fmt, 64, 16, 2, 5)
    cache = paged_layout.pack_cache(f, 16, 3, 3, True).to(DEV)
    g = torch.Generator().manual_seed(6)
    bt = torch.stack([torch.randperm(64, generator=g)[:44] for _ in range(4)]).to(torch.int32).to(DEV)
    q = torch.randn(4, 16, 128, generator=g).to(dtype).to(DEV)
    q_rot = _native.wht_rows(q)
    for chunk in (0, 4):
        sep_rot = paged_decode_attention(q_rot, cache, bt, lens.to(DEV), books, 16, chunk_pages=chunk)
        fused_q = paged_decode_attention(q, cache, bt, lens.to(DEV), books, 16, chunk_pages=chunk, rotate_q=True)
        assert torch.equal(fused_q, sep_rot)
        sep_out = _native.wht_rows(sep_rot)
        fused = paged_decode_attention(q, cache, bt, lens.to(DEV), books, 16, chunk_pages=chunk, rotate_q=True,
                                       derotate_out=True)
        tol = 2e-3 if dtype == torch.float16 else 1.6e-2           # one rounding to the output dtype less than two
        assert (fused.float() - sep_out.float()).abs().max().item() <= tol
        assert (fused[3] == 0).all()
