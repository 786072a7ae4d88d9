#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ from the reference's own Python code.

Run once in a container that has the reference checkout (it cannot travel to
the GPU machine, so only the vectors are committed):

    python tests/golden/make_golden.py /path/to/reference

Everything written here comes from calling the reference unmodified:
turboquant.core.{solve_codebook, make_wht_matrix, PolarQuantConfig,
polarquant_compress} and the pure-torch helpers of
turboquant.kernels.{packed_compress, packed_attention} (unpack_2bit,
unpack_1bit, permute_signs_for_chunked, attention_unpacked_ref).
"""
import math
import os
import sys

import numpy as np
import torch

if len(sys.argv) < 2:
    raise SystemExit("usage: make_golden.py <path to the reference checkout>")
ref_root = sys.argv[1]
sys.path.insert(0, ref_root)
here = os.path.dirname(os.path.abspath(__file__))

from turboquant.core import (PolarQuantConfig, make_codebook, make_wht_matrix,  # noqa: E402
                             polarquant_compress, solve_codebook)
from turboquant.kernels import packed_attention as ref_pa  # noqa: E402
from turboquant.kernels import packed_compress as ref_pc  # noqa: E402

torch.set_num_threads(1)
out = {}

# --- codebooks (core/codebook.py) -----------------------------------------
for d in (64, 128, 256):
    for bits in (1, 2, 3, 4):
        c, b = solve_codebook(d, bits)
        out[f"codebook_d{d}_b{bits}_c"] = np.asarray(c, dtype=np.float64)
        out[f"codebook_d{d}_b{bits}_b"] = np.asarray(b, dtype=np.float64)

# --- WHT matrix (core/rotation.py) -----------------------------------------
for d in (8, 128):
    out[f"wht_d{d}"] = make_wht_matrix(d).numpy()

# --- polarquant_compress (core/quantizer.py) --------------------------------
torch.manual_seed(0)
x = torch.randn(256, 128)
x[:, [3, 40, 77, 120]] *= 10.0          # outlier channels as in the benchmark configs
x[5] = 0.0                              # all-zero vector edge case
out["pq_x"] = x.numpy()
H = make_wht_matrix(128)
for bits in (2, 3, 4):
    c, b = make_codebook(128, bits)
    cfg = PolarQuantConfig(head_dim=128, bits=bits, use_qjl=True)
    for tag, rot in (("rot", H), ("pre", None)):
        r = polarquant_compress(x, c, b, cfg, rot)
        p = f"pq_b{bits}_{tag}_"
        out[p + "indices"] = r["indices"].numpy().astype(np.uint8)
        out[p + "norms"] = r["norms"].numpy()
        out[p + "signs"] = np.packbits((r["signs"].numpy() > 0).astype(np.uint8), axis=1, bitorder="little")
        out[p + "rnorm"] = r["rot_residual_norm"].numpy()
        out[p + "k_mse_rot"] = r["k_mse_rot"].numpy().astype(np.float32)[:8]
    cfg_v = PolarQuantConfig(head_dim=128, bits=bits, use_qjl=False)
    rv = polarquant_compress(x, c, b, cfg_v, H)
    out[f"pq_b{bits}_noqjl_keys"] = np.array(sorted(rv.keys()))
# 3-D input keeps its shape (tests/test_compress.py:53-61)
c3, b3 = make_codebook(128, 3)
torch.manual_seed(0)
x3 = torch.randn(4, 8, 128)
r3 = polarquant_compress(x3, c3, b3, PolarQuantConfig(bits=3), H)
out["pq3d_x"] = x3.numpy()
out["pq3d_indices"] = r3["indices"].numpy().astype(np.uint8)

# --- PolarQuantConfig behaviour ---------------------------------------------
rows = []
for bits in (2, 3, 4):
    for vb in (None, 2, 3, 4):
        cfg = PolarQuantConfig(head_dim=128, bits=bits, v_bits=vb)
        rows.append([bits, -1 if vb is None else vb, cfg.k_bits, cfg.effective_v_bits,
                     int(cfg.is_asymmetric), cfg.n_centroids, cfg.compression_ratio,
                     cfg.k_compression_ratio, cfg.v_compression_ratio, cfg.combined_compression_ratio])
out["config_rows"] = np.asarray(rows, dtype=np.float64)
cfg = PolarQuantConfig(num_layers=40, protect_boundary_layers=True, num_protected_layers=2)
out["config_should_compress_40"] = np.asarray([cfg.should_compress(i) for i in range(40)])
cfg = PolarQuantConfig(num_layers=0)
out["config_should_compress_0"] = np.asarray([cfg.should_compress(i) for i in range(8)])

# --- packing helpers (kernels/packed_compress.py) ----------------------------
g = torch.Generator().manual_seed(1)
pk = torch.randint(0, 256, (16, 32), dtype=torch.uint8, generator=g)
sg = torch.randint(0, 256, (16, 16), dtype=torch.uint8, generator=g)
out["pack_idx_bytes"] = pk.numpy()
out["pack_sign_bytes"] = sg.numpy()
out["unpack_2bit"] = ref_pc.unpack_2bit(pk, 128).numpy()
out["unpack_1bit"] = ref_pc.unpack_1bit(sg, 128).numpy()
out["permute_signs"] = ref_pc.permute_signs_for_chunked(sg).numpy()

# --- attention_unpacked_ref (kernels/packed_attention.py) ---------------------
g = torch.Generator().manual_seed(2)
BH, Sk, D = 4, 96, 128
cent = torch.tensor(solve_codebook(128, 2)[0], dtype=torch.float32)
k_idx_p = torch.randint(0, 256, (BH, Sk, D // 4), dtype=torch.uint8, generator=g)
k_sg_p = torch.randint(0, 256, (BH, Sk, D // 8), dtype=torch.uint8, generator=g)
k_rn = (torch.rand(BH, Sk, generator=g) * 0.1).half()
k_n = (torch.rand(BH, Sk, generator=g) + 0.5).half()
v_idx_p = torch.randint(0, 256, (BH, Sk, D // 4), dtype=torch.uint8, generator=g)
v_n = (torch.rand(BH, Sk, generator=g) + 0.5).half()
Q = (torch.randn(BH, D, generator=g) * 0.1).half()
Qp = (torch.randn(BH, D, generator=g) * 0.1).half()
cs = math.sqrt(math.pi / 2) / math.sqrt(D)
# exactly the unpacking of the reference's self-check (packed_attention.py:383-390)
k_idx = ref_pa.unpack_2bit(k_idx_p.reshape(-1, D // 4), D).reshape(BH, Sk, D)
k_sg = ref_pa.unpack_1bit(k_sg_p.reshape(-1, D // 8), D).reshape(BH, Sk, D)
v_idx = ref_pa.unpack_2bit(v_idx_p.reshape(-1, D // 4), D).reshape(BH, Sk, D)
K_mse = cent[k_idx.long()] * k_n.unsqueeze(-1)
V_mse = cent[v_idx.long()] * v_n.unsqueeze(-1)
ref = ref_pa.attention_unpacked_ref(Q.float(), Qp.float(), K_mse.float(), k_sg.float() * 2 - 1,
                                    k_rn.float(), V_mse.float(), cs)
out["attn_k_idx"] = k_idx_p.numpy()
out["attn_k_signs_seq"] = k_sg_p.numpy()
out["attn_k_signs_perm"] = ref_pc.permute_signs_for_chunked(k_sg_p).numpy()
out["attn_k_rnorm"] = k_rn.numpy()
out["attn_k_norm"] = k_n.numpy()
out["attn_v_idx"] = v_idx_p.numpy()
out["attn_v_norm"] = v_n.numpy()
out["attn_q"] = Q.numpy()
out["attn_qp"] = Qp.numpy()
out["attn_centroids"] = cent.numpy()
out["attn_corr_scale"] = np.float64(cs)
out["attn_ref_out"] = ref.numpy()

# --- the CPU round trip the reference can run itself (turbo3 + QJL, seed 0) -----------------
torch.manual_seed(0)
K = torch.randn(1024, 128)
V = torch.randn(1024, 128)
q = torch.randn(1, 128)
c, b = make_codebook(128, 3)
cfg = PolarQuantConfig(head_dim=128, bits=3, use_qjl=True)
ck = polarquant_compress(K, c, b, cfg, H)
cv = polarquant_compress(V, c, b, PolarQuantConfig(head_dim=128, bits=3, use_qjl=False), H)
q_rot = q @ H
sm = 1.0 / math.sqrt(128)
cs1 = math.sqrt(math.pi / 2) / 128
o_rot = ref_pa.attention_unpacked_ref(q_rot * sm, q_rot * sm, ck["k_mse_rot"][None], ck["signs"][None],
                                      ck["rot_residual_norm"][None], cv["k_mse_rot"][None], cs1)
out["cfg1_K_head"] = K[:4].numpy()            # spot check that the seeded inputs regenerate
out["cfg1_q"] = q.numpy()
out["cfg1_out"] = (o_rot @ H).numpy()
out["cfg1_k_indices_sum"] = np.int64(ck["indices"].sum().item())
out["cfg1_k_indices"] = ck["indices"].numpy().astype(np.uint8)

np.savez_compressed(os.path.join(here, "reference_vectors.npz"), **out)
print("wrote", os.path.join(here, "reference_vectors.npz"), len(out), "arrays")
