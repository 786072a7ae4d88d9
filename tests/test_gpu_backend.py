"""The vLLM attention implementation end to end on a GPU, with hand-built layer and metadata objects.

Follows the reference's hook (turboquant/integration/tq_fp4_backend.py: do_kv_cache_update :456-484,
forward :488-643 with its prefill :532-553 and decode :604-641 branches): a prefill step writes the packed
cache and attends over the raw K/V, a decode step appends one token per sequence and attends over the packed
cache, a mixed step does both.  Decode rows are held to the CPU oracle's round trip in original space
(compress with the reference arithmetic, asymmetric score, de-rotation), prefill rows to plain causal attention.
"""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from oracle import tq_oracle as O
from turboquant.integration import tq_b200_backend as B
from turboquant.integration import vllm_backend as VB
from turboquant.kernels import _native

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HQ, HKV, BS = 16, 4, 16
SCALE = 1 / math.sqrt(128)


def _close(got, ref):
    got, ref = np.asarray(got, np.float32), np.asarray(ref, np.float32)
    d = np.abs(got - ref)
    assert np.isfinite(got).all()
    assert (d - 1e-2 * np.abs(ref)).max() <= 2e-3, f"max abs diff {d.max():.3e}"
    assert np.linalg.norm(got - ref) <= 1e-2 * np.linalg.norm(ref) + 1e-6


def _causal_ref(q, k, v):
    """Plain causal attention in fp32: q [T, Hq, 128], k / v [T, Hkv, 128]."""
    T = q.shape[0]
    g = HQ // HKV
    out = np.zeros((T, HQ, 128), np.float32)
    mask = np.tril(np.ones((T, T), bool))
    for h in range(HQ):
        s = (q[:, h] @ k[:, h // g].T) * SCALE
        s = np.where(mask, s, -np.inf)
        p = np.exp(s - s.max(-1, keepdims=True))
        out[:, h] = (p / p.sum(-1, keepdims=True)) @ v[:, h // g]
    return out


def _oracle_decode_row(q_row, K, V, books):
    """Reference CPU path for one sequence: K / V [L, Hkv, 128] fp32 (fp16-rounded values), q_row [Hq, 128];
    returns [Hq, 128] in original space.  Norms are stored as fp16 in the cache, the rotated query is fp16."""
    H = O.make_wht_matrix(128)
    L = K.shape[0]
    kc, kb = books.kc.cpu().numpy(), books.kb.cpu().numpy()
    vc, vb = books.vc.cpu().numpy(), books.vb.cpu().numpy()
    h16 = lambda a: a.astype(np.float16).astype(np.float32)
    kf = {"idx": np.zeros((1, L, HKV, 128), np.int64), "norm": np.zeros((1, L, HKV), np.float32),
          "signs": np.zeros((1, L, HKV, 128), np.uint8), "rnorm": np.zeros((1, L, HKV), np.float32)}
    vf = {"idx": np.zeros((1, L, HKV, 128), np.int64), "norm": np.zeros((1, L, HKV), np.float32)}
    for h in range(HKV):
        ck = O.polarquant_compress(K[:, h], kc, kb, 3, True, H)
        cv = O.polarquant_compress(V[:, h], vc, vb, 3, False, H)
        kf["idx"][0, :, h], kf["norm"][0, :, h] = ck["indices"], h16(ck["norms"])
        kf["signs"][0, :, h], kf["rnorm"][0, :, h] = ck["signs"] > 0, h16(ck["rot_residual_norm"])
        vf["idx"][0, :, h], vf["norm"][0, :, h] = cv["indices"], h16(cv["norms"])
    q_rot = h16(q_row.astype(np.float32) @ H)[None]
    out_rot = O.paged_decode(q_rot, q_rot, kf, vf, np.zeros((1, 1), np.int64), np.array([L]), kc, vc, SCALE,
                             math.sqrt(math.pi / 2) / 128, L)
    return out_rot[0] @ H


class _Engine:
    """What the engine would hold: the packed cache, a block table per sequence, the raw K/V history (for the oracle)."""

    def __init__(self, impl, nb=96):
        self.impl = impl
        self.layer = SimpleNamespace(layer_name="model.layers.5.self_attn.attn")
        self.cache = torch.zeros(B.kv_cache_shape(nb, BS, HKV, 128, impl.format), dtype=torch.uint8, device=DEV)
        self.free = torch.randperm(nb, generator=torch.Generator().manual_seed(3)).tolist()
        self.tables, self.K, self.V = {}, {}, {}
        self.gen = torch.Generator().manual_seed(17)

    def _slots(self, sid, start, n):
        tab = self.tables.setdefault(sid, [])
        while len(tab) * BS < start + n:
            tab.append(self.free.pop())
        pos = torch.arange(start, start + n)
        return torch.tensor(tab)[pos // BS] * BS + pos % BS

    def step(self, requests):
        """requests: [(sequence id, number of new tokens)].  Runs cache update + forward; returns (out, q, k, v, md)."""
        qs, ks, vs, slots, starts, lens = [], [], [], [], [0], []
        for sid, n in requests:
            old = 0 if sid not in self.K else self.K[sid].shape[0]
            k = torch.randn(n, HKV, 128, generator=self.gen).half()
            v = torch.randn(n, HKV, 128, generator=self.gen).half()
            k[..., [5, 50, 90, 127]] *= 10
            self.K[sid] = k if old == 0 else torch.cat([self.K[sid], k])
            self.V[sid] = v if old == 0 else torch.cat([self.V[sid], v])
            qs.append(torch.randn(n, HQ, 128, generator=self.gen).half())
            ks.append(k)
            vs.append(v)
            slots.append(self._slots(sid, old, n))
            starts.append(starts[-1] + n)
            lens.append(old + n)
        q, k, v = torch.cat(qs), torch.cat(ks), torch.cat(vs)
        T = q.shape[0]
        width = max(len(self.tables[sid]) for sid, _ in requests) + 5      # wider than any sequence needs
        bt = torch.zeros(len(requests), width, dtype=torch.int32)
        for i, (sid, _) in enumerate(requests):
            bt[i, :len(self.tables[sid])] = torch.tensor(self.tables[sid], dtype=torch.int32)
        md = SimpleNamespace(num_actual_tokens=T, max_query_len=max(n for _, n in requests), max_seq_len=max(lens),
                             block_table=bt.to(DEV), seq_lens=torch.tensor(lens, dtype=torch.int32, device=DEV),
                             query_start_loc=torch.tensor(starts, dtype=torch.int32, device=DEV))
        pad = 3                                                              # the engine pads its buffers
        query = torch.zeros(T + pad, HQ * 128, dtype=torch.float16, device=DEV)
        query[:T] = q.reshape(T, -1).to(DEV)
        output = torch.full((T + pad, HQ * 128), 9.0, dtype=torch.float16, device=DEV)
        slot_map = torch.cat([torch.cat(slots), torch.full((pad,), -1, dtype=torch.int64)]).to(DEV)
        self.impl.do_kv_cache_update(self.layer, k.to(DEV), v.to(DEV), self.cache, slot_map)
        res = self.impl.forward(self.layer, query, k.reshape(T, -1).to(DEV), v.reshape(T, -1).to(DEV), self.cache, md,
                                output=output)
        torch.cuda.synchronize()
        assert res is output and _native.read_status(DEV) == 0
        assert (output[T:] == 9.0).all()                                     # rows past num_actual_tokens untouched
        return output[:T].view(T, HQ, 128).float().cpu().numpy(), q.float().numpy(), starts


@pytest.fixture
def impl(monkeypatch):
    pytest.importorskip("vllm")
    monkeypatch.setenv("TQ_B200_FORMAT", "turbo3")
    monkeypatch.setattr(VB, "_config", VB.TurboQuantConfig(128, num_layers=40, k_bits=3, v_bits=3, use_qjl=True))
    return B.TurboQuantB200Impl(HQ, 128, SCALE, HKV)


def test_impl_prefill_decode_and_mixed_steps(impl):
    eng = _Engine(impl)
    books = impl.config.get_state(5, torch.device(DEV)).books
    # step 1: two fresh prefills
    out, q, st = eng.step([("a", 300), ("b", 77)])
    for sid, (lo, hi) in (("a", (st[0], st[1])), ("b", (st[1], st[2]))):
        _close(out[lo:hi], _causal_ref(q[lo:hi], eng.K[sid].float().numpy(), eng.V[sid].float().numpy()))
    # step 2: pure decode, one new token per sequence, attention over the packed cache
    out, q, st = eng.step([("a", 1), ("b", 1)])
    for i, sid in enumerate(("a", "b")):
        _close(out[i], _oracle_decode_row(q[i], eng.K[sid].float().numpy(), eng.V[sid].float().numpy(), books))
    # step 3: a running decode mixed with a new prefill and a one-token sequence
    out, q, st = eng.step([("a", 1), ("c", 40), ("b", 1), ("d", 1)])
    _close(out[0], _oracle_decode_row(q[0], eng.K["a"].float().numpy(), eng.V["a"].float().numpy(), books))
    _close(out[st[1]:st[2]], _causal_ref(q[st[1]:st[2]], eng.K["c"].float().numpy(), eng.V["c"].float().numpy()))
    _close(out[st[2]], _oracle_decode_row(q[st[2]], eng.K["b"].float().numpy(), eng.V["b"].float().numpy(), books))
    _close(out[st[3]:st[4]], _causal_ref(q[st[3]:st[4]], eng.K["d"].float().numpy(), eng.V["d"].float().numpy()))
    # step 4: the sequence prefilled inside the mixed step decodes from the packed cache
    out, q, st = eng.step([("c", 1)])
    _close(out[0], _oracle_decode_row(q[0], eng.K["c"].float().numpy(), eng.V["c"].float().numpy(), books))


def test_impl_rejects_extends_and_protected_layers(impl):
    eng = _Engine(impl)
    eng.step([("a", 20)])
    with pytest.raises(NotImplementedError):
        eng.step([("a", 5)])                       # five more tokens over cached context: an extend
    eng2 = _Engine(B.TurboQuantB200Impl(HQ, 128, SCALE, HKV))      # an implementation object belongs to one layer
    eng2.layer = SimpleNamespace(layer_name="model.layers.0.self_attn.attn")      # first of 40 layers: protected
    with pytest.raises(NotImplementedError):
        eng2.step([("x", 8)])
    assert impl.config.get_state(39, torch.device(DEV)) is None
