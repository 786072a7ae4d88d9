"""Serving hooks: layer gating and per-layer state keep the reference's behaviour
(tests/test_boundary_protection.py and tests/test_asymmetric_kv.py of the reference), cache shapes follow the format."""
import pytest
import torch

from turboquant.core.quantizer import PolarQuantConfig
from turboquant.integration import tq_b200_backend as B
from turboquant.integration.vllm_backend import TurboQuantFP8Config, TurboQuantFP8State, get_tq_fp8_config


def test_boundary_layers_are_protected():
    cfg = TurboQuantFP8Config(head_size=128, num_layers=40, protect_boundary_layers=True, num_protected_layers=2)
    assert [i for i in range(40) if not cfg.should_compress(i)] == [0, 1, 38, 39]
    dev = torch.device("cpu")
    assert cfg.get_state(0, dev) is None and cfg.get_state(39, dev) is None
    st = cfg.get_state(5, dev)
    assert st is not None and st.layer_idx == 5 and cfg.get_state(5, dev) is st       # cached per layer
    assert all(TurboQuantFP8Config(num_layers=40, protect_boundary_layers=False).should_compress(i) for i in range(40))
    assert all(TurboQuantFP8Config(num_layers=0).should_compress(i) for i in range(40))
    # the two gates agree
    pq = PolarQuantConfig(num_layers=40)
    assert all(pq.should_compress(i) == cfg.should_compress(i) for i in range(40))


def test_asymmetric_state():
    st = TurboQuantFP8State(head_size=128, layer_idx=5, device=torch.device("cpu"), k_bits=4, v_bits=2)
    assert len(st.k_centroids) == 16 and len(st.v_centroids) == 4
    assert len(st.k_boundaries) == 15 and len(st.v_boundaries) == 3
    assert st.format.page_bytes == 16 * 100 and not st.use_qjl
    sym = TurboQuantFP8State(head_size=128, layer_idx=5, device=torch.device("cpu"), k_bits=4, v_bits=4)
    assert sym.k_centroids is sym.v_centroids
    t3 = TurboQuantFP8State(head_size=128, layer_idx=1, device=torch.device("cpu"), k_bits=3)
    assert t3.use_qjl and t3.format.page_bytes == 1888
    with pytest.raises(ValueError):
        TurboQuantFP8State(head_size=64, layer_idx=0, device=torch.device("cpu"))


def test_singleton_config():
    a = get_tq_fp8_config(num_layers=12, k_bits=3)
    assert get_tq_fp8_config(num_layers=99) is a and a.num_layers == 12


def test_cache_shape_and_format_env(monkeypatch):
    monkeypatch.setenv("TQ_B200_FORMAT", "turbo3")
    assert B.kv_cache_shape(10, 16, 8, 128) == (10, 8, 1888)
    assert B.kv_cache_shape(10, 32, 4, 128) == (10, 4, 2 * 1888)
    monkeypatch.setenv("TQ_B200_FORMAT", "turbo4")
    assert B.kv_cache_shape(3, 16, 2, 128) == (3, 2, 2112)
    with pytest.raises(ValueError):
        B.kv_cache_shape(3, 24, 2, 128)
    with pytest.raises(ValueError):
        B.kv_cache_shape(3, 16, 2, 64)


def test_vllm_backend_registers_under_custom():
    pytest.importorskip("vllm")
    from vllm.v1.attention.backends.registry import AttentionBackendEnum
    Bk = B.TurboQuantB200Backend
    assert Bk.get_name() == "CUSTOM" and Bk.get_supported_kernel_block_sizes() == [16, 32]
    assert Bk.forward_includes_kv_cache_update is False and Bk.accept_output_buffer is True
    B.register()
    assert AttentionBackendEnum.CUSTOM.get_class() is Bk
    impl = Bk.get_impl_cls()(32, 128, 0.088, 8)
    assert impl.fused_rope_kvcache_supported() is False
    with pytest.raises(NotImplementedError):
        Bk.get_impl_cls()(32, 128, 0.088, 8, sliding_window=128)


def test_split_batch_sorts_decodes_prefills_and_refuses_extends():
    """One step of a v1 engine mixes running decodes with new prefills (the reference splits by
    num_decodes / num_prefills, tq_fp4_backend.py:517-530)."""
    # requests: decode (len 301), prefill of 40, decode (len 78), one-token sequence, padding request
    qsl = [0, 1, 41, 42, 43, 43]
    lens = [301, 40, 78, 1, 0]
    dec, pre = B.split_batch(qsl, lens)
    assert dec == [(0, 0), (2, 41)]
    assert pre == [(1, 1, 41), (3, 42, 43)]
    assert B.split_batch([0, 1, 2], [9, 10]) == ([(0, 0), (1, 1)], [])
    with pytest.raises(NotImplementedError):
        B.split_batch([0, 5], [25])            # five new tokens over twenty cached ones
