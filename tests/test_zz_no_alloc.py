"""tq_decode_paged_static: decode for hosts that cannot allocate device memory (all HBM already given to
a KV-cache pool, or a binding that owns no device allocator).  Called through the C ABI with ctypes and held
to the output of tq_decode_paged on the same inputs and to the CPU oracle, twice in a row with different
problems so that whatever the first call left in the library's fixed scratch array is there when the second one
runs; the device's free memory and torch's allocator are read before and after to show that nothing was allocated."""
import ctypes
import math

import numpy as np
import pytest
import torch

from oracle import tq_oracle as O
from turboquant.kernels import _native, paged_layout
from turboquant.kernels.paged import CacheFormat, Codebooks

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
SCRATCH_BYTES = 16 * 1024 * 1024


def _bind():
    return _native.lib()          # declares the argument types of both decode entry points


def _problem(seed, lens, Hq, Hkv, fmt):
    g = torch.Generator().manual_seed(seed)
    bs = 16
    lens = torch.tensor(lens, dtype=torch.int32)
    ns = len(lens)
    max_blocks = (int(lens.max()) + bs - 1) // bs
    nb = ns * max_blocks
    f = {"k_idx": torch.randint(0, 1 << fmt.k_bits, (nb, bs, Hkv, 128), generator=g, dtype=torch.uint8),
         "v_idx": torch.randint(0, 1 << fmt.v_bits, (nb, bs, Hkv, 128), generator=g, dtype=torch.uint8),
         "k_norm": (torch.rand(nb, bs, Hkv, generator=g) * 4 + 8).half(),
         "v_norm": (torch.rand(nb, bs, Hkv, generator=g) * 4 + 8).half(),
         "k_signs": torch.randint(0, 2, (nb, bs, Hkv, 128), generator=g, dtype=torch.uint8),
         "k_rnorm": (torch.rand(nb, bs, Hkv, generator=g) * 3).half()}
    cache = paged_layout.pack_cache(f, bs, fmt.k_bits, fmt.v_bits, fmt.use_qjl).to(DEV)
    bt = torch.randperm(nb, generator=g).reshape(ns, max_blocks).to(torch.int32).to(DEV)
    q = torch.randn(ns, Hq, 128, generator=g).half().to(DEV)
    return cache, bt, lens.to(DEV), q, nb, max_blocks, f


def _call(L, static, out, q, cache, bt, lens, books, fmt, nb, max_pages, chunk_pages, ws=None):
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    ns, Hq, _ = q.shape
    Hkv = cache.shape[1]
    head = (p(out), p(q), ctypes.c_void_p(0), 0, p(cache), nb, 16, p(bt), bt.stride(0), p(lens), p(books.kc), p(books.vc),
            1 / math.sqrt(128), math.sqrt(math.pi / 2) / 128, 0.0)
    tail = (ctypes.c_void_p(0), ctypes.c_void_p(0), ns, Hq, Hkv, max_pages, fmt.k_bits, fmt.v_bits, int(fmt.use_qjl),
            chunk_pages, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    if static:
        return L.tq_decode_paged_static(*head, *tail)
    return L.tq_decode_paged(*head, p(ws), ws.numel(), *tail)


def test_static_scratch_decode_matches_workspace_decode_twice():
    L = _bind()
    fmt = CacheFormat.named("turbo3")
    books = Codebooks(fmt, DEV)
    # two different problems back to back: many chunks per sequence, so the split-K partials really go
    # through the scratch, and the second problem is smaller so stale partials of the first stay behind it
    for seed, lens, Hq, Hkv, chunk in ((1, [900, 333, 64, 1], 16, 2, 4), (2, [130, 700], 8, 1, 7)):
        cache, bt, lens_d, q, nb, max_blocks, f = _problem(seed, lens, Hq, Hkv, fmt)
        need = L.tq_decode_workspace_bytes(len(lens), Hq, Hkv, max_blocks, chunk)
        assert 0 < need <= SCRATCH_BYTES
        ws = torch.empty(need, dtype=torch.uint8, device=DEV)
        ref = torch.empty_like(q)
        got = torch.empty_like(q)
        assert _call(L, False, ref, q, cache, bt, lens_d, books, fmt, nb, max_blocks, chunk, ws) == 0
        # the entry point's first call on a device looks up the scratch array's address (and the driver may load
        # the kernels' module then): measure around a call made after that
        assert _call(L, True, got, q, cache, bt, lens_d, books, fmt, nb, max_blocks, chunk) == 0
        torch.cuda.synchronize()
        got.zero_()
        free_before, torch_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        assert _call(L, True, got, q, cache, bt, lens_d, books, fmt, nb, max_blocks, chunk) == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before and torch.cuda.memory_allocated() == torch_before
        assert torch.isfinite(got.float()).all()
        d = (got.float() - ref.float()).abs()
        # the same kernels run on the same data: the tests' attention tolerance, in practice identical
        assert (d - 1e-2 * ref.float().abs()).max().item() <= 2e-3
        assert torch.equal(got, ref)
        # and against the CPU oracle on the same logical cache contents
        kf = {"idx": f["k_idx"].numpy(), "norm": f["k_norm"].float().numpy(), "signs": f["k_signs"].numpy(),
              "rnorm": f["k_rnorm"].float().numpy()}
        vf = {"idx": f["v_idx"].numpy(), "norm": f["v_norm"].float().numpy()}
        want = O.paged_decode(q.float().cpu().numpy(), q.float().cpu().numpy(), kf, vf, bt.cpu().numpy(),
                              np.asarray(lens), books.kc.cpu().numpy(), books.vc.cpu().numpy(), 1 / math.sqrt(128),
                              math.sqrt(math.pi / 2) / 128, 16)
        dd = np.abs(got.float().cpu().numpy() - want)
        assert (dd - 1e-2 * np.abs(want)).max() <= 2e-3


def test_static_scratch_refuses_what_does_not_fit():
    L = _bind()
    fmt = CacheFormat.named("turbo3")
    books = Codebooks(fmt, DEV)
    cache, bt, lens_d, q, nb, max_blocks, _ = _problem(3, [64, 64], 8, 1, fmt)
    out = torch.empty_like(q)
    # claim a problem whose partials exceed the 16 MiB array: refused before any launch, output untouched
    out.fill_(7.0)
    big_pages = 1 << 20
    assert L.tq_decode_workspace_bytes(2, 8, 1, big_pages, 1) > SCRATCH_BYTES
    rc = _call(L, True, out, q, cache, bt, lens_d, books, fmt, nb, big_pages, 1)
    torch.cuda.synchronize()
    assert rc == -4
    assert (out == 7.0).all()
