"""The allocation-free LayerNorm backward against the normal entry point.

Some callers of this library cannot allocate device memory: code running inside
another framework's memory pool, latency-critical loops that
must stay off the allocator, processes at the edge of a shared GPU's memory.
``dsw_layernorm_bwd_noalloc`` serves them with a scratch array built into the
library.  The test calls it through its exported C symbol (ctypes, no wrapper),
twice in a row so that the second call sees the first call's leftovers in the
shared array, and compares every output with ``dsw_layernorm_bwd`` given a
fresh scratch tensor.  It also checks that a row width beyond the built-in
limit is refused.  The file name sorts last on purpose: a run that stops at the
first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from diloco_swarm_b200.ops import _build
    lib = ctypes.CDLL(_build.build_cuda())      # rebuilt first when a source is newer
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.dsw_layernorm_bwd_noalloc.restype = ci
    lib.dsw_layernorm_bwd_noalloc.argtypes = [vp] * 10 + [ci, ci, vp]
    lib.dsw_layernorm_bwd.restype = ci
    lib.dsw_layernorm_bwd.argtypes = [vp] * 11 + [ci, ci, vp]
    lib.dsw_layernorm_bwd_blocks.restype = ci
    lib.dsw_layernorm_bwd_blocks.argtypes = [ci]
    return lib


def _case(M, d, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)
    x = (r(M, d) * 2 + 0.3).to(torch.bfloat16)
    dy, dres = r(M, d).to(torch.bfloat16), r(M, d).to(torch.bfloat16)
    gamma = r(d)
    mean = x.float().mean(1)
    rstd = (x.float().var(1, unbiased=False) + 1e-5).rsqrt()
    return x, dy, dres, gamma, mean, rstd


@pytest.mark.parametrize("M,d", [(1000, 768), (4096, 1024)])
def test_noalloc_matches_regular_twice(M, d):
    lib = _lib()
    st = torch.cuda.current_stream().cuda_stream
    for call in range(2):                       # second call reuses the shared array
        x, dy, dres, gamma, mean, rstd = _case(M, d, seed=call)
        outs = []
        for variant in ("regular", "noalloc"):
            dx = torch.empty_like(x)
            dg, db, ds = (torch.full((d,), 0.5, device="cuda") for _ in range(3))
            if variant == "regular":
                scratch = torch.empty(lib.dsw_layernorm_bwd_blocks(M) * 3 * d, device="cuda")
                rc = lib.dsw_layernorm_bwd(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                                           rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(), dg.data_ptr(),
                                           db.data_ptr(), ds.data_ptr(), scratch.data_ptr(), M, d, st)
            else:
                rc = lib.dsw_layernorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                                                   rstd.data_ptr(), dres.data_ptr(), dx.data_ptr(), dg.data_ptr(),
                                                   db.data_ptr(), ds.data_ptr(), M, d, st)
            assert rc == 0, f"{variant} returned {rc}"
            torch.cuda.synchronize()
            outs.append((dx.float(), dg, db, ds))
        for a, b in zip(*outs):
            assert torch.allclose(a, b, rtol=2e-2, atol=1e-3 * float(a.abs().max()) + 1e-6)
        assert torch.isfinite(outs[1][1]).all() and float(outs[1][1].abs().max()) > 0.5


def test_noalloc_rejects_rows_wider_than_the_limit():
    lib = _lib()
    M, d = 8, 4096
    x, dy, dres, gamma, mean, rstd = _case(M, d, seed=3)
    dx = torch.zeros_like(x)
    dg = torch.zeros(d, device="cuda")
    rc = lib.dsw_layernorm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                       None, dx.data_ptr(), dg.data_ptr(), None, None, M, d,
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == -21
    torch.cuda.synchronize()
    assert float(dx.float().abs().max()) == 0.0      # nothing ran
