"""The stand-ins for a memory sanitizer: canary words around symmetric buffers and the bounds-checking
build of the kernel library (-DDSWARM_BOUNDS).  Nothing here makes a kernel touch memory it should not:
the canary test overwrites a guard zone from the host through the buffer's own allocation, and the bounds
build's self-test fails a check without any memory access."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_canaries_around_a_symmetric_buffer():
    from diloco_swarm_b200.parallel.symm import CANARY, GUARD_BYTES, CanaryError, SymmetricBuffer
    dev = torch.device("cuda", 0)
    buf = SymmetricBuffer(1000, dev)
    assert buf.ptr % 256 == 0 and buf.nbytes == 1024
    buf.view(torch.float32, 250).fill_(3.0)                  # the whole payload
    buf.check_canaries()
    assert int(buf._whole[0]) == CANARY and int(buf._whole[-1]) == CANARY
    buf._whole[GUARD_BYTES + buf.nbytes + 5] = 0             # what a stray store behind the buffer would leave
    with pytest.raises(CanaryError, match="behind"):
        buf.check_canaries()
    buf._whole[GUARD_BYTES + buf.nbytes + 5] = CANARY
    buf._whole[GUARD_BYTES - 1] = 1
    with pytest.raises(CanaryError, match="in front of"):
        buf.check_canaries()
    buf._whole[GUARD_BYTES - 1] = CANARY
    buf.close()


def test_engine_step_leaves_every_canary_intact(monkeypatch):
    monkeypatch.setenv("DSWARM_CANARY_CHECK", "1")
    from helpers import make_config, single_world
    from diloco_swarm_b200.models.engine_b200 import B200Engine
    from diloco_swarm_b200.models.gpt2 import GPT2Config
    cfg = make_config(train={"outer_optimizer": {"type": "SGD", "lr": 0.7, "nesterov": True}})
    mc = cfg.model
    eng = B200Engine(GPT2Config(block_size=mc.block_size, vocab_size=mc.vocab_size, n_layer=mc.n_layer, n_head=mc.n_head,
                                n_embd=mc.n_embd), single_world(), cfg, torch.device("cuda", 0))
    ids = torch.randint(0, 500, (4, 65), device="cuda")
    mask = torch.ones(4, 64, dtype=torch.long, device="cuda")
    for _ in range(2):
        eng.forward_backward(0, ids[:, :-1].contiguous(), None, ids[:, 1:].contiguous(), mask, 1.0)
        eng.optimizer_step(1e-3, 1.0)
    eng.outer_step()
    torch.cuda.synchronize()
    eng.check_status()                                        # includes the canaries with DSWARM_CANARY_CHECK=1
    assert len(eng.symmetric_buffers()) >= 2


_BOUNDS_SCRIPT = r"""
import ctypes, torch
from diloco_swarm_b200.ops import kernels as K
from diloco_swarm_b200.ops._lib import cuda_lib, stream_ptr
lib = cuda_lib()
status = lib.dsw_bounds_status
status.restype, status.argtypes = ctypes.c_int, []
selftest = lib.dsw_bounds_selftest
selftest.restype, selftest.argtypes = ctypes.c_int, [ctypes.c_void_p]
assert status() == 0
bf = lambda *s: (torch.randn(*s, device="cuda") * 0.1).to(torch.bfloat16)
# tail shapes of every kernel family with checks compiled in
for M, N, Kd in ((200, 264, 200), (129, 136, 72)):
    a, b, bias, res = bf(M, Kd), bf(N, Kd), torch.randn(N, device="cuda"), bf(M, N)
    for bn in (128, 256, 512):
        K.gemm(a, b, bias=bias, bn=bn)
        K.gemm(a, b, bias=bias, mode=K.EPI_RESID, resid=res, bn=bn)
        K.gemm(a, b, bias=bias, mode=K.EPI_GELU, aux_out=torch.empty_like(res), bn=bn)
        K.gemm(a, b, mode=K.EPI_MUL, aux_in=res, bn=bn)
        K.gemm(a, b, mode=K.EPI_STORE_F32, bn=bn)
for M, d in ((37, 72), (130, 768), (64, 1032)):
    x, g, be = bf(M, d), torch.randn(d, device="cuda"), torch.randn(d, device="cuda")
    y, mean, rstd = K.layernorm_fwd(x, g, be)
    dg, db, ds = (torch.zeros(d, device="cuda") for _ in range(3))
    K.layernorm_bwd(bf(M, d), x, g, mean, rstd, dg, db, dres=bf(M, d), dres_sum=ds)
    K.colsum_accum(x, ds)
n = 1000 * 8 + 3
p, gr, m, v = (torch.randn(n, device="cuda") for _ in range(4))
v.abs_()
K.adamw_step(p, gr, m, v, torch.empty(n, dtype=torch.bfloat16, device="cuda"), 1e-3, (0.9, 0.95), 1e-8, 0.1, 1,
             torch.ones(4, device="cuda"))
logits, tg = bf(33, 504), torch.randint(0, 504, (33,), device="cuda")
K.cross_entropy(logits, tg, None, 1.0, torch.zeros((), device="cuda"), torch.zeros(1, device="cuda"))
torch.cuda.synchronize()
assert status() == 0, "a bounds check failed on a valid call"
assert selftest(stream_ptr()) == 1
torch.cuda.synchronize()
code = status()
assert code // 100000 == 1 and code % 100000 > 0, code      # reported by elementwise.cu with its source line
assert status() == 0                                         # reading clears it
print("bounds build ok", code)
"""


def test_bounds_build_runs_clean_and_reports():
    """The kernels of the bounds build on tail shapes: no check fails; the self-test's deliberate failure (a
    check with no memory access behind it) is reported with its unit and source line, and reading clears it."""
    env = dict(os.environ, DSWARM_LIB_VARIANT="bounds")
    p = subprocess.run([sys.executable, "-c", _BOUNDS_SCRIPT], cwd=ROOT, env=env, capture_output=True, text=True,
                       timeout=900)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-4000:]
    assert "bounds build ok" in p.stdout
