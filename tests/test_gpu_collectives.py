"""Arithmetic of the fused collectives with all replicas emulated on one GPU.

Kernels that wait on one another never share a GPU, so the emulation runs the
kernel once per replica, one after the other, with the cross-GPU barrier off;
slice ownership makes that order-independent.  The barrier itself is checked
with a flag that nothing sets: the wait must run out and report a status.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("R", [1, 2, 4, 8])
def test_outer_sync_matches_torch_sgd(R):
    from diloco_swarm_b200.ops._lib import check, cuda_lib, stream_ptr
    from diloco_swarm_b200.parallel.collectives import shard_size
    from diloco_swarm_b200.parallel.symm import LocalPeerSet
    n = 1 << 18
    lr, mu = 0.7, 0.9
    torch.manual_seed(R)
    theta_g = torch.randn(n, device=DEV)
    ref_p = torch.nn.Parameter(theta_g.clone())
    opt = torch.optim.SGD([ref_p], lr=lr, momentum=mu, nesterov=True)
    shard = shard_size(n, R, 4)
    tg_sh = [torch.zeros(shard, device=DEV) for _ in range(R)]
    for r in range(R):
        part = theta_g[r * shard:(r + 1) * shard]
        tg_sh[r][:part.numel()] = part
    mom_sh = [torch.zeros(shard, device=DEV) for _ in range(R)]
    for outer in range(3):
        locals_ = [ref_p.data.clone() + 1e-2 * torch.randn(n, device=DEV) for _ in range(R)]
        # reference: average pseudo-gradient, torch SGD-Nesterov
        ref_p.grad = torch.stack([ref_p.data - t for t in locals_]).mean(0)
        opt.step()
        peers = LocalPeerSet(locals_)
        for r in range(R):
            check(cuda_lib().dsw_outer_sync(peers.table, None, tg_sh[r].data_ptr(), mom_sh[r].data_ptr(), n, shard, r, R,
                                            lr, mu, 1, 1, 0, 0, 0, None, stream_ptr()), "outer")
        torch.cuda.synchronize()
        for t in locals_:
            assert torch.allclose(t, ref_p.data, atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("R", [2, 4])
@pytest.mark.parametrize("bf16", [False, True])
def test_grad_allreduce(R, bf16):
    from diloco_swarm_b200.ops._lib import check, cuda_lib, stream_ptr
    from diloco_swarm_b200.parallel.collectives import shard_size
    from diloco_swarm_b200.parallel.symm import LocalPeerSet
    n, off, cnt = 1 << 16, 1024, 40000
    grads = [torch.randn(n, device=DEV) for _ in range(R)]
    ref = torch.stack(grads).mean(0)
    orig = [g.clone() for g in grads]
    shard = shard_size(cnt, R, 8)
    if bf16:
        stage = [torch.zeros(n, dtype=torch.bfloat16, device=DEV) for _ in range(R)]
        peers = LocalPeerSet(stage)
        for phase in (1, 2, 4):       # cast-in on all, reduce on all, widen on all
            for r in range(R):
                check(cuda_lib().dsw_grad_allreduce(peers.table, None, grads[r].data_ptr(), off, cnt, shard, r, R, 1, 1,
                                                    0, 0, phase, 0, None, stream_ptr()), "grad")
        tol = 2e-2
    else:
        peers = LocalPeerSet(grads)
        for r in range(R):
            check(cuda_lib().dsw_grad_allreduce(peers.table, None, grads[r].data_ptr(), off, cnt, shard, r, R, 0, 1, 0, 0,
                                                7, 0, None, stream_ptr()), "grad")
        tol = 1e-6
    torch.cuda.synchronize()
    for g, o in zip(grads, orig):
        assert torch.allclose(g[off:off + cnt], ref[off:off + cnt], atol=tol, rtol=tol)
        assert torch.equal(g[:off], o[:off]) and torch.equal(g[off + cnt:], o[off + cnt:])


def test_peer_wait_runs_out_and_reports():
    """R=2 but only one replica launches: its wait for the peer's flag must end
    by itself within the (short) limit and leave ST_PEER_TIMEOUT in the status
    word; the context stays usable."""
    from diloco_swarm_b200.ops._lib import Status, check, cuda_lib, stream_ptr
    from diloco_swarm_b200.parallel.symm import FLAG_WORDS, LocalPeerSet
    n = 4096
    bufs = [torch.ones(n, device=DEV), torch.ones(n, device=DEV)]
    flags = [torch.zeros(FLAG_WORDS, dtype=torch.int32, device=DEV) for _ in range(2)]
    st = Status(torch.device(DEV))
    tg, mom = torch.zeros(n // 2, device=DEV), torch.zeros(n // 2, device=DEV)
    check(cuda_lib().dsw_outer_sync(LocalPeerSet(bufs).table, LocalPeerSet(flags).table, tg.data_ptr(), mom.data_ptr(),
                                    n, n // 2, 0, 2, 0.7, 0.9, 1, 1, 20_000_000, 1, 4, st.ptr, stream_ptr()), "outer")
    torch.cuda.synchronize()
    assert st.read() == 2
    assert torch.equal(bufs[0], torch.ones(n, device=DEV))      # nothing was written
    assert float((torch.ones(4, device=DEV) * 2).sum()) == 8.0   # context still works
