"""tcgen05 GEMM against a plain fp32 PyTorch matmul of the same bf16 inputs."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mk(shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


def _close(out, ref, what):
    out, ref = out.float(), ref.float()
    err = (out - ref).abs().max().item()
    tol = 2e-2 * ref.abs().max().item() + 1e-3
    assert err <= tol, f"{what}: max abs err {err} > {tol}"


SHAPES = [(128, 256, 64), (256, 512, 768), (200, 264, 200), (1024, 768, 3072), (384, 2304, 768), (129, 136, 72)]


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("bn", [128, 256, 512])
def test_gemm_nt(M, N, K, bn):
    from diloco_swarm_b200.ops import kernels as Kn
    from diloco_swarm_b200.ops._lib import Status
    st = Status(torch.device("cuda"))
    a, b = _mk((M, K), seed=1), _mk((N, K), seed=2)
    out = Kn.gemm(a, b, bn=bn, status=st)
    torch.cuda.synchronize()
    st.raise_if_set()
    _close(out, a.float() @ b.float().t(), f"NT {M}x{N}x{K} bn{bn}")


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_nn_dgrad(M, N, K):
    """A K-major, B [K,N] N-major (dx = dy @ W)."""
    from diloco_swarm_b200.ops import kernels as Kn
    from diloco_swarm_b200.ops._lib import Status
    st = Status(torch.device("cuda"))
    a, b = _mk((M, K), seed=3), _mk((K, N), seed=4)
    for bn in (256, 512):
        out = Kn.gemm(a, b, b_t=False, bn=bn, status=st)
        torch.cuda.synchronize()
        st.raise_if_set()
        _close(out, a.float() @ b.float(), f"NN {M}x{N}x{K} bn{bn}")


@pytest.mark.parametrize("M,N,K", SHAPES[:-1] + [(136, 136, 72)])
@pytest.mark.parametrize("split", [1, 3])
def test_gemm_tn_wgrad(M, N, K, split):
    """A [K,M] M-major, B [K,N] N-major, fp32 accumulate (dW += dy^T @ x)."""
    from diloco_swarm_b200.ops import kernels as Kn
    from diloco_swarm_b200.ops._lib import Status
    st = Status(torch.device("cuda"))
    a, b = _mk((K, M), seed=5), _mk((K, N), seed=6)
    base = torch.randn(M, N, device="cuda")
    for bn in (256, 512):
        out = base.clone()
        Kn.gemm(a, b, a_t=True, b_t=False, mode=Kn.EPI_ATOMIC_F32, out=out, split_k=split, bn=bn, status=st)
        torch.cuda.synchronize()
        st.raise_if_set()
        _close(out, base + a.float().t() @ b.float(), f"TN {M}x{N}x{K} split{split} bn{bn}")


def test_gemm_epilogues():
    from diloco_swarm_b200.ops import kernels as Kn
    M, N, K = 512, 768, 256
    a, b = _mk((M, K), seed=7), _mk((N, K), 0.05, seed=8)
    bias = torch.randn(N, device="cuda")
    acc = a.float() @ b.float().t() + bias
    out = Kn.gemm(a, b, bias=bias)
    _close(out, acc, "bias")
    dg = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    out = Kn.gemm(a, b, mode=Kn.EPI_GELU, bias=bias, aux_out=dg)
    xg = acc.clone().requires_grad_(True)
    torch.nn.functional.gelu(xg).sum().backward()
    _close(dg, xg.grad, "gelu derivative")
    _close(out, torch.nn.functional.gelu(acc), "gelu")
    _close(Kn.gemm(a, b, mode=Kn.EPI_GELU, bias=bias), torch.nn.functional.gelu(acc), "gelu without the derivative")
    res = _mk((M, N), seed=9)
    out = Kn.gemm(a, b, mode=Kn.EPI_RESID, bias=bias, resid=res)
    _close(out, acc + res.float(), "residual")
    aux = _mk((M, N), seed=10)
    out = Kn.gemm(a, b, mode=Kn.EPI_MUL, aux_in=aux)
    _close(out, (a.float() @ b.float().t()) * aux.float(), "multiply by the saved derivative")
    out32 = Kn.gemm(a, b, mode=Kn.EPI_STORE_F32)
    _close(out32, a.float() @ b.float().t(), "fp32 store")


@pytest.mark.parametrize("M,N,K", [(200, 264, 200), (129, 136, 72), (640, 1032, 136)])
@pytest.mark.parametrize("bn", [128, 256, 512])
def test_gemm_epilogues_tail_shapes(M, N, K, bn):
    """Every fused epilogue on shapes whose last row and column tiles are partial, at every tile width."""
    from diloco_swarm_b200.ops import kernels as Kn
    from diloco_swarm_b200.ops._lib import Status
    st = Status(torch.device("cuda"))
    a, b = _mk((M, K), seed=21), _mk((N, K), 0.05, seed=22)
    bias = torch.randn(N, device="cuda")
    acc = a.float() @ b.float().t()
    guard = 7.0          # rows past M / columns past N of padded outputs must stay untouched
    def padded(dtype=torch.bfloat16):
        return torch.full((M + 8, N + 8), guard, dtype=dtype, device="cuda")
    def check_guard(t, what):
        assert bool((t[M:, :] == guard).all()) and bool((t[:, N:] == guard).all()), f"{what}: wrote outside the matrix"
    o = padded()
    Kn.gemm(a, b, bias=bias, out=o[:M, :N], bn=bn, status=st)
    _close(o[:M, :N], acc + bias, "bias"); check_guard(o, "bias")
    o, pre = padded(), padded()
    Kn.gemm(a, b, mode=Kn.EPI_GELU, bias=bias, aux_out=pre[:M, :N], out=o[:M, :N], bn=bn, status=st)
    xg = (acc + bias).clone().requires_grad_(True)
    torch.nn.functional.gelu(xg).sum().backward()
    _close(pre[:M, :N], xg.grad, "gelu derivative"); check_guard(pre, "gelu derivative")
    _close(o[:M, :N], torch.nn.functional.gelu(acc + bias), "gelu"); check_guard(o, "gelu")
    res = _mk((M, N), seed=23)
    o = padded()
    Kn.gemm(a, b, mode=Kn.EPI_RESID, bias=bias, resid=res, out=o[:M, :N], bn=bn, status=st)
    _close(o[:M, :N], acc + bias + res.float(), "residual"); check_guard(o, "residual")
    aux = _mk((M, N), 2.0, seed=24)
    o = padded()
    Kn.gemm(a, b, mode=Kn.EPI_MUL, aux_in=aux, out=o[:M, :N], bn=bn, status=st)
    _close(o[:M, :N], acc * aux.float(), "multiply"); check_guard(o, "multiply")
    o32 = padded(torch.float32)
    Kn.gemm(a, b, mode=Kn.EPI_STORE_F32, out=o32[:M, :N], bn=bn, status=st)
    _close(o32[:M, :N], acc, "fp32 store"); check_guard(o32, "fp32 store")
    torch.cuda.synchronize()
    st.raise_if_set()


def test_fast_gelu_matches_erf_form():
    """The epilogues' erf approximation against torch's exact GELU and its derivative over the whole
    range that matters, including the tails: the difference must be far below bf16 resolution."""
    from diloco_swarm_b200.ops import kernels as Kn
    n = 1 << 14
    xs = torch.linspace(-12.0, 12.0, n, device="cuda")
    # a GEMM whose accumulator is exactly x: one non-zero column of A (x, bf16) times ones
    xb = xs.to(torch.bfloat16)
    a = torch.zeros(n, 8, dtype=torch.bfloat16, device="cuda"); a[:, 0] = xb
    b = torch.zeros(8, 8, dtype=torch.bfloat16, device="cuda"); b[:, 0] = 1.0      # every output column = x
    dg = torch.empty(n, 8, dtype=torch.bfloat16, device="cuda")
    g = Kn.gemm(a, b, mode=Kn.EPI_GELU, aux_out=dg)
    ref = torch.nn.functional.gelu(xb.float())
    assert torch.allclose(g[:, 0].float(), ref, atol=1e-6, rtol=2 ** -7)
    x = xb.float().requires_grad_(True)
    torch.nn.functional.gelu(x).sum().backward()
    assert torch.allclose(dg[:, 0].float(), x.grad, atol=1e-6, rtol=2 ** -7)


def test_gemm_persistent_many_tiles():
    """More tiles than SMs, so CTAs loop over tiles and both accumulators are reused."""
    from diloco_swarm_b200.ops import kernels as Kn
    M, N, K = 4096, 2304, 768
    a, b = _mk((M, K), seed=11), _mk((N, K), 0.05, seed=12)
    for bn in (256, 512):
        _close(Kn.gemm(a, b, bn=bn), a.float() @ b.float().t(), f"persistent bn{bn}")
        _close(Kn.gemm(a, b, bn=bn, max_ctas=7), a.float() @ b.float().t(), f"persistent capped grid bn{bn}")
