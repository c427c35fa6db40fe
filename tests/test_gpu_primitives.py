"""GPU parity of the primitive kernels (LayerNorm, SwiGLU, tcgen05 GEMM epilogues, batched
contraction) against plain fp32 PyTorch on the same bf16-rounded inputs, through the C ABI."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def relf(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(BF)


@pytest.mark.parametrize("C", [128, 384, 768])
@pytest.mark.parametrize("rows", [1, 37, 4096])
def test_layernorm(ops, C, rows):
    x = rnd(rows, C, seed=C + rows, scale=3.0) + 0.5
    g = torch.randn(C, generator=torch.Generator().manual_seed(1)) * 0.2 + 1
    b = torch.randn(C, generator=torch.Generator().manual_seed(2)) * 0.1
    y = ops.layernorm(x.cuda(), g.cuda(), b.cuda())
    ops.synchronize_and_check()
    ref = torch.nn.functional.layer_norm(x.float(), (C,), g, b, 1e-5)
    assert relf(y.float().cpu(), ref) < 4e-3  # bf16 output rounding only
    y2 = ops.layernorm(x.cuda())
    ref2 = torch.nn.functional.layer_norm(x.float(), (C,), None, None, 1e-5)
    assert relf(y2.float().cpu(), ref2) < 4e-3


@pytest.mark.parametrize("H", [4, 16])
def test_layernorm_fused_projection(ops, H):
    rows, C = 3000, 128
    x = rnd(rows, C, seed=7)
    w = torch.randn(H, C, generator=torch.Generator().manual_seed(3)) / 11
    y, proj = ops.layernorm(x.cuda(), None, None, proj_w=w.cuda())
    ops.synchronize_and_check()
    ref = torch.nn.functional.layer_norm(x.float(), (C,), None, None, 1e-5)
    assert relf(proj.cpu(), (ref @ w.T).T) < 1e-4  # fp32 path
    assert relf(y.float().cpu(), ref) < 4e-3


def test_layernorm_adaln_modulation(ops):
    S, N, C = 3, 50, 768
    x = rnd(S, N, C, seed=9)
    sc, sh = rnd(N, C, seed=10), rnd(N, C, seed=11)
    y = ops.layernorm(x.cuda(), mod_scale=sc.cuda(), mod_shift=sh.cuda())
    ops.synchronize_and_check()
    ref = torch.sigmoid(sc.float()) * torch.nn.functional.layer_norm(x.float(), (C,)) + sh.float()
    assert relf(y.float().cpu(), ref) < 4e-3


def test_swiglu(ops):
    x = rnd(777, 1024, seed=4)
    y = ops.swiglu(x.cuda())
    ops.synchronize_and_check()
    a, b = x.float().chunk(2, -1)
    assert relf(y.float().cpu(), torch.nn.functional.silu(a) * b) < 4e-3


@pytest.mark.parametrize("M,K,N", [(128, 128, 128), (300, 128, 512), (1000, 384, 2048), (5000, 512, 128),
                                   (129, 768, 768), (64, 1536, 384), (40000, 128, 512)])
def test_linear(ops, M, K, N):
    x, w = rnd(M, K, seed=M), rnd(N, K, seed=N + 1, scale=K ** -0.5)
    bias = torch.randn(N, generator=torch.Generator().manual_seed(5))
    scale = torch.rand(N, generator=torch.Generator().manual_seed(6)) + 0.5
    y = ops.linear(x.cuda(), w.cuda(), bias.cuda(), scale.cuda())
    ops.synchronize_and_check()
    ref = (x.float() @ w.float().T + bias) * scale
    assert relf(y.float().cpu(), ref) < 4e-3
    y0 = ops.linear(x.cuda(), w.cuda())
    assert relf(y0.float().cpu(), x.float() @ w.float().T) < 4e-3


@pytest.mark.parametrize("M,K,N", [(700, 128, 128), (3000, 512, 128), (515, 1536, 384)])
def test_linear_gate_residual(ops, M, K, N):
    x, w = rnd(M, K, seed=1), rnd(N, K, seed=2, scale=K ** -0.5)
    gate, resid = rnd(M, N, seed=3), rnd(M, N, seed=4)
    y = ops.linear_gate_residual(x.cuda(), w.cuda(), gate.cuda(), resid.cuda())
    ops.synchronize_and_check()
    ref = resid.float() + (x.float() @ w.float().T) * torch.sigmoid(gate.float())
    assert relf(y.float().cpu(), ref) < 4e-3
    y = ops.linear_gate_residual(x.cuda(), w.cuda(), None, resid.cuda())
    assert relf(y.float().cpu(), resid.float() + x.float() @ w.float().T) < 4e-3
    # gate shared by rows with equal (row % mod): the AdaLN-Zero conditioning of several samples
    mod = 103
    g2 = rnd(mod, N, seed=8)
    y = ops.linear_gate_residual(x.cuda(), w.cuda(), g2.cuda(), resid.cuda(), row_gate_mod=mod)
    idx = torch.arange(M) % mod
    ref = resid.float() + (x.float() @ w.float().T) * torch.sigmoid(g2.float()[idx])
    ops.synchronize_and_check()
    assert relf(y.float().cpu(), ref) < 4e-3


@pytest.mark.parametrize("M,K,F", [(900, 128, 512), (260, 384, 1536), (100, 768, 1536)])
def test_linear_swiglu(ops, M, K, F):
    x, w1 = rnd(M, K, seed=1), rnd(2 * F, K, seed=2, scale=K ** -0.5)
    y = ops.linear_swiglu(x.cuda(), ops.pack_swiglu_weight(w1).contiguous().cuda())
    ops.synchronize_and_check()
    a, b = (x.float() @ w1.float().T).chunk(2, -1)
    assert relf(y.float().cpu(), torch.nn.functional.silu(a) * b) < 5e-3


@pytest.mark.parametrize("ch,mi,nj,kk", [(4, 128, 256, 64), (3, 200, 200, 200), (128, 96, 96, 96), (2, 1024, 512, 1024),
                                         (5, 40, 40, 40)])
def test_batched_contract(ops, ch, mi, nj, kk):
    a, b = rnd(ch, mi, kk, seed=1), rnd(ch, nj, kk, seed=2)
    out = ops.batched_contract(a.cuda(), b.cuda())
    ops.synchronize_and_check()
    ref = torch.einsum("cik,cjk->cij", a.float(), b.float())
    assert relf(out.float().cpu(), ref) < 4e-3


def test_layernorm_fused_projection_64(ops):
    """64 outputs (the diffusion transformer's pair logits for one super-block: 4 blocks x 16 heads)."""
    rows, C, H = 1500, 128, 64
    x = rnd(rows, C, seed=17)
    w = torch.randn(H, C, generator=torch.Generator().manual_seed(4)) / 11
    g = torch.rand(C, generator=torch.Generator().manual_seed(5)) + 0.5
    _, proj = ops.layernorm(x.cuda(), g.cuda(), None, proj_w=w.cuda(), want_y=False)
    ops.synchronize_and_check()
    ref = torch.nn.functional.layer_norm(x.float(), (C,), g, None, 1e-5)
    assert relf(proj.cpu(), (ref @ w.T).T) < 1e-4


@pytest.mark.parametrize("ch,n", [(2, 64), (3, 200), (4, 333), (2, 520)])
def test_contract_planes_incoming_mn_major(ops, ch, n):
    """'ckj,cki->cij' (nn/d_triangle_multiplication.py:122-124) on untransposed channel planes: the GEMM reads both
    operands with the contraction index as their slow dimension (MN-major tensor-core operands)."""
    ld = (n + 7) // 8 * 8
    a = torch.zeros(ch, n, ld, dtype=BF)
    b = torch.zeros(ch, n, ld, dtype=BF)
    a[:, :, :n] = rnd(ch, n, n, seed=11 + n)
    b[:, :, :n] = rnd(ch, n, n, seed=12 + n)
    # the pad columns are never read: poison them
    a[:, :, n:] = float("nan")
    b[:, :, n:] = float("nan")
    o = ops.stage_trimul_contract_planes_incoming(a.cuda(), b.cuda(), n)
    ops.synchronize_and_check()
    ref = torch.einsum("ckj,cki->cij", a[:, :, :n].float(), b[:, :, :n].float())
    assert relf(o[:, :, :n].float().cpu(), ref) < 4e-3
    # and the outgoing product on the same planes, for the pair
    o2 = ops.stage_trimul_contract_planes(a.nan_to_num(0.).cuda(), b.nan_to_num(0.).cuda(), n)
    ops.synchronize_and_check()
    ref2 = torch.einsum("cik,cjk->cij", a[:, :, :n].float(), b[:, :, :n].float())
    assert relf(o2[:, :, :n].float().cpu(), ref2) < 4e-3
