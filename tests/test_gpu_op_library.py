"""The reference's operator interface on the GPU: ``torch.ops._alpha_attention.*`` (schemas of
xsmm_kernels/csrc/Alpha_Attention.cpp:181-211) called with the argument lists and layouts of the reference's wrappers
(xsmm_kernels/prototypes/*.py), checked against the oracle's restatements of the reference's spec classes.  Results come
back PADDED, as the wrappers expect; the tests narrow them the way the wrappers do."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def relf(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def rb(t):
    return t.to(BF).float()


@pytest.fixture(scope="module")
def lib(pkg, ops):
    from distributed_xfold_b200 import op_library
    op_library.register()
    return torch.ops._alpha_attention


@pytest.mark.parametrize("n,flag", [(40, 0), (40, 1), (64, 0)])
def test_op_triangle_multiplication(lib, oracle, n, flag):
    g = torch.Generator().manual_seed(50 + n + flag)
    st = oracle.make_trimul_state(g, "")
    z = torch.randn(n, n, 128, generator=g)
    mask = (torch.rand(n, n, generator=g) > 0.2).float()
    # load_xsmm_params de-interleaves projection and gate (nn/d_triangle_multiplication.py:128-129)
    de = lambda w: torch.cat([w[0::2], w[1::2]], 0)
    out = lib.traingle_multiplication_forward(
        z.to(BF).cuda().contiguous(), mask[..., None].cuda().contiguous(), flag,
        st["left_norm_input.weight"].to(BF).cuda(), st["left_norm_input.bias"].to(BF).cuda(),
        de(st["projection.weight"]).to(BF).cuda(), de(st["gate.weight"]).to(BF).cuda(),
        st["center_norm.weight"].to(BF).cuda(), st["center_norm.bias"].to(BF).cuda(),
        st["output_projection.weight"].to(BF).cuda(), st["gating_linear.weight"].to(BF).cuda())
    torch.cuda.synchronize()
    npad = (n + 31) // 32 * 32
    assert tuple(out.shape) == (npad, npad, 128)
    ref = oracle.triangle_multiplication({k: rb(v) for k, v in st.items()}, "", rb(z), mask, flag == 0)
    assert relf(out[:n, :n].float().cpu(), ref) < 3e-2
    assert float(out[n:].float().abs().sum()) == 0.0 and float(out[:, n:].float().abs().sum()) == 0.0


def _attn_weights(g, c, h, d, with_out):
    ws = {n: torch.randn(c, h, d, generator=g) / 8 for n in ("query_w", "key_w", "value_w", "gating_w")}
    ws["query_b"] = torch.randn(1, h, d, generator=g) / 8
    if with_out:
        ws["output_w"] = torch.randn(h, d, c, generator=g) / 8
    return ws


def test_op_grid_self_attention(lib, oracle):
    b, s, c, h, d = 7, 50, 128, 4, 32
    g = torch.Generator().manual_seed(60)
    ws = _attn_weights(g, c, h, d, True)
    x = torch.randn(b, s, c, generator=g)
    bias = 1e9 * ((torch.rand(b, 1, 1, s, generator=g) > 0.2).float() - 1)
    nb = torch.randn(h, s, s, generator=g)
    out = lib.grid_self_attn_forward(x.to(BF).cuda(), bias.cuda(), nb.cuda(), ws["query_w"].to(BF).cuda(),
                                     ws["key_w"].to(BF).cuda(), ws["value_w"].to(BF).cuda(), ws["gating_w"].to(BF).cuda(),
                                     ws["output_w"].to(BF).cuda(), d, d)
    torch.cuda.synchronize()
    assert tuple(out.shape) == (b, 64, c)
    ref = oracle.gated_attention(rb(x), bias, nb, rb(ws["query_w"]), rb(ws["key_w"]), rb(ws["value_w"]), rb(ws["gating_w"]),
                                 rb(ws["output_w"]))
    assert relf(out[:, :s].float().cpu(), ref) < 2e-2


@pytest.mark.parametrize("c,h", [(384, 16), (768, 16)])
def test_op_batch_diffusion_self_attention(lib, oracle, c, h):
    b, s, d = 2, 70, c // h
    g = torch.Generator().manual_seed(61 + c)
    ws = _attn_weights(g, c, h, d, False)
    x = torch.randn(b, s, c, generator=g)
    bias = 1e9 * ((torch.rand(1, 1, 1, s, generator=g) > 0.2).float() - 1)
    nb = torch.randn(h, s, s, generator=g)
    out = lib.batch_diffusion_self_attention_forward(x.to(BF).cuda(), bias.cuda(), nb.cuda(), ws["query_w"].to(BF).cuda(),
                                                     ws["query_b"].cuda(), ws["key_w"].to(BF).cuda(), ws["value_w"].to(BF).cuda(),
                                                     ws["gating_w"].to(BF).cuda(), d, d)
    torch.cuda.synchronize()
    assert tuple(out.shape) == (b, 128, h, d)
    ref = oracle.gated_attention(rb(x), bias, nb, rb(ws["query_w"]), rb(ws["key_w"]), rb(ws["value_w"]), rb(ws["gating_w"]),
                                 None, query_b=ws["query_b"])
    assert relf(out[:, :s].float().cpu(), ref) < 2e-2


def test_op_batch_diffusion_cross_attention(lib, oracle):
    b, s, k, c, h, d = 6, 32, 128, 128, 4, 32
    g = torch.Generator().manual_seed(62)
    ws = _attn_weights(g, c, h, d, False)
    qd, md = torch.randn(b, s, c, generator=g), torch.randn(b, k, c, generator=g)
    bb = torch.randn(b, h, s, k, generator=g)
    out = lib.batch_diffusion_cross_attention_forward(qd.to(BF).cuda(), md.to(BF).cuda(), bb.cuda(), ws["query_w"].to(BF).cuda(),
                                                      ws["query_b"].cuda(), ws["key_w"].to(BF).cuda(), ws["value_w"].to(BF).cuda(),
                                                      ws["gating_w"].to(BF).cuda(), d, d)
    torch.cuda.synchronize()
    assert tuple(out.shape) == (b, 64, h, d)
    ref = oracle.cross_attention(rb(qd), rb(md), bb, rb(ws["query_w"]), ws["query_b"], rb(ws["key_w"]), rb(ws["value_w"]),
                                 rb(ws["gating_w"]))
    assert relf(out[:, :s].float().cpu(), ref) < 2e-2


def test_op_transition(lib, oracle):
    g = torch.Generator().manual_seed(63)
    st = oracle.make_transition_state(g, "", 128)
    x = torch.randn(9, 21, 128, generator=g)
    out = lib.transition_forward(x.to(BF).cuda(), st["transition1.weight"].T.contiguous().to(BF).cuda(),
                                 st["transition2.weight"].T.contiguous().cuda(), st["input_layer_norm.weight"].to(BF).cuda(),
                                 st["input_layer_norm.bias"].to(BF).cuda())
    torch.cuda.synchronize()
    ref = oracle.transition({k: rb(v) for k, v in st.items()}, "", rb(x))
    assert tuple(out.shape) == tuple(x.shape) and relf(out.float().cpu(), ref) < 2e-2
