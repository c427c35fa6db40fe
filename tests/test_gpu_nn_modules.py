"""GPU parity of the module classes (the reference's names and forward signatures) against the CPU
oracle: every forward returns what the reference's forward returns (the update, or the updated
activations for the transformer / block).  bf16 tolerance 2e-2 relative Frobenius (3e-2 on updates)."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def relf(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def rounded(st):
    return {k: v.to(BF).float() for k, v in st.items()}


@pytest.fixture(scope="module")
def nnm(ops):
    import distributed_xfold_b200.nn as m
    from distributed_xfold_b200.distribute_utils import DeviceMesh
    m.mesh1 = DeviceMesh(1, 1, 1)
    return m


@pytest.mark.parametrize("outgoing", [True, False])
def test_xsmm_triangle_multiplication_module(nnm, oracle, outgoing):
    n = 72
    g = torch.Generator().manual_seed(1)
    st = oracle.make_trimul_state(g, "")
    z = torch.randn(n, n, 128, generator=g).to(BF)
    mask = (torch.rand(n, n, generator=g) > 0.1).float()
    mod = nnm.XSMMTriangleMultiplication(128, outgoing).cuda()
    mod.load_state_dict(st)
    upd = mod(z.cuda(), mask.cuda())
    ref = oracle.triangle_multiplication(rounded(st), "", z.float(), mask, outgoing)
    assert upd.shape == z.shape and relf(upd.float().cpu(), ref) < 3e-2


@pytest.mark.parametrize("transpose", [False, True])
def test_grid_self_attention_module_full_and_sharded(nnm, oracle, transpose):
    n = 80
    g = torch.Generator().manual_seed(2)
    st = oracle.make_grid_attention_state(g, "")
    z = torch.randn(n, n, 128, generator=g).to(BF)
    sm = (torch.rand(n, generator=g) > 0.1).float()
    pm = sm[:, None] * sm[None, :]
    mod = nnm.DistributeGridSelfAttention(nnm.mesh1, 128, 4, transpose).cuda()
    mod.load_state_dict(st)
    ref = oracle.grid_self_attention(rounded(st), "", z.float(), pm, z.float(), transpose)
    upd = mod(z.cuda(), pm.cuda(), full_pair=z.cuda())
    assert relf(upd.float().cpu()[pm > 0], ref[pm > 0]) < 3e-2
    # the reference's sharded call: a row shard (starting node) or column shard (ending node) + the full pair
    sl = slice(16, 48)
    shard = z[:, sl] if transpose else z[sl]
    upd_s = mod(shard.cuda().contiguous(), pm[sl].cuda(), full_pair=z.cuda())
    ref_s = oracle.grid_self_attention(rounded(st), "", shard.float(), pm[sl], z.float(), transpose)
    valid = (pm[:, sl] if transpose else pm[sl]) > 0
    assert upd_s.shape == shard.shape and relf(upd_s.float().cpu()[valid], ref_s[valid]) < 3e-2


def test_transition_module(nnm, oracle):
    g = torch.Generator().manual_seed(3)
    st = oracle.make_transition_state(g, "", 128)
    x = torch.randn(33, 35, 128, generator=g).to(BF)
    mod = nnm.DistributeTransition(nnm.mesh1, 128, 4).cuda()
    mod.load_state_dict(st)
    assert relf(mod(x.cuda()).float().cpu(), oracle.transition(rounded(st), "", x.float())) < 2e-2


def test_adaptive_layernorm_and_adaln_zero_modules(nnm, oracle):
    g = torch.Generator().manual_seed(4)
    n, c, cc = 70, 768, 384
    x = torch.randn(2, n, c, generator=g).to(BF)
    cond = torch.randn(n, cc, generator=g).to(BF)
    st = oracle.make_adaptive_layernorm_state(g, "", c, cc, True)
    mod = nnm.AdaptiveLayerNorm(c, cc, True).cuda()
    mod.load_state_dict(st)
    assert relf(mod(x.cuda(), cond.cuda()).float().cpu(), oracle.adaptive_layernorm(rounded(st), "", x.float(), cond.float())) < 1e-2
    st = oracle.make_adaln_zero_state(g, "", c, c, cc, True)
    mod = nnm.DistributeAdaLNZero(nnm.mesh1, c, c, cc, True).cuda()
    mod.load_state_dict(st)
    assert relf(mod(x.cuda(), cond.cuda()).float().cpu(), oracle.adaln_zero(rounded(st), "", x.float(), cond.float())) < 1e-2
    st = oracle.make_diffusion_transition_state(g, "", c, cc, 2, True)
    mod = nnm.DistributeDiffusionTransition(nnm.mesh1, c, cc, 2, True).cuda()
    mod.load_state_dict(st)
    assert relf(mod(x.cuda(), cond.cuda()).float().cpu(), oracle.diffusion_transition(rounded(st), "", x.float(), cond.float())) < 2e-2


@pytest.mark.parametrize("cond_on,batched", [(True, True), (False, False)])
def test_self_attention_module(nnm, oracle, cond_on, batched):
    g = torch.Generator().manual_seed(5)
    n, c, cc = 90, (768 if cond_on else 384), 384
    st = oracle.make_self_attention_state(g, "", c, cc, cond_on)
    x = torch.randn(*((2, n, c) if batched else (n, c)), generator=g).to(BF)
    cond = torch.randn(n, cc, generator=g).to(BF) if cond_on else None
    mask = (torch.rand(n, generator=g) > 0.1).float()
    pl = torch.randn(16, n, n, generator=g)
    mod = nnm.DistributeSelfAttention(nnm.mesh1, c, cc, 16, cond_on, batched).cuda()
    mod.load_state_dict(st)
    got = mod(x.cuda(), mask.cuda(), pl.cuda(), None if cond is None else cond.cuda())
    ref = oracle.self_attention(rounded(st), "", x.float(), mask, pl, None if cond is None else cond.float(), 16)
    sel = (slice(None), mask > 0) if batched else (mask > 0,)
    assert relf(got.float().cpu()[sel], ref[sel]) < 2e-2


def test_diffusion_transformer_module(nnm, oracle):
    g = torch.Generator().manual_seed(6)
    n, blocks = 64, 4
    st = oracle.make_diffusion_transformer_state(g, "", 768, 384, 128, 16, blocks, 4)
    act = torch.randn(2, n, 768, generator=g).to(BF)
    cond = torch.randn(n, 384, generator=g).to(BF)
    pair = torch.randn(n, n, 128, generator=g).to(BF)
    mask = torch.ones(n)
    mod = nnm.DistributeDiffusionTransformer(nnm.mesh1, num_blocks=blocks, use_batch_infer=True).cuda()
    mod.load_state_dict(st)
    a = act.cuda()
    out = mod(a, mask.cuda(), cond.cuda(), pair.cuda())
    assert out.data_ptr() == a.data_ptr()  # in place, as the reference's `act +=`
    ref = oracle.diffusion_transformer(rounded(st), "", act.float(), mask, cond.float(), pair.float(), 16, blocks, 4)
    assert relf(out.float().cpu(), ref) < 2e-2


def test_pairformer_block_module(nnm, ops, oracle):
    g = torch.Generator().manual_seed(7)
    n = 64
    st = oracle.make_pairformer_block_state(g, "")
    z, s, pm, sm = oracle.make_inputs(8, n, pad_frac=0.1)
    z, s = z.to(BF), s.to(BF)
    mod = nnm.DistributePairformerBlock(nnm.mesh1).cuda()
    mod.load_state_dict(st)
    zd, sd = z.cuda(), s.cuda()
    rz_, rs_ = mod(zd, pm.cuda(), sd, sm.cuda())
    ops.synchronize_and_check()
    rz, rs = oracle.pairformer_block(rounded(st), "", z.float(), pm, s.float(), sm)
    assert rz_.data_ptr() == zd.data_ptr()
    assert relf(zd.float().cpu()[pm > 0], rz[pm > 0]) < 2e-2 and relf(sd.float().cpu()[sm > 0], rs[sm > 0]) < 2e-2
