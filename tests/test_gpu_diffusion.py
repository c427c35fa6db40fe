"""GPU parity of the DiffusionTransformer composition (AdaLN, AttentionPairBias 16 x 48, AdaLN-Zero,
DiffusionTransition) against the CPU oracle, whose forward is pinned to the reference's
DistributeDiffusionTransformer.forward.  bf16 tolerance: relative Frobenius <= 2e-2 on the activations
and <= 3e-2 on the accumulated update."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def relf(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


@pytest.mark.parametrize("n,samples,blocks", [(96, 1, 4), (150, 2, 8)])
def test_diffusion_transformer(ops, oracle, n, samples, blocks):
    from distributed_xfold_b200 import diffusion
    g = torch.Generator().manual_seed(1000 + n)
    st = oracle.make_diffusion_transformer_state(g, "", 768, 384, 128, 16, blocks, 4)
    act = torch.randn(samples, n, 768, generator=g).to(BF)
    cond = torch.randn(n, 384, generator=g).to(BF)
    pair = torch.randn(n, n, 128, generator=g).to(BF)
    mask = (torch.rand(n, generator=g) > 0.1).float()
    rst = {k: v.to(BF).float() for k, v in st.items()}
    with torch.no_grad():
        ref = oracle.diffusion_transformer(rst, "", act.float(), mask, cond.float(), pair.float(), 16, blocks, 4)
    model = diffusion.PackedDiffusionTransformer(st, "", "cuda", 16, blocks, 4)
    pl = model.pair_logits(pair.cuda().contiguous())
    a = act.cuda().contiguous()
    model.forward(a, mask.cuda(), cond.cuda().contiguous(), pl)
    ops.synchronize_and_check()
    got = a.float().cpu()
    valid = mask > 0
    assert torch.isfinite(got).all()
    assert relf(got[:, valid], ref[:, valid]) < 2e-2
    assert relf((got - act.float())[:, valid], (ref - act.float())[:, valid]) < 3e-2


def test_diffusion_single_sample_2d_input(ops, oracle):
    """[N, 768] activations (use_batch_infer False in the reference) take the same path."""
    from distributed_xfold_b200 import diffusion
    n, blocks = 64, 4
    g = torch.Generator().manual_seed(77)
    st = oracle.make_diffusion_transformer_state(g, "", 768, 384, 128, 16, blocks, 4)
    act = torch.randn(n, 768, generator=g).to(BF)
    cond = torch.randn(n, 384, generator=g).to(BF)
    pair = torch.randn(n, n, 128, generator=g).to(BF)
    mask = torch.ones(n)
    rst = {k: v.to(BF).float() for k, v in st.items()}
    with torch.no_grad():
        ref = oracle.diffusion_transformer(rst, "", act.float(), mask, cond.float(), pair.float(), 16, blocks, 4)
    model = diffusion.PackedDiffusionTransformer(st, "", "cuda", 16, blocks, 4)
    a = act.cuda().contiguous()
    model.forward(a, mask.cuda(), cond.cuda().contiguous(), model.pair_logits(pair.cuda().contiguous()))
    ops.synchronize_and_check()
    assert relf(a.float().cpu(), ref) < 2e-2
