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


# the last case is the full depth of the reference's transformer (24 blocks in 6 super-blocks of 4,
# nn/d_diffusion_transformer.py:267-310) at a size the CPU oracle finishes in seconds
@pytest.mark.parametrize("n,samples,blocks", [(96, 1, 4), (150, 2, 8), (128, 1, 24)])
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


def test_sampler_loop_around_the_gpu_transformer(ops, oracle):
    """The sampler of d_alphafold3.py:316-404 (host arithmetic in diffusion_head.py) driving the DiffusionTransformer on
    the GPU, against the same loop around the CPU oracle's transformer.  The atom encoder / decoder of the reference's
    denoiser are outside this path; fixed random linear maps stand in for them (positions -> token activations ->
    position update), identical on both sides, so what is compared is the transformer inside the EDM-preconditioned
    Euler loop over a few steps, with several samples batched (use_batch_infer)."""
    from distributed_xfold_b200 import diffusion, diffusion_head as dh
    n, atoms, blocks, steps, samples = 48, 4, 4, 3, 2
    g = torch.Generator().manual_seed(31)
    st = oracle.make_diffusion_transformer_state(g, "", 768, 384, 128, 16, blocks, 4)
    rst = {k: v.to(BF).float() for k, v in st.items()}
    cond = torch.randn(n, 384, generator=g).to(BF)
    pair = torch.randn(n, n, 128, generator=g).to(BF)
    seq_mask = torch.ones(n)
    atom_mask = torch.ones(n, atoms)
    enc = (torch.randn(atoms * 3, 768, generator=g) / (atoms * 3) ** 0.5).to(BF).float()   # stand-in atom encoder
    dec = (torch.randn(768, atoms * 3, generator=g) / 768 ** 0.5).to(BF).float()           # stand-in atom decoder
    levels = 160.0 * (0.05 / 160.0) ** torch.linspace(0, 1, steps + 1)

    model = diffusion.PackedDiffusionTransformer(st, "", "cuda", 16, blocks, 4)
    pl = model.pair_logits(pair.cuda().contiguous())
    cond_d, mask_d = cond.cuda().contiguous(), seq_mask.cuda()

    def denoiser(transformer):
        def f(noisy, t_hat, step):
            act = ((noisy * dh.input_scaling(t_hat)).flatten(-2) @ enc).to(BF)             # [S, n, 768]
            out = transformer(act)
            upd = (torch.nn.functional.layer_norm(out.float(), (768,)) @ dec).reshape(noisy.shape)
            return dh.denoised_positions(noisy, upd, t_hat, atom_mask[None])
        return f

    def gpu_transformer(act):
        a = act.cuda().contiguous()
        model.forward(a, mask_d, cond_d, pl)
        ops.synchronize_and_check()
        return a.cpu()

    def cpu_transformer(act):
        with torch.no_grad():
            return oracle.diffusion_transformer(rst, "", act.float(), seq_mask, cond.float(), pair.float(), 16, blocks, 4)

    sched = dh.SamplerSchedule(levels)
    assert dh.use_batch_infer(samples, 1)
    got = dh.sample_diffusion(denoiser(gpu_transformer), sched, atom_mask, samples, generator=torch.Generator().manual_seed(5))
    ref = dh.sample_diffusion(denoiser(cpu_transformer), sched, atom_mask, samples, generator=torch.Generator().manual_seed(5))
    assert got.shape == (samples, n, atoms, 3) and torch.isfinite(got).all()
    assert relf(got, ref) < 2e-2
