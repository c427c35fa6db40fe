"""Parity AFTER THE TRUNK: the 48-block Pairformer loop (d_alphafold3.py:242-244) on the sm_100a kernels against the
fp32 CPU oracle's ``pairformer_stack`` on identical seeded inputs and (bf16-rounded) weights, with a random 10 % padding
mask.  The bound is the one the path is specified to: relative Frobenius error of the pair and single representations
after the LAST block <= 2e-2 over unpadded positions.  The error after every block is printed (run with -s), so a
failure shows where it grows.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
TOL = 2e-2


def _curve(ops, oracle, n, num_blocks, seed):
    st = oracle.make_pairformer_stack_state(seed, num_blocks)
    z, s, pm, sm = oracle.make_inputs(seed + 1, n, pad_frac=0.1)
    st_r = {k: v.to(BF).float() for k, v in st.items()}
    zr, sr = z.to(BF).float(), s.to(BF).float()
    trunk = ops.PackedPairformerStack.from_state(st, num_blocks, "cuda")
    # the product path: ONE call for the whole loop
    zd, sd = z.to(BF).cuda().contiguous(), s.to(BF).cuda().contiguous()
    pmd, smd = pm.cuda(), sm.cuda()
    ops.pairformer_stack_(zd, sd, pmd, smd, trunk)
    ops.synchronize_and_check()
    # block by block on both sides, for the error curve (and the loop must equal the one-call result bit for bit)
    zb, sb = z.to(BF).cuda().contiguous(), s.to(BF).cuda().contiguous()
    valid, svalid = pm > 0, sm > 0
    curve = []
    with torch.no_grad():
        for i in range(num_blocks):
            zr, sr = oracle.pairformer_block(st_r, f"trunk_pairformer.{i}.", zr, pm, sr, sm)
            ops.pairformer_block_(zb, sb, pmd, smd, trunk.blocks[i])
            ez = oracle.rel_frobenius(zb.float().cpu()[valid], zr[valid])
            es = oracle.rel_frobenius(sb.float().cpu()[svalid], sr[svalid])
            curve.append((ez, es))
    ops.synchronize_and_check()
    assert torch.equal(zb, zd) and torch.equal(sb, sd)
    assert torch.isfinite(zd.float()).all() and torch.isfinite(sd.float()).all()
    print(f"\nerror after block k (N={n}, {num_blocks} blocks): pair / single")
    for i, (ez, es) in enumerate(curve):
        print(f"  block {i + 1:2d}: {ez:.3e}  {es:.3e}")
    return curve


@pytest.mark.parametrize("n,num_blocks", [(64, 48), (128, 48), (256, 48)])
def test_trunk_parity_after_last_block(ops, oracle, n, num_blocks):
    curve = _curve(ops, oracle, n, num_blocks, seed=200 + n)
    ez, es = curve[-1]
    assert ez <= TOL and es <= TOL, f"after block {num_blocks}: pair {ez:.3e}, single {es:.3e} (bound {TOL})"
