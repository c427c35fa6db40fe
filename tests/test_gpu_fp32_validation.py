"""The fp32 validation build (``xfold_pairformer_stack_f32_fwd``: float32 storage, float32 FMA arithmetic) against the
fp32 CPU oracle and against the reference's own output, to the 1e-4 the float32 configuration is specified to:

* one block at N = 256 with z, s ~ N(0,1), an all-ones mask and seed-0 weights -- the reference's CPU-runnable
  configuration;
* the reference's own DistributePairformerBlock.forward output (golden vector);
* the 48-block trunk with a 10 % padding mask: here the float32 path stays within 1e-4 of the oracle after the LAST
  block, which separates what the bf16 kernels lose through 48 blocks (storage rounding, amplified) from the algorithm.
Errors are relative Frobenius norms over unpadded positions.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-4


def test_fp32_block_n256_config1(ops, oracle):
    n = 256
    g = torch.Generator().manual_seed(0)
    st = oracle.make_pairformer_block_state(g, "")
    z, s, pm, sm = oracle.make_inputs(1, n, pad_frac=0.0)
    with torch.no_grad():
        rz, rs = oracle.pairformer_block(st, "", z, pm, s, sm, row_chunk=64)
    w = ops.PackedPairformerBlockF32(st, "", "cuda")
    zd, sd = z.cuda().contiguous(), s.cuda().contiguous()
    ops.pairformer_stack_f32_(zd, sd, pm.cuda(), sm.cuda(), [w])
    ops.synchronize_and_check()
    ez, es = oracle.rel_frobenius(zd.cpu(), rz), oracle.rel_frobenius(sd.cpu(), rs)
    print(f"\nfp32 block N={n}: pair {ez:.3e}, single {es:.3e}")
    assert ez <= TOL and es <= TOL


def test_fp32_block_reference_golden(ops, oracle, golden):
    meta = golden["ref/pairformer_block"]["meta"]
    ref_z, ref_s = golden["ref/pairformer_block"]["out"]
    n = meta["n"]
    g = torch.Generator().manual_seed(meta["seed"])
    st = oracle.make_pairformer_block_state(g, "")
    z = torch.randn(n, n, 128, generator=g)
    s = torch.randn(n, 384, generator=g)
    sm = (torch.rand(n, generator=g) > 0.15).float()
    pm = sm[:, None] * sm[None, :]
    w = ops.PackedPairformerBlockF32(st, "", "cuda")
    zd, sd = z.cuda().contiguous(), s.cuda().contiguous()
    ops.pairformer_stack_f32_(zd, sd, pm.cuda(), sm.cuda(), [w])
    ops.synchronize_and_check()
    assert oracle.rel_frobenius(zd.cpu()[pm > 0], ref_z[pm > 0]) <= TOL
    assert oracle.rel_frobenius(sd.cpu()[sm > 0], ref_s[sm > 0]) <= TOL


@pytest.mark.parametrize("n", [64, 128])
def test_fp32_trunk_48_blocks(ops, oracle, n):
    nb = 48
    st = oracle.make_pairformer_stack_state(200 + n, nb)
    z, s, pm, sm = oracle.make_inputs(201 + n, n, pad_frac=0.1)
    blocks = [ops.PackedPairformerBlockF32(st, f"trunk_pairformer.{i}.", "cuda") for i in range(nb)]
    zd, sd = z.cuda().contiguous(), s.cuda().contiguous()
    ops.pairformer_stack_f32_(zd, sd, pm.cuda(), sm.cuda(), blocks)
    ops.synchronize_and_check()
    rz, rs = z, s
    with torch.no_grad():
        for i in range(nb):
            rz, rs = oracle.pairformer_block(st, f"trunk_pairformer.{i}.", rz, pm, rs, sm)
    ez = oracle.rel_frobenius(zd.cpu()[pm > 0], rz[pm > 0])
    es = oracle.rel_frobenius(sd.cpu()[sm > 0], rs[sm > 0])
    print(f"\nfp32 trunk, {nb} blocks, N={n}: pair {ez:.3e}, single {es:.3e}")
    assert ez <= TOL and es <= TOL
