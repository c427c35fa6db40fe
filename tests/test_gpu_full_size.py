"""Checks at the sizes the benchmark configurations name, where the fp32 CPU oracle of a whole block would take
minutes: size-independent properties of the block at N = 1024, and the reference's awkward token count N = 764
(not a multiple of any tile size; distribute_utils.py:107-121 splits it 7 x 96 + 92) against the oracle for
TriangleMultiplication.

Properties (every sub-layer of the block treats tokens symmetrically):
* relabelling the tokens relabels the outputs: block(P z P^T, P s) = P block(z, s) P^T.  The two sides run the
  same arithmetic on differently placed data (different tiles, different accumulation order), so they agree to
  bf16 rounding, not bitwise;
* what padded tokens hold never reaches an unpadded position.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def relf(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


@pytest.fixture(scope="module")
def block_1024(ops, oracle):
    n = 1024
    g = torch.Generator().manual_seed(4242)
    st = oracle.make_pairformer_block_state(g, "")
    w = ops.PackedPairformerBlock(st, "", "cuda")
    z, s, pm, sm = oracle.make_inputs(4243, n, pad_frac=0.1)
    return n, w, z.to(BF), s.to(BF), pm, sm


def run_block(ops, w, z, s, pm, sm):
    zd, sd = z.cuda().contiguous(), s.cuda().contiguous()
    ops.pairformer_block_(zd, sd, pm.cuda(), sm.cuda(), w)
    ops.synchronize_and_check()
    assert torch.isfinite(zd.float()).all() and torch.isfinite(sd.float()).all()
    return zd, sd


def test_block_n1024_token_relabelling(ops, block_1024):
    n, w, z, s, pm, sm = block_1024
    z1, s1 = run_block(ops, w, z, s, pm, sm)
    perm = torch.randperm(n, generator=torch.Generator().manual_seed(7))
    zp = z[perm][:, perm].contiguous()
    z2, s2 = run_block(ops, w, zp, s[perm].contiguous(), pm[perm][:, perm].contiguous(), sm[perm].contiguous())
    pc = perm.cuda()
    z1p, s1p = z1[pc][:, pc], s1[pc]
    valid = (pm[perm][:, perm] > 0).cuda()
    upd_ref = z1p.float() - zp.cuda().float()
    upd = z2.float() - zp.cuda().float()
    assert relf(z2.float()[valid], z1p.float()[valid]) < 2e-2
    assert relf(upd[valid], upd_ref[valid]) < 3e-2
    sv = (sm[perm] > 0).cuda()
    assert relf(s2.float()[sv], s1p.float()[sv]) < 2e-2
    del z1, z2, z1p


def test_block_n1024_padding_is_inert(ops, block_1024):
    n, w, z, s, pm, sm = block_1024
    z1, s1 = run_block(ops, w, z, s, pm, sm)
    pad = sm == 0
    assert int(pad.sum()) > 0
    g = torch.Generator().manual_seed(8)
    z_alt, s_alt = z.clone(), s.clone()
    z_alt[pad] = (3.0 * torch.randn(int(pad.sum()), n, 128, generator=g)).to(BF)
    z_alt[:, pad] = (3.0 * torch.randn(n, int(pad.sum()), 128, generator=g)).to(BF)
    s_alt[pad] = (3.0 * torch.randn(int(pad.sum()), 384, generator=g)).to(BF)
    z2, s2 = run_block(ops, w, z_alt, s_alt, pm, sm)
    valid = (pm > 0).cuda()
    # identical inputs at every position that can reach an unpadded output: identical arithmetic, identical results
    assert torch.equal(z1[valid], z2[valid])
    assert torch.equal(s1[(sm > 0).cuda()], s2[(sm > 0).cuda()])


@pytest.mark.parametrize("outgoing", [True, False])
def test_triangle_multiplication_n764(ops, oracle, outgoing):
    n = 764
    g = torch.Generator().manual_seed(764)
    st = oracle.make_trimul_state(g, "")
    z = torch.randn(n, n, 128, generator=g).to(BF)
    sm = (torch.rand(n, generator=g) > 0.1).float()
    mask = sm[:, None] * sm[None, :]
    rst = {k: v.to(BF).float() for k, v in st.items()}
    torch.set_num_threads(max(torch.get_num_threads(), 8))
    ref = z.float() + oracle.triangle_multiplication(rst, "", z.float(), mask, outgoing)
    w = ops.PackedTriMul(st, "", "cuda")
    zd = z.cuda().contiguous()
    ops.triangle_multiplication_(zd, mask.cuda(), w, outgoing)
    ops.synchronize_and_check()
    v = mask > 0
    got = zd.float().cpu()
    assert relf(got[v], ref[v]) < 2e-2
    assert relf(got[v] - z.float()[v], ref[v] - z.float()[v]) < 3e-2
