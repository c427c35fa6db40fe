"""GPU: the same call on the same inputs gives the same bits.  The kernels take their work items in a fixed order and
use no atomics, so a difference between two runs would mean a race between the roles of a kernel (producer, issuers,
softmax warps) or between kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.mark.parametrize("n", [64, 100, 128, 256])
def test_block_and_attention_repeat_bit_for_bit(ops, oracle, n):
    g = torch.Generator().manual_seed(5 + n)
    st = oracle.make_grid_attention_state(g, "")
    w = ops.PackedTriAttn(st, "", "cuda")
    z = torch.randn(n, n, 128, generator=g).to(BF).cuda()
    pm = ((torch.rand(n, generator=g) > 0.1).float()[:, None] * torch.ones(n)[None, :]).cuda().contiguous()
    for transpose in (False, True):
        outs = []
        for _ in range(4):
            zz = z.clone()
            ops.triangle_attention_(zz, pm, w, transpose)
            ops.synchronize_and_check()
            outs.append(zz)
        assert all(torch.equal(o, outs[0]) for o in outs[1:])
    wb = ops.PackedPairformerBlock(oracle.make_pairformer_block_state(g, ""), "", "cuda")
    s = torch.randn(n, 384, generator=g).to(BF).cuda()
    sm = torch.ones(n).cuda()
    outs = []
    for _ in range(4):
        zz, ss = z.clone(), s.clone()
        ops.pairformer_block_(zz, ss, pm, sm, wb)
        ops.synchronize_and_check()
        outs.append((zz, ss))
    assert all(torch.equal(o[0], outs[0][0]) and torch.equal(o[1], outs[0][1]) for o in outs[1:])
