"""GPU parity of the row-sharded Pairformer block (the multi-GPU path) against the CPU oracle.

With one GPU the block runs with a single shard, which still exercises every row-shard stage
function of the C ABI; with two or more visible GPUs it also runs as NCCL ranks (one process per
GPU, ragged shards included).  Same tolerances as the single-GPU module tests."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def relf(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def _reference(oracle, n, seed, pad):
    g = torch.Generator().manual_seed(seed)
    st = oracle.make_pairformer_block_state(g, "")
    z, s, pm, sm = oracle.make_inputs(seed + 1, n, pad_frac=pad)
    z, s = z.to(BF), s.to(BF)
    rst = {k: v.to(BF).float() for k, v in st.items()}
    with torch.no_grad():
        rz, rs = oracle.pairformer_block(rst, "", z.float(), pm, s.float(), sm)
    return st, z, s, pm, sm, rz, rs


@pytest.mark.parametrize("n,pad", [(96, 0.0), (131, 0.1)])
def test_row_sharded_block_single_shard(ops, oracle, n, pad):
    from distributed_xfold_b200 import row_sharded
    st, z, s, pm, sm, rz, rs = _reference(oracle, n, 800 + n, pad)
    w = ops.PackedPairformerBlock(st, "", "cuda")
    sh = row_sharded.RowSharding(n)
    zd, sd = z.cuda().contiguous(), s.cuda().contiguous()
    pmd = pm.cuda()
    zd, sd = row_sharded.pairformer_block(sh, row_sharded.CudaStages(), zd, sd, pmd, pmd.t().contiguous(), sm.cuda(), w)
    ops.synchronize_and_check()
    assert relf(zd.float().cpu()[pm > 0], rz[pm > 0]) < 2e-2
    assert relf(sd.float().cpu()[sm > 0], rs[sm > 0]) < 2e-2
    assert relf((zd.float().cpu() - z.float())[pm > 0], (rz - z.float())[pm > 0]) < 3e-2


def _rank_main(rank, world, port, n, pad, use_peer, channel, ret):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    ge.load_package()
    O = ge.load_oracle()
    from distributed_xfold_b200 import ops, row_sharded
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    g = torch.Generator().manual_seed(900 + n)
    st = O.make_pairformer_block_state(g, "")
    z, s, pm, sm = O.make_inputs(901 + n, n, pad_frac=pad)
    w = ops.PackedPairformerBlock(st, "", f"cuda:{rank}")
    sh = row_sharded.RowSharding(n)
    if channel is not None:
        sh.force_channel_sharded = channel
    if use_peer:
        assert sh.enable_peer_exchange(f"cuda:{rank}"), getattr(sh, "peer_error", "")
        # at these sizes only the b operand (2 MB per rank) is above 1 MB: it takes the peer-store gather, as it does
        # at benchmark size with the default threshold
        sh.PEER_GATHER_MIN_BYTES = 1 << 20
    zd = z[sh.rows].to(BF).cuda().contiguous()
    sd = s.to(BF).cuda().contiguous()
    pmd = pm.cuda()
    zd, sd = row_sharded.pairformer_block(sh, row_sharded.CudaStages(), zd, sd, pmd, pmd.t().contiguous(), sm.cuda(), w)
    ops.synchronize_and_check(rank)
    full = sh.gather_rows(zd)
    if rank == 0:
        ret["z"], ret["s"] = full.float().cpu(), sd.float().cpu()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("use_peer,channel", [(False, None), (True, None), (True, True), (False, True)])
@pytest.mark.parametrize("n,pad", [(128, 0.0), (131, 0.1)])
def test_row_sharded_block_nccl_ranks(pkg, oracle, n, pad, use_peer, channel):
    """use_peer: the distributed transposes (and the exchanges of the channel-sharded contraction) run as peer-memory
    kernels of the library plus a bounded flag barrier; otherwise as pairwise send/recv.
    channel: force the channel-sharded TriangleMultiplication contraction (the default from 4 ranks on)."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two or more GPUs")
    from distributed_xfold_b200.distribute_utils import find_free_port
    st, z, s, pm, sm, rz, rs = _reference(oracle, n, 900 + n, pad)
    ret = mp.Manager().dict()
    mp.spawn(_rank_main, args=(world, find_free_port(), n, pad, use_peer, channel, ret), nprocs=world, join=True)
    assert relf(ret["z"][pm > 0], rz[pm > 0]) < 2e-2
    assert relf(ret["s"][sm > 0], rs[sm > 0]) < 2e-2


def _trunk_rank_main(rank, world, port, n, pad, nblocks, ret):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as ge
    ge.load_package()
    O = ge.load_oracle()
    from distributed_xfold_b200 import ops, row_sharded
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    st = O.make_pairformer_stack_state(700 + n, nblocks)
    z, s, pm, sm = O.make_inputs(701 + n, n, pad_frac=pad)
    stack = ops.PackedPairformerStack.from_state(st, nblocks, f"cuda:{rank}")
    sh = row_sharded.RowSharding(n)
    trunk = row_sharded.ShardedTrunk(sh, f"cuda:{rank}")
    sd = s.to(BF).cuda().contiguous()
    pmd, smd = pm.cuda().contiguous(), sm.cuda().contiguous()
    for rep in range(2):   # the second pass starts from buffers and flags the first one left behind
        trunk.load(z[sh.rows].to(BF).cuda())
        sd.copy_(s.to(BF).cuda())
        zs = trunk.run(sd, pmd, smd, stack)
        ops.synchronize_and_check(rank)
    full = sh.gather_rows(zs.contiguous())
    if rank == 0:
        ret["z"], ret["s"] = full.float().cpu(), sd.float().cpu()
    ref_rows, ref_s = zs.clone(), sd.clone()   # zs is a view of the trunk's buffer: copy before it is released
    if n % (8 * world) == 0:
        # even shards of whole tiles: the sharded path reproduces the one-GPU call bit for bit
        z1, s1 = z.to(BF).cuda().contiguous(), s.to(BF).cuda().contiguous()
        ops.pairformer_stack_(z1, s1, pmd, smd, stack)
        ops.synchronize_and_check(rank)
        assert torch.equal(z1[sh.rows], ref_rows) and torch.equal(s1, ref_s)
    dist.barrier()
    trunk.close()
    # a second instance, built with the overlap setting spelled out (one chunk: every exchange follows its GEMM), gives
    # the same bits
    for chunks, reserve in ((1, 0),):
        other = row_sharded.ShardedTrunk(sh, f"cuda:{rank}", chunks=chunks, reserved_sms=reserve)
        other.load(z[sh.rows].to(BF).cuda())
        sd.copy_(s.to(BF).cuda())
        zo = other.run(sd, pmd, smd, stack)
        ops.synchronize_and_check(rank)
        dz = float((zo.float() - ref_rows.float()).abs().max())
        ds = float((sd.float() - ref_s.float()).abs().max())
        assert dz == 0.0 and ds == 0.0, (chunks, reserve, dz, ds)
        dist.barrier()
        other.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("n,pad,nblocks", [(128, 0.0, 2), (131, 0.1, 2), (200, 0.1, 3)])
def test_sharded_trunk_one_call(pkg, oracle, n, pad, nblocks):
    """The whole stack of blocks on the row shards as ONE C-ABI call per rank (peer-memory exchanges and flag barriers
    inside; the incoming TriangleMultiplication on untransposed planes) against the fp32 oracle's block loop."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs two or more GPUs")
    from distributed_xfold_b200.distribute_utils import find_free_port
    st = {k: v.to(BF).float() for k, v in oracle.make_pairformer_stack_state(700 + n, nblocks).items()}
    z, s, pm, sm = oracle.make_inputs(701 + n, n, pad_frac=pad)
    rz, rs = z.to(BF).float(), s.to(BF).float()
    with torch.no_grad():
        for i in range(nblocks):
            rz, rs = oracle.pairformer_block(st, f"trunk_pairformer.{i}.", rz, pm, rs, sm)
    ret = mp.Manager().dict()
    mp.spawn(_trunk_rank_main, args=(world, find_free_port(), n, pad, nblocks, ret), nprocs=world, join=True)
    assert relf(ret["z"][pm > 0], rz[pm > 0]) < 2e-2
    assert relf(ret["s"][sm > 0], rs[sm > 0]) < 2e-2
