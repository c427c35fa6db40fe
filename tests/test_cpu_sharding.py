"""CPU tests (gloo, world size 2 and 3): the row-sharded Pairformer block reproduces the unsharded
oracle when its stages are computed by the oracle-based stand-in, i.e. the distributed transposes,
the b / bias / pair-logit gathers, the incoming-as-transposed-outgoing rewrite and the mask
conventions are right.  Also the host-side sharding utilities against the reference's rule."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, n, ret, channel_sharded=None):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import __graft_entry__ as ge
    ge.load_package()
    O = ge.load_oracle()
    from distributed_xfold_b200 import row_sharded
    from distributed_xfold_b200.distribute_utils import setup_gloo, cleanup
    import stage_double
    torch.set_num_threads(1)
    setup_gloo(rank, world, port)
    g = torch.Generator().manual_seed(5)
    st = O.make_pairformer_block_state(g, "")
    z, s, pm, sm = O.make_inputs(6, n, pad_frac=0.15)
    sh = row_sharded.RowSharding(n)
    if channel_sharded is not None:
        sh.force_channel_sharded = channel_sharded
        assert sh.channel_sharded == channel_sharded
    zs, ss = z[sh.rows].clone(), s.clone()
    with torch.no_grad():
        zs, ss = row_sharded.pairformer_block(sh, stage_double.OracleStages(O), zs, ss, pm, pm.t().contiguous(), sm,
                                              stage_double.Weights(st, ""))
    full = sh.gather_rows(zs)
    if rank == 0:
        ret["z"], ret["s"] = full, ss
    dist.barrier()
    cleanup()


@pytest.mark.parametrize("world,n,channel_sharded", [(2, 24, None), (3, 20, None), (2, 17, None), (2, 17, True), (4, 22, None), (8, 30, None)])
def test_row_sharded_block_matches_oracle(pkg, oracle, world, n, channel_sharded):
    """channel_sharded: the contraction on channel slices (rows -> channels exchange, product, rows back) instead of the
    gather of b; it is the default from 4 ranks on, and forced at 2 ranks with a ragged shard."""
    from distributed_xfold_b200.distribute_utils import find_free_port
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, find_free_port(), n, ret, channel_sharded), nprocs=world, join=True)
    g = torch.Generator().manual_seed(5)
    st = oracle.make_pairformer_block_state(g, "")
    z, s, pm, sm = oracle.make_inputs(6, n, pad_frac=0.15)
    with torch.no_grad():
        rz, rs = oracle.pairformer_block(st, "", z, pm, s, sm)
    valid = pm > 0
    assert oracle.rel_frobenius(ret["z"][valid], rz[valid]) < 1e-4
    assert oracle.rel_frobenius(ret["s"][sm > 0], rs[sm > 0]) < 1e-4


def test_shard_info_matches_reference_rule(pkg, oracle, golden):
    from distributed_xfold_b200.distribute_utils import ShardInfo
    for key, val in golden.items():
        if key.startswith("shard_info/"):
            n, p = val["meta"]["n"], val["meta"]["p"]
            assert ShardInfo(n, p).get_shard_size_list() == val["out"] == oracle.ShardInfo(n, p).sizes
    s = ShardInfo(764, 8)
    assert s.get_shard_size_list() == [96] * 7 + [92] and s.get_per_chunk_size() == 96
    assert [(x.start, x.stop) for x in s.get_shard_slice_list()][-1] == (672, 764)


def test_device_mesh_and_shard_linear(pkg):
    from distributed_xfold_b200.distribute_utils import DeviceMesh, shard_linear
    m = DeviceMesh(8, dp_size=4, tp_size=2)
    assert m.device_mesh.tolist() == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert m.get_dp_shard_num(5) == 2 and m.get_tp_shard_num(5) == 1
    assert m.get_rank_coords(5).tolist() == [[2, 1]]
    with pytest.raises(ValueError):
        DeviceMesh(8, 3, 2)
    lin = torch.nn.Linear(6, 8, bias=True)
    col = shard_linear(lin, 5, m, out=True)      # tp rank 1 of 2: output rows 4..7
    assert torch.equal(col.weight, lin.weight[4:]) and torch.equal(col.bias, lin.bias[4:])
    row = shard_linear(lin, 4, m, out=False)     # tp rank 0: input columns 0..2, full bias
    assert torch.equal(row.weight, lin.weight[:, :3]) and torch.equal(row.bias, lin.bias)
    with pytest.raises(TypeError):
        shard_linear(torch.nn.ReLU(), 0, m)


@pytest.mark.parametrize("world,n", [(2, 511), (3, 625), (4, 1022), (8, 1001)])
def test_peer_gather_branch_is_the_same_on_every_rank(pkg, world, n):
    """With ragged shards a rank's own byte count straddles any size threshold (N = 511 on 2 ranks: 256 and 255 rows,
    exactly 32 MiB and just below).  The choice between the peer-store gather and the library collective must not
    depend on it, or one rank waits at the flag barrier while the other sits in a collective."""
    from distributed_xfold_b200 import row_sharded
    ld = (n + 7) // 8 * 8
    row_bytes = 128 * ld * 2                                    # one row of the b operand [rows, 128, ld]
    shards = [row_sharded.RowSharding(n, world=world, rank=r) for r in range(world)]
    assert len({sh.r for sh in shards}) > 1                     # the partition is ragged
    for threshold in (shards[0].r * row_bytes, shards[-1].r * row_bytes + 16, n * row_bytes, n * row_bytes + 16, 1):
        picks = []
        for sh in shards:
            sh.peer = object()                                  # peer exchange available on every rank
            sh.PEER_GATHER_MIN_BYTES = threshold
            picks.append(sh.uses_peer_gather(row_bytes, operand_b=True))
            assert not sh.uses_peer_gather(row_bytes, operand_b=False)   # bias / logit gathers never take the peer buffer
        assert len(set(picks)) == 1, (threshold, picks)
