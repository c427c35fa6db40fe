"""Pairformer block on a pair representation partitioned by token rows over the ranks of one
process group (one process per GPU) -- the layout of the reference's 'dp' axis in the trunk
(nn/d_pairformer.py:119-156, distribute_utils.py:101-128), taken one step further: the pair
representation STAYS sharded through the whole block, TriangleMultiplication included (the
reference's sharded TriMul, nn/d_triangle_multiplication.py:48-99, is written but not wired in).

Per block and rank, with R = rows held by the rank and zT the row shard of the transposed pair
representation (zT[j][i] = z[i][j]):

    z   : TriMul outgoing        gather b rows            (all-gather, N*N*c / P elements per peer), or from 4 ranks
                                                          on: a, b to channel slices, product, output rows back
    zT  : TriMul incoming        the same                 'ckj,cki->cij' on z is 'cik,cjk->cij' on zT
    z   : TriAttn starting node  gather the pair bias     (4 * N * N bf16 in total, [head, query, key])
    zT  : TriAttn ending node    gather the pair bias, then pair Transition (token-local)
    z   : pair logits, gathered; the single path is replicated on every rank (it is < 1 % of the work)

with a distributed transpose (all-to-all of R x R_peer blocks) between the layouts, in place of the
reference's two all-gathers of the whole pair representation per block (nn/d_pairformer.py:134-155).

The arithmetic is delegated to a *stage backend*: ``CudaStages`` calls the sm_100a kernels through
the C ABI; the CPU tests plug in a double built on the oracle to check the sharding algebra under
gloo.  Nothing in this file computes on tensors itself except the layout glue.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist

from .distribute_utils import ShardInfo


def _exchange(send: List[torch.Tensor], recv: List[torch.Tensor], group) -> None:
    """Pairwise exchange: send[q] goes to group rank q, recv[p] arrives from group rank p."""
    me = dist.get_rank(group)
    world = dist.get_world_size(group)
    recv[me].copy_(send[me])
    ops = []
    for off in range(1, world):
        dst, src = (me + off) % world, (me - off) % world
        ops.append(dist.P2POp(dist.isend, send[dst], dist.get_global_rank(group, dst) if group is not None else dst,
                              group))
        ops.append(dist.P2POp(dist.irecv, recv[src], dist.get_global_rank(group, src) if group is not None else src,
                              group))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()


class RowSharding:
    """Row partition of an N-token pair representation over a process group."""

    def __init__(self, n_tokens: int, group=None, world: Optional[int] = None, rank: Optional[int] = None):
        self.group = group
        # world / rank may be given explicitly to work out a partition without a process group
        self.world = world if world is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        self.n = n_tokens
        info = ShardInfo(n_tokens, self.world)
        self.sizes, self.slices = info.shard_size_list, info.shard_slice_list
        self.rows = self.slices[self.rank]
        self.r = self.sizes[self.rank]

    # -- collectives on shards -------------------------------------------------------------------
    # A gather smaller than this (in bytes of the GATHERED tensor) stays with the library collective.
    PEER_GATHER_MIN_BYTES = 32 << 20

    def uses_peer_gather(self, row_bytes: int, operand_b: bool) -> bool:
        """Whether ``gather_rows`` takes the peer-store path.  Every rank must come to the same answer, or one side
        would wait at the flag barrier while the other sits in a library collective: so the test uses only what
        all ranks share -- the caller's statement that this is the b operand of the TriangleMultiplication, the
        token count and the bytes per gathered row (never this rank's own row count, which differs on ragged
        partitions)."""
        return bool(operand_b) and getattr(self, "peer", None) is not None and self.n * row_bytes >= self.PEER_GATHER_MIN_BYTES

    def gather_rows(self, local: torch.Tensor, operand_b: bool = False) -> torch.Tensor:
        """[R_me, ...] on every rank -> [N, ...] (ragged row counts allowed).  ``operand_b``: the tensor is the b operand
        of the TriangleMultiplication contraction, the one gather that may go through the peer-mapped buffer (see
        ``PeerExchange.gather_rows`` for why only that one)."""
        if self.world == 1:
            return local
        if local.is_cuda and local.dtype == torch.bfloat16 and self.uses_peer_gather(2 * math.prod(local.shape[1:]), operand_b):
            return self.peer.gather_rows(local)
        out = local.new_empty((self.n,) + tuple(local.shape[1:]))
        if len(set(self.sizes)) == 1:
            dist.all_gather_into_tensor(out, local.contiguous(), group=self.group)
            return out
        pad = max(self.sizes)
        buf = local.new_zeros((pad,) + tuple(local.shape[1:]))
        buf[: self.r] = local
        parts = [torch.empty_like(buf) for _ in range(self.world)]
        dist.all_gather(parts, buf, group=self.group)
        for p, (sl, sz) in enumerate(zip(self.slices, self.sizes)):
            out[sl] = parts[p][:sz]
        return out

    def gather_last_dim(self, local: torch.Tensor, pitch: int) -> torch.Tensor:
        """[..., R_me] on every rank -> [..., pitch] whose first N entries are the concatenation."""
        parts = self.gather_rows(local.movedim(-1, 0).contiguous()) if self.world > 1 else local.movedim(-1, 0)
        out = local.new_zeros(tuple(local.shape[:-1]) + (pitch,))
        out[..., : self.n] = parts.movedim(0, -1)
        return out

    def enable_peer_exchange(self, device) -> bool:
        """Switches ``transpose`` to the one-kernel peer-memory exchange over NVLink (symmetric-memory
        buffers mapped into every rank + the C-ABI scatter / flag-barrier kernels).  Returns False, and keeps
        the send/recv path, when symmetric memory cannot be set up."""
        if self.world == 1:
            return False
        try:
            self.peer = PeerExchange(self, device)
            return True
        except Exception as e:  # pragma: no cover - depends on the machine's P2P capabilities
            self.peer = None
            self.peer_error = repr(e)
            return False

    # -- channel-sharded TriangleMultiplication contraction -------------------------------------------
    @property
    def channel_sharded(self) -> bool:
        """The contraction 'cik,cjk->cij' is independent per channel.  Gathering b on every rank moves
        (P-1)/P * N^2 c elements into each rank; handing every rank 128 / P channels of a and b for ALL rows and
        sending its output rows back moves (P-1)/P * 3 N^2 c / P: less from P = 4 on."""
        forced = getattr(self, "force_channel_sharded", None)
        if forced is not None:
            return bool(forced) and 128 % self.world == 0 and self.world > 1
        return self.world >= 4 and 128 % self.world == 0

    def rows_to_channels(self, a: torch.Tensor, b: torch.Tensor):
        """a, b [R_me, 128, ld] -> planes [128 / P, N, ld] of this rank's channels, all rows."""
        if getattr(self, "peer", None) is not None and a.is_cuda:
            return self.peer.rows_to_channels(a, b)
        cq = 128 // self.world
        out = []
        for t in (a, b):
            send = [t[:, q * cq:(q + 1) * cq, :].transpose(0, 1).contiguous() for q in range(self.world)]   # [cq, R_me, ld]
            recv = [t.new_empty((cq, sz, t.shape[2])) for sz in self.sizes]
            _exchange(send, recv, self.group)
            out.append(torch.cat(recv, dim=1))
        return out[0], out[1]

    def channels_to_rows(self, o: torch.Tensor) -> torch.Tensor:
        """o [128 / P, N, ldo] of this rank's channels -> [R_me, 128, ldo] of this rank's rows, all channels."""
        if getattr(self, "peer", None) is not None and o.is_cuda:
            return self.peer.channels_to_rows(o)
        send = [o[:, sl, :].transpose(0, 1).contiguous() for sl in self.slices]                              # [R_q, cq, ldo]
        recv = [o.new_empty((self.r, o.shape[0], o.shape[2])) for _ in range(self.world)]
        _exchange(send, recv, self.group)
        return torch.cat(recv, dim=1)

    def transpose(self, z: torch.Tensor) -> torch.Tensor:
        """Row shard of z [R_me, N, c] -> row shard of z^T: out[j_local, i] = z_global[i, j_global]."""
        if self.world == 1:
            return z.transpose(0, 1).contiguous()
        if getattr(self, "peer", None) is not None and z.is_cuda:
            return self.peer.transpose(z)
        c = z.shape[-1]
        send = [z[:, sl, :].transpose(0, 1).contiguous() for sl in self.slices]          # to q: [R_q, R_me, c]
        recv = [z.new_empty((self.r, sz, c)) for sz in self.sizes]                       # from p: [R_me, R_p, c]
        _exchange(send, recv, self.group)
        return torch.cat(recv, dim=1)


class PeerExchange:
    """Distributed transpose through peer-mapped memory: each rank stores its tokens directly into the
    owning rank's buffer with one kernel (``xfold_transpose_scatter_fwd``), then the ranks meet at a bounded
    flag barrier (``xfold_peer_barrier``).  Two buffers alternate, so a buffer is rewritten only after the
    barrier that follows its last read (the ordering argument is written out in the header comment of csrc/peer.cu)."""

    def __init__(self, sh: "RowSharding", device, channels: int = 128):
        import torch.distributed._symmetric_memory as symm
        from . import peer_ops as ops
        self.sh, self.ops, self.c = sh, ops, channels
        group = sh.group if sh.group is not None else dist.group.WORLD
        rmax = max(sh.sizes)
        self.bufs, self.ptrs = [], []
        for _ in range(2):
            t = symm.empty(rmax * sh.n * channels, dtype=torch.bfloat16, device=device)
            h = symm.rendezvous(t, group)
            off = t.data_ptr() - int(h.buffer_ptrs[sh.rank])
            self.bufs.append(t)
            self.ptrs.append([int(p) + off for p in h.buffer_ptrs])
        self.flags = symm.empty(8, dtype=torch.int32, device=device)
        self.flags.zero_()
        h = symm.rendezvous(self.flags, group)
        off = self.flags.data_ptr() - int(h.buffer_ptrs[sh.rank])
        self.flag_ptrs = [int(p) + off for p in h.buffer_ptrs]
        self.starts = [sl.start for sl in sh.slices] + [sh.n]
        self.k = 0
        self.epoch = 0
        self.symm, self.group = symm, group
        self.planes = None  # buffers of the channel-sharded contraction, made on first use
        torch.cuda.synchronize(device)
        dist.barrier(group=sh.group)  # every rank's flags are zero before anyone signals

    def transpose(self, z: torch.Tensor) -> torch.Tensor:
        sh = self.sh
        z = z.contiguous()
        k = self.k
        if z.data_ptr() == self.bufs[k].data_ptr():  # never scatter a buffer into itself
            k ^= 1
        self.ops.transpose_scatter(z, sh.rows.start, self.ptrs[k], self.starts)
        self.epoch += 1
        self.ops.peer_barrier(self.flag_ptrs, sh.rank, sh.world, self.epoch, z.device)
        self.k = k ^ 1
        return self.bufs[k][: sh.r * sh.n * self.c].view(sh.r, sh.n, self.c)


    # -- all-gather of the b operand of the TriangleMultiplication by peer stores ------------------------
    # One buffer serves every such gather.  Ordering: the peers store into it at TriangleMultiplication t + 1 only
    # after they passed the flag barrier of the distributed transpose that lies between TriangleMultiplication t and
    # t + 1 in every block (and between the last one of a block and the first one of the next); a rank signals that
    # barrier in stream order AFTER its contraction kernel of TriangleMultiplication t, the only reader of the
    # buffer.  So every read of gather t has finished before any store of gather t + 1 starts.  No other gather has
    # a barrier between its consumer and the next writer, which is why RowSharding.gather_rows sends only the
    # b operand here (its callers say so explicitly; the size of a tensor never decides it) and the pair bias and
    # pair logits stay with the library collective.

    def gather_rows(self, local: torch.Tensor) -> torch.Tensor:
        sh = self.sh
        local = local.contiguous()
        row_bytes = local[0].numel() * 2
        if row_bytes % 16 or local.data_ptr() % 16:
            raise ValueError("peer gather needs 16-byte aligned rows")
        total = sh.n * row_bytes
        g = getattr(self, "gbuf", None)
        if g is None or g["bytes"] < total:
            t = self.symm.empty(total // 2, dtype=torch.bfloat16, device=local.device)
            h = self.symm.rendezvous(t, self.group)
            off = t.data_ptr() - int(h.buffer_ptrs[sh.rank])
            torch.cuda.synchronize(local.device)
            dist.barrier(group=sh.group)
            g = self.gbuf = {"bytes": total, "t": t, "ptrs": [int(p) + off for p in h.buffer_ptrs]}
        self.ops.peer_allgather(local, sh.rows.start * row_bytes, g["ptrs"])
        self._barrier(local.device)
        return g["t"][: total // 2].view((sh.n,) + tuple(local.shape[1:]))

    # -- channel-sharded contraction: operand planes and output rows in peer-mapped buffers ------------
    def _plane_buffers(self, ld: int, ldo: int, device):
        sh = self.sh
        if self.planes is not None and self.planes["ld"] == ld and self.planes["ldo"] == ldo:
            return self.planes
        cq, rmax = 128 // sh.world, max(sh.sizes)
        bufs = {"ld": ld, "ldo": ldo}
        for name, numel in (("a", cq * sh.n * ld), ("b", cq * sh.n * ld), ("o", rmax * 128 * ldo)):
            t = self.symm.empty(numel, dtype=torch.bfloat16, device=device)
            if ld != sh.n or ldo != sh.n:
                t.zero_()  # pad columns stay zero: the scatters only ever write whole rows of the same pitch
            h = self.symm.rendezvous(t, self.group)
            off = t.data_ptr() - int(h.buffer_ptrs[sh.rank])
            bufs[name] = t
            bufs[name + "_ptrs"] = [int(p) + off for p in h.buffer_ptrs]
        torch.cuda.synchronize(device)
        dist.barrier(group=sh.group)
        self.planes = bufs
        return bufs

    def _barrier(self, device):
        self.epoch += 1
        self.ops.peer_barrier(self.flag_ptrs, self.sh.rank, self.sh.world, self.epoch, device)

    def rows_to_channels(self, a: torch.Tensor, b: torch.Tensor):
        sh = self.sh
        ld = a.shape[2]
        p = self._plane_buffers(ld, (sh.n + 7) // 8 * 8, a.device)
        self.ops.scatter_channels(a.contiguous(), b.contiguous(), sh.n, sh.rows.start, p["a_ptrs"], p["b_ptrs"])
        self._barrier(a.device)
        cq = 128 // sh.world
        return p["a"].view(cq, sh.n, ld), p["b"].view(cq, sh.n, ld)

    def channels_to_rows(self, o: torch.Tensor) -> torch.Tensor:
        sh = self.sh
        p = self._plane_buffers(self.planes["ld"], o.shape[2], o.device)
        cq = 128 // sh.world
        self.ops.scatter_rows(o.contiguous(), sh.rank * cq, p["o_ptrs"], self.starts)
        self._barrier(o.device)
        return p["o"][: sh.r * 128 * o.shape[2]].view(sh.r, 128, o.shape[2])


class ShardedTrunk:
    """The row-sharded block / trunk as ONE C-ABI call per stack of blocks (``xfold_pairformer_stack_sharded_fwd``): this
    class only sets up what that call needs -- the peer-mapped (symmetric-memory) buffers every rank's kernels store
    into, handed to the library as a shard context -- and keeps the pair shard in one of those buffers between calls.
    World sizes 2, 4 and 8 (the channel slices of the TriangleMultiplication need 128 % world == 0); for anything else,
    and on the CPU, ``pairformer_block`` above composes the same stages with collectives."""

    def __init__(self, sh: "RowSharding", device, chunks: Optional[int] = None, reserved_sms: int = 0):
        import ctypes as C
        import torch.distributed._symmetric_memory as symm
        from . import _cabi
        if sh.world not in (2, 4, 8):
            raise ValueError("ShardedTrunk: 2, 4 or 8 ranks")
        self.sh, self._cabi, self._C = sh, _cabi, C
        self.device = torch.device(device)
        self.dev = self.device.index
        group = sh.group if sh.group is not None else dist.group.WORLD
        n, world, rmax = sh.n, sh.world, max(sh.sizes)
        ld = (n + 7) // 8 * 8
        cq = 128 // world
        self.ld = ld
        self._keep = []

        def shared(numel, dtype=torch.bfloat16, zero=False):
            t = symm.empty(numel, dtype=dtype, device=self.device)
            if zero:
                t.zero_()
            h = symm.rendezvous(t, group)
            off = t.data_ptr() - int(h.buffer_ptrs[sh.rank])
            self._keep.append((t, h))
            return t, (C.c_void_p * world)(*[int(p) + off for p in h.buffer_ptrs])

        self.zbuf = [None, None]
        self.zbuf[0], z0p = shared(rmax * n * 128)
        self.zbuf[1], z1p = shared(rmax * n * 128)
        _, pa = shared(cq * n * ld, zero=ld != n)
        _, pb = shared(cq * n * ld, zero=ld != n)
        _, po = shared(rmax * 128 * ld, zero=ld != n)
        _, bias = shared(16 * n * ld, zero=True)
        _, flags = shared(8, dtype=torch.int32, zero=True)
        starts = (C.c_int * (world + 1))(*([sl.start for sl in sh.slices] + [n]))
        self._ptrs = (z0p, z1p, pa, pb, po, bias, flags, starts)
        desc = _cabi.ShardDesc(world, sh.rank, n, starts, z0p, z1p, pa, pb, po, bias, flags)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=sh.group)  # every rank's flags are zero before anyone signals
        lib = _cabi.load()
        out = C.c_void_p()
        _cabi.check(lib.xfold_shard_ctx_create(_cabi.ctx(self.dev), C.byref(desc), C.byref(out)), self.dev,
                    "xfold_shard_ctx_create")
        self.handle = out.value
        if chunks is not None:   # chunks of a producing stage whose rows travel while the next chunk is computed
            _cabi.check(lib.xfold_shard_ctx_set_overlap(self.handle, int(chunks), int(reserved_sms)), self.dev,
                        "xfold_shard_ctx_set_overlap")
        self.ws = torch.empty(lib.xfold_shard_workspace_bytes(self.handle), dtype=torch.uint8, device=self.device)
        self.slot = 0

    def shard_view(self, slot: Optional[int] = None) -> torch.Tensor:
        """This rank's rows [R, N, 128] inside the peer-mapped buffer that currently holds them."""
        sh = self.sh
        k = self.slot if slot is None else slot
        return self.zbuf[k][: sh.r * sh.n * 128].view(sh.r, sh.n, 128)

    def load(self, z_shard: torch.Tensor) -> None:
        """Copies this rank's rows into the library's buffer (the one copy a caller with its own z tensor needs)."""
        self.shard_view().copy_(z_shard)

    def run(self, s: Optional[torch.Tensor], pair_mask: torch.Tensor, seq_mask: Optional[torch.Tensor], stack) -> torch.Tensor:
        """Runs every block of ``stack`` (an ops.PackedPairformerStack) on the shard held in the buffer; returns the view of
        the updated rows.  pair_mask: the full [N, N] float32 mask (replicated); s: bf16 [N, 384], updated in place."""
        C, _cabi = self._C, self._cabi
        lib = _cabi.load()
        out = C.c_int(self.slot)
        stream = torch.cuda.current_stream(self.dev).cuda_stream
        rc = lib.xfold_pairformer_stack_sharded_fwd(_cabi.ctx(self.dev), self.handle, self.slot,
                                                    None if s is None else s.data_ptr(), pair_mask.data_ptr(),
                                                    None if seq_mask is None else seq_mask.data_ptr(), stack.c, len(stack),
                                                    self.ws.data_ptr(), self.ws.numel(), stream, C.byref(out))
        _cabi.check(rc, self.dev, "xfold_pairformer_stack_sharded_fwd")
        self.slot = out.value
        return self.shard_view()

    def close(self) -> None:
        if self.handle:
            self._cabi.load().xfold_shard_ctx_destroy(self.handle)
            self.handle = None


class CudaStages:
    """Stage backend on the C ABI (sm_100a kernels)."""

    def __init__(self):
        from . import ops
        self.ops = ops

    def __getattr__(self, name):
        return getattr(self.ops, "stage_" + name)


def _contract(sh: RowSharding, stages, a: torch.Tensor, b: torch.Tensor, n: int) -> torch.Tensor:
    """o[i, c, j] = sum_k a[i, c, k] b[j, c, k] for this rank's rows i: either against the gathered rows of b, or, from
    four ranks on, per channel slice on all rows with an exchange before and after (see RowSharding.channel_sharded)."""
    if sh.channel_sharded:
        ap, bp = sh.rows_to_channels(a, b)
        return sh.channels_to_rows(stages.trimul_contract_planes(ap, bp, n))
    return stages.trimul_contract(a, sh.gather_rows(b, operand_b=True), n)


def pairformer_block(sh: RowSharding, stages, z: torch.Tensor, s: Optional[torch.Tensor], pair_mask: torch.Tensor,
                     pair_mask_t: torch.Tensor, seq_mask: Optional[torch.Tensor], w) -> tuple:
    """One block.  z: this rank's rows [R, N, c] (updated, returned); s: replicated [N, c_s];
    pair_mask / pair_mask_t: the full [N, N] mask and its transpose (replicated, float32)."""
    n, rows = sh.n, sh.rows
    ldq = (n + 7) // 8 * 8
    # TriangleMultiplication, outgoing edges, on z
    a, b, g = stages.trimul_project(z, pair_mask[rows], w.tri_out)
    stages.trimul_output(_contract(sh, stages, a, b, n), g, z, w.tri_out)
    # incoming edges: the same product on the transposed layout
    zt = sh.transpose(z)
    a, b, g = stages.trimul_project(zt, pair_mask_t[rows], w.tri_in)
    stages.trimul_output(_contract(sh, stages, a, b, n), g, zt, w.tri_in)
    del a, b, g
    # TriangleAttention, starting node, on z: the local rows are QUERY rows of the bias [head, query, key]
    z = sh.transpose(zt)
    x, bias_loc = stages.triattn_bias(z, w.att_start, False)          # [4, R, ldq]
    bias = sh.gather_rows(bias_loc.transpose(0, 1).contiguous()).transpose(0, 1).contiguous()   # [4, N, ldq]
    stages.triattn_core(x, bias, pair_mask[rows], w.att_start, z)
    # ending node on zT: token zT[j][i] is pair (i, j), so the local rows are KEY rows of the bias;
    # the mask rows are the ones the reference passes (pair_mask[shard])
    zt = sh.transpose(z)
    x, bias_loc = stages.triattn_bias(zt, w.att_end, True)            # [4, N, R]
    bias = sh.gather_last_dim(bias_loc, ldq)                          # [4, N, ldq]
    stages.triattn_core(x, bias, pair_mask[rows], w.att_end, zt)
    del x, bias, bias_loc
    stages.transition(zt, w.pair_transition)
    z = sh.transpose(zt)
    if s is not None and w.with_single:
        pl_loc = stages.pair_logits(z, w)                             # [16, R, ldq]
        pl = sh.gather_rows(pl_loc.transpose(0, 1).contiguous()).transpose(0, 1).contiguous()
        stages.single_update(s, pl, seq_mask, w)
    return z, s


def trimul_out_in(sh: RowSharding, stages, z: torch.Tensor, pair_mask: torch.Tensor, pair_mask_t: torch.Tensor,
                  w_out, w_in) -> torch.Tensor:
    """z += TriMul_outgoing(z); z += TriMul_incoming(z) on the row shard (nn/d_pairformer.py:122-123 with the sharded
    form of nn/d_triangle_multiplication.py:48-99): the first two sub-layers of a block, also timed on their own."""
    n, rows = sh.n, sh.rows
    a, b, g = stages.trimul_project(z, pair_mask[rows], w_out)
    stages.trimul_output(_contract(sh, stages, a, b, n), g, z, w_out)
    zt = sh.transpose(z)
    a, b, g = stages.trimul_project(zt, pair_mask_t[rows], w_in)
    stages.trimul_output(_contract(sh, stages, a, b, n), g, zt, w_in)
    return sh.transpose(zt)


def pairformer_stack(sh: RowSharding, stages, z: torch.Tensor, s: Optional[torch.Tensor], pair_mask: torch.Tensor,
                     pair_mask_t: torch.Tensor, seq_mask: Optional[torch.Tensor], blocks) -> tuple:
    """The trunk loop (d_alphafold3.py:242-244) on the row shard: z stays sharded from the first block to the last."""
    for w in blocks:
        z, s = pairformer_block(sh, stages, z, s, pair_mask, pair_mask_t, seq_mask, w)
    return z, s
