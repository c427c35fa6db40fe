"""PairformerBlock module (reference: nn/d_pairformer.py:32-171, DistributePairformerBlock) and the trunk's loop
over its blocks (reference: d_alphafold3.py:43-44, 242-244)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from ..distribute_utils import ShardInfo, init_dist_info
from .d_attention import DistributeGridSelfAttention
from .d_diffusion_transformer import DistributeSelfAttention
from .d_primitives import DistributeTransition, LayerNorm, Transition
from .d_triangle_multiplication import XSMMTriangleMultiplication


class DistributePairformerBlock(nn.Module):
    """``forward(pair, pair_mask, single, seq_mask)`` -> (pair, single).

    World size 1: the whole block is one C-ABI call, in place on bf16 copies of the inputs.
    dp_size > 1: every rank is given the FULL pair (as in the reference); the block runs on the rank's row
    shard with the pair representation kept sharded throughout, and the full pair is re-assembled at the end.
    Callers that keep the shard across blocks use ``row_sharded.pairformer_block`` directly and skip that gather.
    """

    def __init__(self, device_mesh, n_heads: int = 16, c_pair: int = 128, c_single: int = 384, c_hidden_mul: int = 128,
                 n_heads_pair: int = 4, num_intermediate_factor: int = 4, with_single: bool = True) -> None:
        super().__init__()
        init_dist_info(self, device_mesh)
        self.n_heads, self.with_single, self.c_pair, self.c_single = n_heads, with_single, c_pair, c_single
        self.num_intermediate_factor = num_intermediate_factor
        self.triangle_multiplication_outgoing = XSMMTriangleMultiplication(c_pair=c_pair, _outgoing=True)
        self.triangle_multiplication_incoming = XSMMTriangleMultiplication(c_pair=c_pair, _outgoing=False)
        self.pair_attention1 = DistributeGridSelfAttention(device_mesh, c_pair=c_pair, num_head=n_heads_pair, transpose=False)
        self.pair_attention2 = DistributeGridSelfAttention(device_mesh, c_pair=c_pair, num_head=n_heads_pair, transpose=True)
        self.pair_transition = DistributeTransition(device_mesh, c_x=c_pair, num_intermediate_factor=num_intermediate_factor)
        if with_single:
            self.single_pair_logits_norm = LayerNorm(c_pair)
            self.single_pair_logits_projection = nn.Linear(c_pair, n_heads, bias=False)
            self.single_attention_ = DistributeSelfAttention(device_mesh, c_x=c_single, num_head=n_heads,
                                                             use_single_cond=False, use_batch_infer=False)
            self.single_transition = Transition(c_x=c_single)
        self._packed = None

    def shard_params(self) -> None:
        if self.tp_size > 1:
            raise NotImplementedError("weight sharding (tp > 1) is outside the row-sharded hot path (trunk tp is 1)")

    def load_xsmm_params(self) -> None:
        self._packed = ops.PackedPairformerBlock(self.state_dict(), "", self.pair_transition.transition1.weight.device,
                                                 self.with_single)

    def xsmm_forward(self, pair: torch.Tensor, pair_mask: torch.Tensor, single: Optional[torch.Tensor] = None,
                     seq_mask: Optional[torch.Tensor] = None, head: int = 0):
        if self._packed is None:
            self.load_xsmm_params()
        ops._need_cuda(pair)
        z = pair.to(torch.bfloat16).contiguous()
        s = None if single is None else single.to(torch.bfloat16).contiguous()
        pm = pair_mask.float()
        sm = None if seq_mask is None else seq_mask.float()
        if not self.use_dp:
            ops.pairformer_block_(z, s if self.with_single else None, pm, sm, self._packed)
        else:
            from ..row_sharded import CudaStages, RowSharding, pairformer_block
            sh = RowSharding(z.shape[0], self.dp_shard_group)
            zs, s = pairformer_block(sh, CudaStages(), z[sh.rows].contiguous(), s if self.with_single else None, pm,
                                     pm.t().contiguous(), sm, self._packed)
            z = sh.gather_rows(zs)
        pair.copy_(z)
        if self.with_single:
            single.copy_(s)
            return pair, single
        return pair

    forward = xsmm_forward


class DistributePairformerStack(nn.Module):
    """The Pairformer part of the reference's ``DistributeEvoformer``: the module list ``trunk_pairformer``
    (d_alphafold3.py:43-44) and the loop over it (d_alphafold3.py:242-244); the confidence head runs the same
    loop over its four blocks (d_alphafold3.py:283-293).  Parameter names are ``trunk_pairformer.{i}.<block names>``,
    as in the reference's state dict.

    ``forward(pair, pair_mask, single, seq_mask)`` -> (pair, single).  World size 1: the whole loop is ONE C-ABI
    call.  dp_size > 1: the pair representation is cut into row shards once, stays sharded through all blocks
    (the reference re-assembles it after every block, nn/d_pairformer.py:134-156) and is gathered once at the end.
    """

    def __init__(self, device_mesh, num_layer: int = 48, with_single: bool = True, **block_args) -> None:
        super().__init__()
        init_dist_info(self, device_mesh)
        self.trunk_pairformer = nn.ModuleList(
            [DistributePairformerBlock(device_mesh, with_single=with_single, **block_args) for _ in range(num_layer)])
        self.with_single = with_single
        self._packed = None
        self._sharding = None

    def shard_params(self) -> None:
        for b in self.trunk_pairformer:
            b.shard_params()

    def load_xsmm_params(self) -> None:
        for b in self.trunk_pairformer:
            b.load_xsmm_params()
        self._packed = ops.PackedPairformerStack(b._packed for b in self.trunk_pairformer)

    def xsmm_forward(self, pair: torch.Tensor, pair_mask: torch.Tensor, single: Optional[torch.Tensor] = None,
                     seq_mask: Optional[torch.Tensor] = None):
        if self._packed is None:
            self.load_xsmm_params()
        ops._need_cuda(pair)
        z = pair.to(torch.bfloat16).contiguous()
        s = None if single is None or not self.with_single else single.to(torch.bfloat16).contiguous()
        pm = pair_mask.float()
        sm = None if seq_mask is None else seq_mask.float()
        if not self.use_dp:
            ops.pairformer_stack_(z, s, pm, sm, self._packed)
        else:
            from ..row_sharded import CudaStages, RowSharding, pairformer_stack
            sh = self._sharding
            if sh is None or sh.n != z.shape[0]:
                sh = self._sharding = RowSharding(z.shape[0], self.dp_shard_group)
                sh.enable_peer_exchange(z.device)
            zs, s = pairformer_stack(sh, CudaStages(), z[sh.rows].contiguous(), s, pm, pm.t().contiguous(), sm,
                                     self._packed)
            z = sh.gather_rows(zs)
        pair.copy_(z)
        if self.with_single:
            single.copy_(s)
            return pair, single
        return pair

    forward = xsmm_forward
