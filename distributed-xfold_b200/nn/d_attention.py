"""TriangleAttention module (reference: nn/d_attention.py:23-111, DistributeGridSelfAttention)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..distribute_utils import init_dist_info
from ._common import triattn_update
from .d_primitives import LayerNorm


class DistributeGridSelfAttention(nn.Module):
    """``forward(pair, mask, full_pair=None)`` returns the update.  ``transpose=True`` is the ending node;
    the pair bias comes from ``full_pair`` and is not transposed (reference :62, :99)."""

    def __init__(self, device_mesh, c_pair: int = 128, num_head: int = 4, transpose: bool = False):
        super().__init__()
        if c_pair != 128 or num_head != 4:
            raise ValueError("the sm_100a TriangleAttention kernel is built for c_pair = 128, 4 heads of 32")
        self.c_pair, self.num_head, self.transpose = c_pair, num_head, transpose
        self.qkv_dim = c_pair // num_head
        self.act_norm = LayerNorm(c_pair)
        self.pair_bias_projection = nn.Linear(c_pair, num_head, bias=False)
        self.q_projection = nn.Linear(c_pair, c_pair, bias=False)
        self.k_projection = nn.Linear(c_pair, c_pair, bias=False)
        self.v_projection = nn.Linear(c_pair, c_pair, bias=False)
        self.gating_query = nn.Linear(c_pair, c_pair, bias=False)
        self.output_projection = nn.Linear(c_pair, c_pair, bias=False)
        init_dist_info(self, device_mesh)
        self._packed = None

    def shard_params(self) -> None:
        if self.tp_size > 1:
            raise NotImplementedError("head sharding (tp > 1) is outside the row-sharded hot path (trunk tp is 1)")

    def load_xsmm_params(self) -> None:
        self._packed = ops.PackedTriAttn(self.state_dict(), "", self.q_projection.weight.device, self.num_head)
        self.key_dim = self.value_dim = self.qkv_dim

    def xsmm_forward(self, pair: torch.Tensor, mask: torch.Tensor, full_pair=None) -> torch.Tensor:
        if self._packed is None:
            self.load_xsmm_params()
        if full_pair is None or full_pair is pair or full_pair.shape == pair.shape:
            if full_pair is not None and full_pair is not pair and not torch.equal(full_pair, pair):
                raise ValueError("with an unsharded pair, full_pair must be the pair itself")
            return triattn_update(pair, mask, self._packed, self.transpose)
        # row shard (starting node) / column shard (ending node) with the bias taken from the full pair
        fp = full_pair.to(torch.bfloat16).contiguous()
        _, bias_t = ops.stage_triattn_bias(fp, self._packed, False)      # [4, N, pad8(N)], [head, query, key]
        n = fp.shape[0]
        z = pair.transpose(0, 1) if self.transpose else pair
        z = z.to(torch.bfloat16).contiguous()
        x, _ = ops.stage_triattn_bias(z, self._packed, False)            # x = act_norm(shard)
        upd = torch.zeros_like(z)
        ops.stage_triattn_core(x, bias_t, mask, self._packed, upd)
        upd = upd.transpose(0, 1) if self.transpose else upd
        return upd.to(pair.dtype)

    forward = xsmm_forward
