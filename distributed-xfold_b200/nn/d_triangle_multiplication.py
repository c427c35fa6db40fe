"""TriangleMultiplication modules (reference: nn/d_triangle_multiplication.py:22-191)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..distribute_utils import init_dist_info
from ._common import trimul_update
from .d_primitives import LayerNorm


class XSMMTriangleMultiplication(nn.Module):
    """Unsharded TriMul; ``forward(pair, mask)`` returns the update [N, N, c_pair].
    Outgoing: 'cik,cjk->cij'; incoming: 'ckj,cki->cij' (reference :122-124)."""

    def __init__(self, c_pair: int = 128, _outgoing: bool = True) -> None:
        super().__init__()
        if c_pair != 128:
            raise ValueError("the sm_100a TriangleMultiplication kernels are built for c_pair = 128")
        self.c_pair = c_pair
        self.left_norm_input = LayerNorm(c_pair)
        self.projection = nn.Linear(c_pair, 2 * c_pair, bias=False)
        self.gate = nn.Linear(c_pair, 2 * c_pair, bias=False)
        self.center_norm = LayerNorm(c_pair)
        self.output_projection = nn.Linear(c_pair, c_pair, bias=False)
        self.gating_linear = nn.Linear(c_pair, c_pair, bias=False)
        self._outgoing = _outgoing
        self.c_equation = "ikc,jkc->ijc" if _outgoing else "kjc,kic->ijc"
        self.equation = "cik,cjk->cij" if _outgoing else "ckj,cki->cij"
        self._packed = None

    def load_xsmm_params(self) -> None:
        """Packs the weights for the kernels: a/b de-interleaved (even/odd rows), bf16 (reference :126-138).
        The module's own parameters are left as they are."""
        self._packed = ops.PackedTriMul(self.state_dict(), "", self.projection.weight.device)

    def xsmm_forward(self, pair: torch.Tensor, mask: torch.Tensor, head: int = 0) -> torch.Tensor:
        if self._packed is None:
            self.load_xsmm_params()
        return trimul_update(pair, mask, self._packed, self._outgoing)

    forward = xsmm_forward


class DistributeTriangleMultiplication(XSMMTriangleMultiplication):
    """Row-/column-sharded TriMul (reference :22-99): outgoing takes the row shard [N/P, N, c], incoming the
    column shard [N, N/P, c]; b is all-gathered over the dp group.  Returns the shard's update."""

    def __init__(self, device_mesh, c_pair: int = 128, _outgoing: bool = True) -> None:
        super().__init__(c_pair, _outgoing)
        init_dist_info(self, device_mesh)

    def shard_params(self) -> None:
        if self.tp_size > 1:
            raise NotImplementedError("channel sharding (tp > 1) of TriMul is outside the row-sharded hot path")

    def xsmm_forward(self, pair: torch.Tensor, mask: torch.Tensor, head: int = 0) -> torch.Tensor:
        if not self.use_dp:
            return super().xsmm_forward(pair, mask, head)
        from ..row_sharded import RowSharding
        if self._packed is None:
            self.load_xsmm_params()
        n = max(pair.shape[:-1])
        sh = RowSharding(n, self.dp_shard_group)
        # incoming on a column shard is the outgoing product on its transpose (rows = the shard's columns)
        z = pair if self._outgoing else pair.transpose(0, 1)
        m = mask if (mask is None or self._outgoing) else mask.transpose(0, 1)
        z = z.to(torch.bfloat16).contiguous()
        a, b, g = ops.stage_trimul_project(z, m, self._packed)
        o = ops.stage_trimul_contract(a, sh.gather_rows(b), n)
        upd = torch.zeros_like(z)
        ops.stage_trimul_output(o, g, upd, self._packed)     # 0 + update
        upd = upd if self._outgoing else upd.transpose(0, 1)
        return upd.to(pair.dtype)

    forward = xsmm_forward
