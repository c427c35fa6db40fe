"""LayerNorm / Transition modules (reference: nn/d_primitives.py:21-38; xfold.fastnn.LayerNorm)."""
from __future__ import annotations

import torch
import torch.nn as nn

from .. import ops
from ..distribute_utils import init_dist_info, shard_linear
from ._common import transition_update


class LayerNorm(nn.LayerNorm):
    """``xfold.fastnn.LayerNorm(c, elementwise_affine=True, bias=True)`` with eps 1e-5
    (call sites e.g. nn/d_triangle_multiplication.py:109-112); forward runs the CUDA kernel."""

    def __init__(self, c: int, elementwise_affine: bool = True, bias: bool = True, eps: float = 1e-5):
        super().__init__(c, eps=eps, elementwise_affine=elementwise_affine, bias=bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        ops._need_cuda(x)
        f = lambda t: None if t is None else t.detach().float().contiguous()
        return ops.layernorm(x.to(torch.bfloat16).contiguous(), f(self.weight), f(self.bias), self.eps).to(x.dtype)


class Transition(nn.Module):
    """LN -> Linear(c, 2*f*c) -> SiLU(first half) * second half -> Linear(f*c, c)
    (kernel_test/transition.py:24-43)."""

    def __init__(self, c_x: int, num_intermediate_factor: int = 4) -> None:
        super().__init__()
        self.c_x, self.num_intermediate_factor = c_x, num_intermediate_factor
        self.input_layer_norm = LayerNorm(c_x)
        self.transition1 = nn.Linear(c_x, 2 * num_intermediate_factor * c_x, bias=False)
        self.transition2 = nn.Linear(num_intermediate_factor * c_x, c_x, bias=False)
        self._packed = None

    def load_xsmm_params(self) -> None:
        self._packed = ops.PackedTransition(self.state_dict(), "", self.transition1.weight.device)

    def xsmm_forward(self, x: torch.Tensor) -> torch.Tensor:
        if self._packed is None:
            self.load_xsmm_params()
        return transition_update(x, self._packed)

    forward = xsmm_forward


class DistributeTransition(Transition):
    def __init__(self, device_mesh, c_x: int, num_intermediate_factor: int = 4) -> None:
        super().__init__(c_x, num_intermediate_factor)
        init_dist_info(self, device_mesh)

    def shard_params(self) -> None:
        """Weight sharding over the tp axis (reference :27-29). The trunk runs with tp = 1; a tp > 1 GLU
        pairs different gate/value columns than the unsharded layer (the reference has the same property),
        so the fused kernel is only used unsharded."""
        if self.tp_size > 1:
            raise NotImplementedError("Transition weight sharding (tp > 1) is outside the row-sharded hot path")
        self.transition1 = shard_linear(self.transition1, self.rank, self.device_mesh, True)
        self.transition2 = shard_linear(self.transition2, self.rank, self.device_mesh, False)
        self._packed = None
