"""Diffusion-transformer modules (reference: nn/d_diffusion_transformer.py:37-310)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from .. import diffusion, ops
from ..distribute_utils import init_dist_info
from .d_primitives import LayerNorm

BF16 = torch.bfloat16


def _b(x):
    ops._need_cuda(x)
    return x.to(BF16).contiguous()


class AdaptiveLayerNorm(nn.Module):
    """sigmoid(Linear_b(LN_nb(cond))) * LN_noaffine(x) + Linear_nb(LN_nb(cond)); plain LayerNorm without
    conditioning (reference :37-74)."""

    def __init__(self, c_x: int, c_single_cond: int, use_single_cond: bool = False) -> None:
        super().__init__()
        self.c_x, self.c_single_cond, self.use_single_cond = c_x, c_single_cond, use_single_cond
        if use_single_cond:
            self.layer_norm = LayerNorm(c_x, elementwise_affine=False, bias=False)
            self.single_cond_layer_norm = LayerNorm(c_single_cond, bias=False)
            self.single_cond_scale = nn.Linear(c_single_cond, c_x, bias=True)
            self.single_cond_bias = nn.Linear(c_single_cond, c_x, bias=False)
        else:
            self.layer_norm = LayerNorm(c_x)
        self._packed = None

    def forward(self, x: torch.Tensor, single_cond: Optional[torch.Tensor] = None) -> torch.Tensor:
        assert (single_cond is None) == (self.use_single_cond is False)
        if not self.use_single_cond:
            return self.layer_norm(x)
        if self._packed is None:
            self._packed = diffusion._PackedAdaLN(self.state_dict(), "", self.single_cond_scale.weight.device)
        return self._packed(_b(x), _b(single_cond)).to(x.dtype)


class DistributeAdaptiveLayerNorm(AdaptiveLayerNorm):
    pass


class DistributeAdaLNZero(nn.Module):
    """transition2(x) [* sigmoid(adaptive_zero_cond(cond))] (reference :80-118).  Conventions for what the
    absent base-class constructor decides: ``transition2`` without bias, ``adaptive_zero_cond`` with bias."""

    def __init__(self, device_mesh, c_in: int, c_out: int, c_single_cond: int, use_single_cond: bool = False,
                 shard_out: bool = False) -> None:
        super().__init__()
        self.c_in, self.c_out, self.c_single_cond, self.use_single_cond = c_in, c_out, c_single_cond, use_single_cond
        self.transition2 = nn.Linear(c_in, c_out, bias=False)
        if use_single_cond:
            self.adaptive_zero_cond = nn.Linear(c_single_cond, c_out, bias=True)
        self.shard_out = shard_out
        self.tpp_transition2 = None
        init_dist_info(self, device_mesh)

    def shard_params(self) -> None:
        if self.tp_size > 1:
            raise NotImplementedError("weight sharding (tp > 1) is outside the sample-parallel diffusion hot path")

    def forward(self, x: torch.Tensor, single_cond: Optional[torch.Tensor] = None) -> torch.Tensor:
        assert (single_cond is None) == (self.use_single_cond is False)
        dev = self.transition2.weight.device
        w = self.transition2.weight
        if self.tpp_transition2 is not None:       # [H, D, c] layout set by DistributeSelfAttention.load_xsmm_params
            w = self.tpp_transition2.reshape(-1, self.c_out).T
        xb = _b(x)
        wb = ops._b16(w, dev)
        if not self.use_single_cond:
            return ops.linear(xb, wb).to(x.dtype)
        gate = ops.linear(_b(single_cond), ops._b16(self.adaptive_zero_cond.weight, dev),
                          ops._f32(self.adaptive_zero_cond.bias, dev))
        n = gate.shape[0]
        return ops.linear_gate_residual(xb, wb, gate, None, row_gate_mod=n).to(x.dtype)


class DistributeDiffusionTransition(nn.Module):
    """AdaLN -> GLU (factor 2) -> AdaLN-Zero; returns the update (reference :120-145)."""

    def __init__(self, device_mesh, c_x: int, c_single_cond: int, num_intermediate_factor: int = 2,
                 use_single_cond: bool = False) -> None:
        super().__init__()
        self.c_x, self.c_single_cond = c_x, c_single_cond
        self.num_intermediate_factor, self.use_single_cond = num_intermediate_factor, use_single_cond
        self.adaptive_layernorm = AdaptiveLayerNorm(c_x, c_single_cond, use_single_cond)
        self.transition1 = nn.Linear(c_x, 2 * num_intermediate_factor * c_x, bias=False)
        self.adaptive_zero_init = DistributeAdaLNZero(device_mesh, num_intermediate_factor * c_x, c_x, c_single_cond,
                                                      use_single_cond, shard_out=False)
        init_dist_info(self, device_mesh)
        self._w1 = None

    def shard_params(self) -> None:
        if self.tp_size > 1:
            raise NotImplementedError("weight sharding (tp > 1) is outside the sample-parallel diffusion hot path")

    def forward(self, x: torch.Tensor, single_cond: Optional[torch.Tensor] = None) -> torch.Tensor:
        xn = self.adaptive_layernorm(x, single_cond)
        if self._w1 is None:
            self._w1 = ops._b16(ops.pack_swiglu_weight(self.transition1.weight), self.transition1.weight.device)
        c = ops.linear_swiglu(_b(xn), self._w1)
        return self.adaptive_zero_init(c, single_cond).to(x.dtype)


class DistributeSelfAttention(nn.Module):
    """AttentionPairBias; returns the update (reference :148-265).  x [N, c] or [S, N, c]; mask [N];
    pair_logits [H, N, N]."""

    def __init__(self, device_mesh, c_x: int = 768, c_single_cond: int = 384, num_head: int = 16,
                 use_single_cond: bool = False, use_batch_infer: bool = False) -> None:
        super().__init__()
        self.c_x, self.c_single_cond, self.num_head = c_x, c_single_cond, num_head
        self.qkv_dim = c_x // num_head
        self.use_single_cond, self.use_batch_infer = use_single_cond, use_batch_infer
        self.adaptive_layernorm = AdaptiveLayerNorm(c_x, c_single_cond, use_single_cond)
        self.q_projection = nn.Linear(c_x, c_x, bias=True)
        self.k_projection = nn.Linear(c_x, c_x, bias=False)
        self.v_projection = nn.Linear(c_x, c_x, bias=False)
        self.gating_query = nn.Linear(c_x, c_x, bias=False)
        self.adaptive_zero_init = DistributeAdaLNZero(device_mesh, c_x, c_x, c_single_cond, use_single_cond,
                                                      shard_out=False)
        init_dist_info(self, device_mesh)
        self._packed = None

    def shard_params(self) -> None:
        if self.tp_size > 1:
            raise NotImplementedError("head sharding (tp > 1) is outside the sample-parallel diffusion hot path")

    def load_xsmm_params(self) -> None:
        self._packed = ops.PackedSelfAttention(self.state_dict(), "", self.q_projection.weight.device, self.num_head)
        self.key_dim = self.value_dim = self.qkv_dim

    def xsmm_forward(self, x: torch.Tensor, mask: torch.Tensor, pair_logits: Optional[torch.Tensor] = None,
                     single_cond: Optional[torch.Tensor] = None) -> torch.Tensor:
        assert (single_cond is None) == (self.use_single_cond is False)
        if self._packed is None:
            self.load_xsmm_params()
        xn = _b(self.adaptive_layernorm(x, single_cond))
        batched = xn.dim() == 3
        xb = xn if batched else xn[None]
        n = xb.shape[1]
        if pair_logits is None:
            pair_logits = torch.zeros(self.num_head, n, n, device=x.device)
        o = ops.attention_pair_bias_core(xb, self._packed, pair_logits.float().contiguous(),
                                         None if mask is None else mask.float())
        dev = self.q_projection.weight.device
        if self.use_single_cond:
            az = self.adaptive_zero_init
            gate = ops.linear(_b(single_cond), ops._b16(az.adaptive_zero_cond.weight, dev),
                              ops._f32(az.adaptive_zero_cond.bias, dev))
            out = ops.linear_gate_residual(o, self._packed.w_out, gate, None, row_gate_mod=n)
        else:
            out = ops.linear(o, self._packed.w_out)
        return (out if batched else out[0]).to(x.dtype)

    forward = xsmm_forward


class DistributeDiffusionTransformer(nn.Module):
    """24 blocks in 6 super-blocks (reference :267-310).  ``forward(act, mask, single_cond, pair_cond)``
    updates ``act`` in place and returns it, as the reference does."""

    def __init__(self, device_mesh, c_act: int = 768, c_single_cond: int = 384, c_pair_cond: int = 128,
                 num_head: int = 16, num_blocks: int = 24, super_block_size: int = 4,
                 use_batch_infer: bool = False) -> None:
        super().__init__()
        self.c_act, self.c_single_cond, self.c_pair_cond = c_act, c_single_cond, c_pair_cond
        self.num_head, self.num_blocks, self.super_block_size = num_head, num_blocks, super_block_size
        self.num_super_blocks = num_blocks // super_block_size
        self.pair_input_layer_norm = LayerNorm(c_pair_cond)
        self.pair_logits_projection = nn.ModuleList(
            [nn.Linear(c_pair_cond, super_block_size * num_head, bias=False) for _ in range(self.num_super_blocks)])
        self.self_attention = nn.ModuleList(
            [DistributeSelfAttention(device_mesh, c_act, c_single_cond, num_head, use_single_cond=True,
                                     use_batch_infer=use_batch_infer) for _ in range(num_blocks)])
        self.transition_block = nn.ModuleList(
            [DistributeDiffusionTransition(device_mesh, c_act, c_single_cond, use_single_cond=True)
             for _ in range(num_blocks)])
        init_dist_info(self, device_mesh)
        self._packed = None
        self._pair_logits = None

    def shard_params(self) -> None:
        if self.tp_size > 1:
            raise NotImplementedError("head sharding (tp > 1) is outside the sample-parallel diffusion hot path")

    def load_xsmm_params(self) -> None:
        self._packed = diffusion.PackedDiffusionTransformer(self.state_dict(), "", self.pair_input_layer_norm.weight.device,
                                                            self.num_head, self.num_blocks, self.super_block_size)

    def precompute_pair_logits(self, pair_cond: torch.Tensor) -> None:
        """Optional: compute the step-invariant pair logits once; later forwards reuse them."""
        if self._packed is None:
            self.load_xsmm_params()
        self._pair_logits = self._packed.pair_logits(_b(pair_cond))

    def xsmm_forward(self, act: torch.Tensor, mask: torch.Tensor, single_cond: torch.Tensor, pair_cond: torch.Tensor):
        if self._packed is None:
            self.load_xsmm_params()
        pl = self._pair_logits if self._pair_logits is not None else self._packed.pair_logits(_b(pair_cond))
        a = _b(act)
        self._packed.forward(a, None if mask is None else mask.float(), _b(single_cond), pl)
        if a.data_ptr() != act.data_ptr():
            act.copy_(a)
        return act

    forward = xsmm_forward
