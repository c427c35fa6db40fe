"""DiffusionTransformer on the sm_100a kernels (reference: nn/d_diffusion_transformer.py:37-310).

24 blocks in 6 super-blocks; per block  act += AttentionPairBias(act, mask, pair_logits, single_cond)
and  act += DiffusionTransition(act, single_cond).  Everything below is a composition of C-ABI calls:

    AdaptiveLayerNorm        -> conditioning GEMM on LN(single_cond), then LayerNorm with fused modulation
    q/k/v/gate projections   -> one GEMM with query bias and D^-0.5 folded into the epilogue
    attention (16 x 48 -> 64)-> flash kernel with the fp32 pair bias
    AdaLNZero                -> output GEMM whose epilogue multiplies by sigmoid(cond) per token row and adds the residual
    DiffusionTransition      -> GEMM with SwiGLU epilogue, then the AdaLNZero GEMM

The pair logits depend only on the step-invariant ``pair_cond``; ``pair_logits()`` computes them once
per inference (the reference recomputes them every denoising step, nn/d_diffusion_transformer.py:299-305;
results are identical).  Samples are independent: ``shard_samples`` gives each rank its share by the
reference's ShardInfo rule (d_alphafold3.py:381-385); no collective is needed inside the transformer.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from . import ops
from .distribute_utils import ShardInfo

State = Dict[str, torch.Tensor]
BF16 = torch.bfloat16


class _PackedAdaLN:
    """AdaptiveLayerNorm with conditioning: scale and shift projections stacked into one [2c, c_cond] GEMM."""

    def __init__(self, state: State, prefix: str, device):
        self.cond_ln_g = ops._f32(state[prefix + "single_cond_layer_norm.weight"], device)
        w = torch.cat([state[prefix + "single_cond_scale.weight"], state[prefix + "single_cond_bias.weight"]], 0)
        self.w = ops._b16(w, device)
        c = state[prefix + "single_cond_scale.weight"].shape[0]
        b = torch.zeros(2 * c)
        b[:c] = state[prefix + "single_cond_scale.bias"].detach().float().cpu()
        self.b = ops._f32(b, device)
        self.c = c

    def __call__(self, x: torch.Tensor, cond: torch.Tensor) -> torch.Tensor:
        cn = ops.layernorm(cond, self.cond_ln_g, None)
        mod = ops.linear(cn, self.w, self.b)                      # [N, 2c]: scale | shift
        sc, sh = mod[:, : self.c].contiguous(), mod[:, self.c:].contiguous()
        return ops.layernorm(x, mod_scale=sc, mod_shift=sh)       # sigmoid(scale) * LN(x) + shift


class _PackedAdaLNZero:
    def __init__(self, state: State, prefix: str, device, w_out: torch.Tensor):
        self.w_out = w_out
        self.wc = ops._b16(state[prefix + "adaptive_zero_cond.weight"], device)
        bc = state.get(prefix + "adaptive_zero_cond.bias")
        self.bc = None if bc is None else ops._f32(bc, device)

    def __call__(self, x: torch.Tensor, cond: torch.Tensor, resid: torch.Tensor, n_tokens: int) -> torch.Tensor:
        gate = ops.linear(cond, self.wc, self.bc)                 # [N, c]; the kernel applies the sigmoid
        return ops.linear_gate_residual(x, self.w_out, gate, resid, row_gate_mod=n_tokens, out=resid)


class PackedDiffusionBlock:
    def __init__(self, state: State, p_att: str, p_tr: str, device, num_head: int = 16):
        self.att = ops.PackedSelfAttention(state, p_att, device, num_head)
        self.att_ln = _PackedAdaLN(state, p_att + "adaptive_layernorm.", device)
        self.att_zero = _PackedAdaLNZero(state, p_att + "adaptive_zero_init.", device, self.att.w_out)
        self.tr_ln = _PackedAdaLN(state, p_tr + "adaptive_layernorm.", device)
        self.tr_w1 = ops._b16(ops.pack_swiglu_weight(state[p_tr + "transition1.weight"]), device)
        self.tr_zero = _PackedAdaLNZero(state, p_tr + "adaptive_zero_init.", device,
                                        ops._b16(state[p_tr + "adaptive_zero_init.transition2.weight"], device))


class PackedDiffusionTransformer:
    def __init__(self, state: State, prefix: str, device, num_head: int = 16, num_blocks: int = 24,
                 super_block_size: int = 4):
        self.num_head, self.num_blocks, self.sb = num_head, num_blocks, super_block_size
        self.pair_ln_g = ops._f32(state.get(prefix + "pair_input_layer_norm.weight"), device)
        self.pair_ln_b = ops._f32(state.get(prefix + "pair_input_layer_norm.bias"), device)
        self.pl_w = [ops._f32(state[prefix + f"pair_logits_projection.{i}.weight"], device)
                     for i in range(num_blocks // super_block_size)]
        self.blocks = [PackedDiffusionBlock(state, prefix + f"self_attention.{i}.", prefix + f"transition_block.{i}.",
                                            device, num_head) for i in range(num_blocks)]

    def pair_logits(self, pair_cond: torch.Tensor) -> List[torch.Tensor]:
        """[N, N, 128] bf16 -> per super-block float16 [super_block_size, heads, N, pad8(N)], the prepared operand of the
        attention kernel (values times log2(e)): half the resident bytes of the float32 logits, and no conversion inside
        the 200 denoising steps.  ('n s (b h) -> b h n s', nn/d_diffusion_transformer.py:301-305.)"""
        n = pair_cond.shape[0]
        out = []
        for w in self.pl_w:
            _, proj = ops.layernorm(pair_cond, self.pair_ln_g, self.pair_ln_b, proj_w=w, want_y=False)
            prepared = ops.prepare_pair_bias(proj.reshape(self.sb * self.num_head, n, n))
            del proj
            out.append(prepared.reshape(self.sb, self.num_head, n, prepared.shape[-1]))
        return out

    def forward(self, act: torch.Tensor, mask: Optional[torch.Tensor], single_cond: torch.Tensor,
                pair_logits: List[torch.Tensor]) -> torch.Tensor:
        """act bf16 [S, N, 768] or [N, 768] (updated in place and returned); single_cond bf16 [N, 384]."""
        squeeze = act.dim() == 2
        a = act[None] if squeeze else act
        n = a.shape[1]
        for i, blk in enumerate(self.blocks):
            pl = pair_logits[i // self.sb][i % self.sb]
            xn = blk.att_ln(a, single_cond)
            o = ops.attention_pair_bias_core(xn, blk.att, pl, mask)
            blk.att_zero(o, single_cond, a, n)
            xn = blk.tr_ln(a, single_cond)
            h = ops.linear_swiglu(xn, blk.tr_w1)
            blk.tr_zero(h, single_cond, a, n)
        return act


def shard_samples(num_samples: int, world: int, rank: int) -> slice:
    """Samples owned by ``rank`` (ShardInfo rule, d_alphafold3.py:381-385)."""
    return ShardInfo(num_samples, world).get_shard_slice_list()[rank]
