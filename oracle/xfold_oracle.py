"""CPU oracle for the Pairformer / diffusion-transformer hot path.

THIS FILE IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It restates, in plain fp32
PyTorch on the CPU, the arithmetic of the reference's Python modules so that the
CUDA kernels can be checked against it.  Only the test-suite, the smoke entry
and the CPU-baseline leg of the benchmark may import it; the product package
never does.

Every function cites the reference file (path inside the reference project) it
follows.  Parameters are taken from a flat ``state`` dict whose keys are the
reference's own ``state_dict`` names under a ``prefix`` (for example
``"triangle_multiplication_outgoing.projection.weight"``), so the very same
dict can be loaded into the reference's modules when they are importable.

Pinning status
--------------
* ``triangle_multiplication`` is checked against the reference's own
  ``XSMMTriangleMultiplication.forward`` and (two gloo ranks)
  ``DistributeTriangleMultiplication.forward`` by ``oracle/pin_against_reference.py``;
  the resulting vectors live in ``tests/golden``.
* ``gated_attention`` / ``transition`` / ``self_attention_core`` are checked
  against the plain-torch specification classes that the reference's kernel
  tests carry (``GatingAttention``, ``Transition``, ``SelfAttention1``).
* ``adaptive_layernorm``, ``adaln_zero`` (forward), ``self_attention`` (forward),
  ``diffusion_transformer`` (forward) and ``pairformer_block`` (forward) are
  checked against the reference's own ``forward`` methods executed over stand-in
  base classes (the third-party ``xfold`` package that supplies the base-class
  constructors is not part of the reference tree).  What stays *unpinned* is
  only what those absent constructors decide: the bias flags of
  ``AdaLNZero.transition2`` (taken as no bias) and ``adaptive_zero_cond`` (taken
  as bias) and of ``DiffusionTransformer.pair_input_layer_norm`` (taken as a
  full affine LayerNorm).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F

State = Dict[str, torch.Tensor]
LN_EPS = 1e-5  # xsmm_kernels/csrc/triangle_multiplication.h:51-52, transition.h:26


# ----------------------------------------------------------------------------
# small helpers
# ----------------------------------------------------------------------------
def _get(state: State, prefix: str, name: str) -> Optional[torch.Tensor]:
    return state.get(prefix + name)


def layer_norm(x, weight=None, bias=None, eps: float = LN_EPS):
    """LayerNorm over the last dim (xfold.fastnn.LayerNorm as used at
    nn/d_triangle_multiplication.py:109-112; eps from the C++ LayerNormFwdTPP)."""
    return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)


def linear(x, weight, bias=None):
    return F.linear(x, weight, bias)


class ShardInfo:
    """Row partition rule of distribute_utils.py:101-128: ceil(N/P) rows per
    rank, the last rank takes the remainder (N 764, P 8 -> 7 x 96 + 92)."""

    def __init__(self, tensor_size: int, num_shard: int):
        assert num_shard <= tensor_size
        if tensor_size % num_shard:
            per = math.ceil(tensor_size / num_shard)
            rem = tensor_size % per
            sizes = [per] * (num_shard - 1) + [rem]
        else:
            per = tensor_size // num_shard
            sizes = [per] * num_shard
        self.sizes = sizes
        offs = [0]
        for s in sizes:
            offs.append(offs[-1] + s)
        self.slices = [slice(offs[i], offs[i + 1]) for i in range(num_shard)]


# ----------------------------------------------------------------------------
# TriangleMultiplication
# ----------------------------------------------------------------------------
def triangle_multiplication(state: State, prefix: str, pair, mask, outgoing: bool):
    """nn/d_triangle_multiplication.py:141-178 (XSMMTriangleMultiplication.forward).

    pair [R, N, c] (R == N when unsharded), mask [R, N] or None -> update [R, N, c].
    Even output rows of ``projection``/``gate`` are ``a``, odd rows are ``b``
    (:162-165).  Equation strings :122-124: outgoing 'cik,cjk->cij',
    incoming 'ckj,cki->cij' i.e. out[i,j] = sum_k a[k,j] * b[k,i].
    """
    c = pair.shape[-1]
    x = layer_norm(pair, _get(state, prefix, "left_norm_input.weight"),
                   _get(state, prefix, "left_norm_input.bias"))
    proj = linear(x, state[prefix + "projection.weight"]).permute(2, 0, 1)
    if mask is not None:
        proj = proj * mask[None, ...]
    gate = linear(x, state[prefix + "gate.weight"]).permute(2, 0, 1)
    proj = proj * torch.sigmoid(gate)
    proj = proj.reshape(c, 2, *proj.shape[1:])
    a, b = proj[:, 0], proj[:, 1]
    eq = "cik,cjk->cij" if outgoing else "ckj,cki->cij"
    o = torch.einsum(eq, a, b).permute(1, 2, 0)
    o = layer_norm(o, _get(state, prefix, "center_norm.weight"),
                   _get(state, prefix, "center_norm.bias"))
    o = linear(o, state[prefix + "output_projection.weight"])
    g = linear(x, state[prefix + "gating_linear.weight"])
    return o * torch.sigmoid(g)


def triangle_multiplication_sharded(state: State, prefix: str, shard, mask_shard, full_b_gather, outgoing: bool):
    """nn/d_triangle_multiplication.py:48-99 with the all-gather of ``b``
    replaced by ``full_b_gather(b_local) -> b_full`` so that one process can
    emulate P ranks.  Outgoing takes the row shard [N/P, N, c]; incoming takes
    the column shard [N, N/P, c] (comment at :81; rule of test_utils/test_einsum.py)."""
    c = shard.shape[-1]
    x = layer_norm(shard, _get(state, prefix, "left_norm_input.weight"),
                   _get(state, prefix, "left_norm_input.bias"))
    proj = linear(x, state[prefix + "projection.weight"]).permute(2, 0, 1)
    if mask_shard is not None:
        proj = proj * mask_shard[None, ...]
    gate = linear(x, state[prefix + "gate.weight"]).permute(2, 0, 1)
    proj = proj * torch.sigmoid(gate)
    proj = proj.reshape(c, 2, *proj.shape[1:])
    a, b = proj[:, 0], proj[:, 1]
    b = full_b_gather(b)
    eq = "cik,cjk->cij" if outgoing else "ckj,cki->cij"
    o = torch.einsum(eq, a, b).permute(1, 2, 0)
    o = layer_norm(o, _get(state, prefix, "center_norm.weight"),
                   _get(state, prefix, "center_norm.bias"))
    o = linear(o, state[prefix + "output_projection.weight"])
    g = linear(x, state[prefix + "gating_linear.weight"])
    return o * torch.sigmoid(g)


# ----------------------------------------------------------------------------
# gated multi-head attention cores
# ----------------------------------------------------------------------------
def gated_attention(q_data, bias, nonbatched_bias, query_w, key_w, value_w, gating_w, output_w,
                    query_b=None, row_chunk: int = 0):
    """Spec classes of the kernel tests: xsmm_kernels/kernel_test/grid_self_attenion_bf16.py:61-95
    (GatingAttention) and batch_diffusion_self_attention.py:62-87 (SelfAttention1,
    which adds ``query_b`` and drops the output projection -> pass ``output_w=None``).

    q_data [B, S, c]; bias broadcastable to [B, 1, 1, S]; nonbatched_bias [H, S, S];
    weights [c, H, D]; output_w [H, D, c_out] or None.
    ``row_chunk`` > 0 evaluates the batch in slices to bound host memory.
    """
    D = query_w.shape[-1]

    def one(qd, bs):
        q = torch.einsum("bqa,ahc->bqhc", qd, query_w)
        if query_b is not None:
            q = q + query_b
        q = q * D ** (-0.5)
        k = torch.einsum("bka,ahc->bkhc", qd, key_w)
        v = torch.einsum("bka,ahc->bkhc", qd, value_w)
        logits = torch.einsum("bqhc,bkhc->bhqk", q, k) + bs
        if nonbatched_bias is not None:
            logits = logits + nonbatched_bias[None]
        w = torch.softmax(logits, dim=-1)
        o = torch.einsum("bhqk,bkhc->bqhc", w, v)
        o = o * torch.sigmoid(torch.einsum("bqc,chv->bqhv", qd, gating_w))
        if output_w is not None:
            o = torch.einsum("bqhc,hco->bqo", o, output_w)
        return o

    B = q_data.shape[0]
    if row_chunk <= 0 or row_chunk >= B:
        return one(q_data, bias)
    outs = []
    for s in range(0, B, row_chunk):
        bs = bias[s:s + row_chunk] if bias.shape[0] == B else bias
        outs.append(one(q_data[s:s + row_chunk], bs))
    return torch.cat(outs, 0)


def cross_attention(q_data, m_data, batched_bias, query_w, query_b, key_w, value_w, gating_w):
    """Spec class of the reference's kernel test for `batch_diffusion_cross_attention_forward`
    (xsmm_kernels/kernel_test/batch_diffusion_cross_attention.py:23-87, CrossAttention.forward): the gated attention of
    the atom cross-attention encoder / decoder (nn/d_diffusion_transformer.py:313-543), queries and keys from different
    token sets, one bias per batch entry, no output projection.

    q_data [B, S, a]; m_data [B, K, m]; batched_bias [B, H, S, K]; query_w / gating_w [a, H, D]; query_b [1, H, D];
    key_w / value_w [m, H, D] -> [B, S, H, D]."""
    D = query_w.shape[-1]
    q = (torch.einsum("bqa,ahc->bqhc", q_data, query_w) + query_b) * D ** (-0.5)
    k = torch.einsum("bka,ahc->bkhc", m_data, key_w)
    v = torch.einsum("bka,ahc->bkhc", m_data, value_w)
    logits = torch.einsum("bqhc,bkhc->bhqk", q, k) + batched_bias
    w = torch.softmax(logits, dim=-1)
    o = torch.einsum("bhqk,bkhc->bqhc", w, v)
    return o * torch.sigmoid(torch.einsum("bqc,chv->bqhv", q_data, gating_w))


def grid_self_attention(state: State, prefix: str, pair, mask, full_pair=None, transpose: bool = False,
                        num_head: int = 4, row_chunk: int = 0):
    """nn/d_attention.py:58-111 (DistributeGridSelfAttention.xsmm_forward / forward).

    pair [R, N, c] (row shard; for ``transpose`` the caller passes the column
    shard [N, R, c]); mask has the row shard's shape [R, N]; the pair bias is
    projected from ``full_pair`` and is NOT transposed for the ending node (:62, :99).
    """
    if full_pair is None:
        full_pair = pair
    c = pair.shape[-1]
    D = c // num_head
    lnw, lnb = _get(state, prefix, "act_norm.weight"), _get(state, prefix, "act_norm.bias")
    x = layer_norm(pair, lnw, lnb)
    nb = linear(layer_norm(full_pair, lnw, lnb), state[prefix + "pair_bias_projection.weight"]).permute(2, 0, 1)
    bias = 1e9 * (mask[:, None, None, :] - 1)
    if transpose:
        x = x.permute(1, 0, 2)
    shp = (c, num_head, D)
    qw = state[prefix + "q_projection.weight"].T.reshape(shp)
    kw = state[prefix + "k_projection.weight"].T.reshape(shp)
    vw = state[prefix + "v_projection.weight"].T.reshape(shp)
    gw = state[prefix + "gating_query.weight"].T.reshape(shp)
    ow = state[prefix + "output_projection.weight"].T.reshape(num_head, D, c)
    out = gated_attention(x, bias, nb, qw, kw, vw, gw, ow, row_chunk=row_chunk)
    if transpose:
        out = out.permute(1, 0, 2)
    return out


# ----------------------------------------------------------------------------
# Transition (SwiGLU MLP)
# ----------------------------------------------------------------------------
def gated_linear_unit(x, weight_t):
    """xfold.fastnn.gated_linear_unit as pinned by kernel_test/transition.py:37-43 and
    csrc/transition.h:65-88: y = x @ W; first half goes through SiLU, times second half."""
    y = x @ weight_t
    a, b = torch.chunk(y, 2, dim=-1)
    return F.silu(a) * b


def transition(state: State, prefix: str, x):
    """nn/d_primitives.py:31-38 (DistributeTransition.forward), world size 1."""
    x = layer_norm(x, _get(state, prefix, "input_layer_norm.weight"), _get(state, prefix, "input_layer_norm.bias"))
    c = gated_linear_unit(x, state[prefix + "transition1.weight"].T)
    return linear(c, state[prefix + "transition2.weight"])


# ----------------------------------------------------------------------------
# Diffusion transformer pieces
# ----------------------------------------------------------------------------
def adaptive_layernorm(state: State, prefix: str, x, single_cond=None):
    """nn/d_diffusion_transformer.py:37-74 (AdaptiveLayerNorm)."""
    if single_cond is None:
        return layer_norm(x, _get(state, prefix, "layer_norm.weight"), _get(state, prefix, "layer_norm.bias"))
    x = layer_norm(x)
    sc = layer_norm(single_cond, state[prefix + "single_cond_layer_norm.weight"], None)
    scale = linear(sc, state[prefix + "single_cond_scale.weight"], state[prefix + "single_cond_scale.bias"])
    bias = linear(sc, state[prefix + "single_cond_bias.weight"])
    return torch.sigmoid(scale) * x + bias


def adaln_zero(state: State, prefix: str, x, single_cond=None):
    """nn/d_diffusion_transformer.py:96-118 (DistributeAdaLNZero.forward), tp 1.
    Convention fixed here (constructor is in the absent xfold package):
    ``transition2`` has no bias; ``adaptive_zero_cond`` has a bias."""
    out = linear(x, state[prefix + "transition2.weight"], _get(state, prefix, "transition2.bias"))
    if single_cond is not None:
        cond = linear(single_cond, state[prefix + "adaptive_zero_cond.weight"],
                      _get(state, prefix, "adaptive_zero_cond.bias"))
        out = torch.sigmoid(cond) * out
    return out


def diffusion_transition(state: State, prefix: str, x, single_cond=None):
    """nn/d_diffusion_transformer.py:142-145 (DistributeDiffusionTransition.forward)."""
    x = adaptive_layernorm(state, prefix + "adaptive_layernorm.", x, single_cond)
    c = gated_linear_unit(x, state[prefix + "transition1.weight"].T)
    return adaln_zero(state, prefix + "adaptive_zero_init.", c, single_cond)


def dot_product_attention(q, k, v, mask=None, bias=None):
    """test_utils/test_grid_attn.py:262-279 (dot_product_attention_torch): scale by
    D^-0.5, add bias, masked_fill(~mask, -1e9), softmax, times v."""
    q = q * q.shape[-1] ** -0.5
    logits = q @ k.transpose(-1, -2)
    if bias is not None:
        logits = logits + bias
    if mask is not None:
        logits = logits.masked_fill(~mask.bool(), -1e9)
    return torch.softmax(logits, dim=-1) @ v


def self_attention(state: State, prefix: str, x, mask, pair_logits=None, single_cond=None, num_head: int = 16):
    """nn/d_diffusion_transformer.py:221-265 (DistributeSelfAttention.forward).
    x [N, c] or [S, N, c]; mask [N]; pair_logits [H, N, N]."""
    xn = adaptive_layernorm(state, prefix + "adaptive_layernorm.", x, single_cond)
    q = linear(xn, state[prefix + "q_projection.weight"], state[prefix + "q_projection.bias"])
    k = linear(xn, state[prefix + "k_projection.weight"])
    v = linear(xn, state[prefix + "v_projection.weight"])
    batched = xn.dim() == 3
    if not batched:
        q, k, v = q[None], k[None], v[None]
    B, N, C = q.shape
    D = C // num_head
    q, k, v = (t.reshape(B, N, num_head, D).permute(0, 2, 1, 3) for t in (q, k, v))
    m = mask[None, None, None, :].bool() if mask is not None else None
    o = dot_product_attention(q, k, v, mask=m, bias=pair_logits)
    o = o.permute(0, 2, 1, 3).reshape(B, N, C)
    if not batched:
        o = o[0]
    o = o * torch.sigmoid(linear(xn, state[prefix + "gating_query.weight"]))
    return adaln_zero(state, prefix + "adaptive_zero_init.", o, single_cond)


def diffusion_transformer(state: State, prefix: str, act, mask, single_cond, pair_cond,
                          num_head: int = 16, num_blocks: int = 24, super_block_size: int = 4):
    """nn/d_diffusion_transformer.py:289-310 (DistributeDiffusionTransformer.forward)."""
    pair_act = layer_norm(pair_cond, _get(state, prefix, "pair_input_layer_norm.weight"),
                          _get(state, prefix, "pair_input_layer_norm.bias"))
    act = act.clone()
    for sb in range(num_blocks // super_block_size):
        pl = linear(pair_act, state[prefix + f"pair_logits_projection.{sb}.weight"])
        n = pl.shape[0]
        pl = pl.reshape(n, n, super_block_size, num_head).permute(2, 3, 0, 1)  # 'n s (b h) -> b h n s'
        for j in range(super_block_size):
            i = sb * super_block_size + j
            act = act + self_attention(state, prefix + f"self_attention.{i}.", act, mask, pl[j], single_cond, num_head)
            act = act + diffusion_transition(state, prefix + f"transition_block.{i}.", act, single_cond)
    return act


# ----------------------------------------------------------------------------
# Pairformer block / stack
# ----------------------------------------------------------------------------
def pairformer_block(state: State, prefix: str, pair, pair_mask, single=None, seq_mask=None,
                     n_heads: int = 16, n_heads_pair: int = 4, row_chunk: int = 0):
    """nn/d_pairformer.py:99-171 (DistributePairformerBlock.forward), world size 1.
    Returns (pair, single) as new tensors."""
    pair = pair + triangle_multiplication(state, prefix + "triangle_multiplication_outgoing.", pair, pair_mask, True)
    pair = pair + triangle_multiplication(state, prefix + "triangle_multiplication_incoming.", pair, pair_mask, False)
    pair = pair + grid_self_attention(state, prefix + "pair_attention1.", pair, pair_mask, pair, False,
                                      n_heads_pair, row_chunk)
    pair = pair + grid_self_attention(state, prefix + "pair_attention2.", pair, pair_mask, pair, True,
                                      n_heads_pair, row_chunk)
    pair = pair + transition(state, prefix + "pair_transition.", pair)
    if single is None:
        return pair, None
    pl = linear(layer_norm(pair, _get(state, prefix, "single_pair_logits_norm.weight"),
                           _get(state, prefix, "single_pair_logits_norm.bias")),
                state[prefix + "single_pair_logits_projection.weight"]).permute(2, 0, 1)
    single = single + self_attention(state, prefix + "single_attention_.", single, seq_mask, pl, None, n_heads)
    single = single + transition(state, prefix + "single_transition.", single)
    return pair, single


def pairformer_block_sharded(state: State, prefix: str, pair, pair_mask, single, seq_mask, world: int,
                             n_heads: int = 16, n_heads_pair: int = 4):
    """Single-process emulation of nn/d_pairformer.py:119-156 for ``world`` row-shard
    ranks: TriMul on the full pair, TriAttn-start on each row shard, gather,
    TriAttn-end + Transition on each column shard, gather, then the single path."""
    n = pair.shape[0]
    sl = ShardInfo(n, world).slices
    pair = pair + triangle_multiplication(state, prefix + "triangle_multiplication_outgoing.", pair, pair_mask, True)
    pair = pair + triangle_multiplication(state, prefix + "triangle_multiplication_incoming.", pair, pair_mask, False)
    rows = [pair[s] + grid_self_attention(state, prefix + "pair_attention1.", pair[s], pair_mask[s], pair, False,
                                          n_heads_pair) for s in sl]
    pair = torch.cat(rows, 0)
    cols = []
    for s in sl:
        sh = pair[:, s]
        sh = sh + grid_self_attention(state, prefix + "pair_attention2.", sh, pair_mask[s], pair, True, n_heads_pair)
        sh = sh + transition(state, prefix + "pair_transition.", sh)
        cols.append(sh)
    pair = torch.cat(cols, 1)
    pl = linear(layer_norm(pair, _get(state, prefix, "single_pair_logits_norm.weight"),
                           _get(state, prefix, "single_pair_logits_norm.bias")),
                state[prefix + "single_pair_logits_projection.weight"]).permute(2, 0, 1)
    single = single + self_attention(state, prefix + "single_attention_.", single, seq_mask, pl, None, n_heads)
    single = single + transition(state, prefix + "single_transition.", single)
    return pair, single


def pairformer_block_rounded(state: State, prefix: str, pair, pair_mask, single, seq_mask, dtype=torch.bfloat16,
                             n_heads: int = 16, n_heads_pair: int = 4):
    """``pairformer_block`` with the representations STORED in ``dtype`` between sub-layers and fp32 arithmetic
    inside them: every sub-layer reads the rounded representation, its update is rounded, and the sum is rounded
    again.  These are the roundings any implementation has that keeps z and s in ``dtype`` (the reference's bf16
    wrappers cast on entry and exit of every fused op, nn/d_triangle_multiplication.py:187-190,
    nn/d_attention.py:75-78), so the distance of this function from ``pairformer_block`` is the error floor of
    ``dtype`` storage for a given depth and set of weights, whatever the kernels inside do."""
    def r(t):
        return t.to(dtype).float()
    pair, single = r(pair), r(single)
    pair = r(pair + r(triangle_multiplication(state, prefix + "triangle_multiplication_outgoing.", pair, pair_mask, True)))
    pair = r(pair + r(triangle_multiplication(state, prefix + "triangle_multiplication_incoming.", pair, pair_mask, False)))
    pair = r(pair + r(grid_self_attention(state, prefix + "pair_attention1.", pair, pair_mask, pair, False, n_heads_pair)))
    pair = r(pair + r(grid_self_attention(state, prefix + "pair_attention2.", pair, pair_mask, pair, True, n_heads_pair)))
    pair = r(pair + r(transition(state, prefix + "pair_transition.", pair)))
    pl = linear(layer_norm(pair, _get(state, prefix, "single_pair_logits_norm.weight"),
                           _get(state, prefix, "single_pair_logits_norm.bias")),
                state[prefix + "single_pair_logits_projection.weight"]).permute(2, 0, 1)
    single = r(single + r(self_attention(state, prefix + "single_attention_.", single, seq_mask, pl, None, n_heads)))
    single = r(single + r(transition(state, prefix + "single_transition.", single)))
    return pair, single


def pairformer_stack(state: State, pair, pair_mask, single, seq_mask, num_blocks: int, row_chunk: int = 0):
    """d_alphafold3.py:242-244: the 48-block loop of DistributeEvoformer.forward."""
    for i in range(num_blocks):
        pair, single = pairformer_block(state, f"trunk_pairformer.{i}.", pair, pair_mask, single, seq_mask,
                                        row_chunk=row_chunk)
    return pair, single


# ----------------------------------------------------------------------------
# seeded weight factory (Linear ~ N(0, 1/fan_in), LayerNorm gamma = 1, beta = 0)
# ----------------------------------------------------------------------------
# ---------------------------------------------------------------------------------------------
# Diffusion head arithmetic around the transformer (nn/d_diffusion_head.py:172-227) and the sampler loop
# (d_alphafold3.py:316-404), restated line by line in float64 loops over steps.  Parity unpinned: the reference's
# loop is a method of the whole model (atom encoder / decoder and the noise schedule come from the absent xfold
# package), so these functions are checked against the product's host code, not against a run of the reference.
# ---------------------------------------------------------------------------------------------
SIGMA_DATA = 16.0


def diffusion_head_mix(positions_noisy, position_update, noise_level, atom_mask):
    skip_scaling = SIGMA_DATA ** 2 / (noise_level ** 2 + SIGMA_DATA ** 2)
    out_scaling = noise_level * SIGMA_DATA / torch.sqrt(noise_level ** 2 + SIGMA_DATA ** 2)
    return (skip_scaling * positions_noisy + out_scaling * position_update) * atom_mask[..., None]


def sampler_constants(noise_levels, gamma_0=0.8, gamma_min=1.0, noise_scale=1.003):
    noise_level_prev = noise_levels[:-1]
    noise_level = noise_levels[1:]
    gamma = gamma_0 * (noise_level > gamma_min)
    t_hat = noise_level_prev * (1 + gamma)
    return noise_level, t_hat, noise_scale * torch.sqrt(t_hat ** 2 - noise_level_prev ** 2)


def sample_diffusion(denoiser, noise_levels, positions0, step_scale=1.5):
    """positions0: the initial draw, already multiplied by noise_levels[0]."""
    noise_level, t_hat, noise_scale = sampler_constants(noise_levels)
    positions = positions0
    for step_idx in range(noise_level.shape[0]):
        positions_noisy = positions + noise_scale[step_idx]
        positions_denoised = denoiser(positions_noisy, t_hat[step_idx], step_idx)
        grad = (positions_noisy - positions_denoised) / t_hat[step_idx]
        d_t = noise_level[step_idx] - t_hat[step_idx]
        positions = positions_noisy + step_scale * d_t * grad
    return positions


def _lin(g, out_f, in_f, bias=False):
    w = torch.randn(out_f, in_f, generator=g) / math.sqrt(in_f)
    b = torch.randn(out_f, generator=g) / math.sqrt(in_f) if bias else None
    return w, b


def _put_linear(state, name, g, out_f, in_f, bias=False):
    w, b = _lin(g, out_f, in_f, bias)
    state[name + ".weight"] = w
    if b is not None:
        state[name + ".bias"] = b


def _put_ln(state, name, c, affine=True, bias=True):
    if affine:
        state[name + ".weight"] = torch.ones(c)
        if bias:
            state[name + ".bias"] = torch.zeros(c)


def make_trimul_state(g, prefix: str, c: int = 128) -> State:
    s: State = {}
    _put_ln(s, prefix + "left_norm_input", c)
    _put_linear(s, prefix + "projection", g, 2 * c, c)
    _put_linear(s, prefix + "gate", g, 2 * c, c)
    _put_ln(s, prefix + "center_norm", c)
    _put_linear(s, prefix + "output_projection", g, c, c)
    _put_linear(s, prefix + "gating_linear", g, c, c)
    return s


def make_grid_attention_state(g, prefix: str, c: int = 128, num_head: int = 4) -> State:
    s: State = {}
    _put_ln(s, prefix + "act_norm", c)
    _put_linear(s, prefix + "pair_bias_projection", g, num_head, c)
    for n in ("q_projection", "k_projection", "v_projection", "gating_query", "output_projection"):
        _put_linear(s, prefix + n, g, c, c)
    return s


def make_transition_state(g, prefix: str, c: int, factor: int = 4) -> State:
    s: State = {}
    _put_ln(s, prefix + "input_layer_norm", c)
    _put_linear(s, prefix + "transition1", g, 2 * factor * c, c)
    _put_linear(s, prefix + "transition2", g, c, factor * c)
    return s


def make_adaptive_layernorm_state(g, prefix: str, c: int, c_cond: int, use_cond: bool) -> State:
    s: State = {}
    if use_cond:
        s[prefix + "single_cond_layer_norm.weight"] = torch.ones(c_cond)
        _put_linear(s, prefix + "single_cond_scale", g, c, c_cond, bias=True)
        _put_linear(s, prefix + "single_cond_bias", g, c, c_cond)
    else:
        _put_ln(s, prefix + "layer_norm", c)
    return s


def make_adaln_zero_state(g, prefix: str, c_in: int, c_out: int, c_cond: int, use_cond: bool) -> State:
    s: State = {}
    _put_linear(s, prefix + "transition2", g, c_out, c_in)
    if use_cond:
        _put_linear(s, prefix + "adaptive_zero_cond", g, c_out, c_cond, bias=True)
    return s


def make_self_attention_state(g, prefix: str, c: int, c_cond: int, use_cond: bool) -> State:
    s: State = {}
    s.update(make_adaptive_layernorm_state(g, prefix + "adaptive_layernorm.", c, c_cond, use_cond))
    _put_linear(s, prefix + "q_projection", g, c, c, bias=True)
    _put_linear(s, prefix + "k_projection", g, c, c)
    _put_linear(s, prefix + "v_projection", g, c, c)
    _put_linear(s, prefix + "gating_query", g, c, c)
    s.update(make_adaln_zero_state(g, prefix + "adaptive_zero_init.", c, c, c_cond, use_cond))
    return s


def make_diffusion_transition_state(g, prefix: str, c: int, c_cond: int, factor: int = 2, use_cond: bool = True) -> State:
    s: State = {}
    s.update(make_adaptive_layernorm_state(g, prefix + "adaptive_layernorm.", c, c_cond, use_cond))
    _put_linear(s, prefix + "transition1", g, 2 * factor * c, c)
    s.update(make_adaln_zero_state(g, prefix + "adaptive_zero_init.", factor * c, c, c_cond, use_cond))
    return s


def make_diffusion_transformer_state(g, prefix: str, c_act=768, c_cond=384, c_pair=128, num_head=16,
                                     num_blocks=24, super_block_size=4) -> State:
    s: State = {}
    _put_ln(s, prefix + "pair_input_layer_norm", c_pair)
    for sb in range(num_blocks // super_block_size):
        _put_linear(s, prefix + f"pair_logits_projection.{sb}", g, super_block_size * num_head, c_pair)
    for i in range(num_blocks):
        s.update(make_self_attention_state(g, prefix + f"self_attention.{i}.", c_act, c_cond, True))
        s.update(make_diffusion_transition_state(g, prefix + f"transition_block.{i}.", c_act, c_cond, 2, True))
    return s


def make_pairformer_block_state(g, prefix: str, c_pair=128, c_single=384, n_heads=16, n_heads_pair=4,
                                with_single=True) -> State:
    s: State = {}
    s.update(make_trimul_state(g, prefix + "triangle_multiplication_outgoing.", c_pair))
    s.update(make_trimul_state(g, prefix + "triangle_multiplication_incoming.", c_pair))
    s.update(make_grid_attention_state(g, prefix + "pair_attention1.", c_pair, n_heads_pair))
    s.update(make_grid_attention_state(g, prefix + "pair_attention2.", c_pair, n_heads_pair))
    s.update(make_transition_state(g, prefix + "pair_transition.", c_pair))
    if with_single:
        _put_ln(s, prefix + "single_pair_logits_norm", c_pair)
        _put_linear(s, prefix + "single_pair_logits_projection", g, n_heads, c_pair)
        s.update(make_self_attention_state(g, prefix + "single_attention_.", c_single, 0, False))
        s.update(make_transition_state(g, prefix + "single_transition.", c_single))
    return s


def make_pairformer_stack_state(seed: int, num_blocks: int) -> State:
    g = torch.Generator().manual_seed(seed)
    s: State = {}
    for i in range(num_blocks):
        s.update(make_pairformer_block_state(g, f"trunk_pairformer.{i}."))
    return s


def make_inputs(seed: int, n: int, c_pair=128, c_single=384, pad_frac: float = 0.0):
    """z, s ~ N(0,1); ``pad_frac`` of the tokens padded (seq_mask Bernoulli(1 - pad_frac),
    pair_mask = outer(seq_mask)); generated on the CPU so both sides see identical values."""
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(n, n, c_pair, generator=g)
    s = torch.randn(n, c_single, generator=g)
    if pad_frac > 0:
        seq_mask = (torch.rand(n, generator=g) >= pad_frac).float()
    else:
        seq_mask = torch.ones(n)
    pair_mask = seq_mask[:, None] * seq_mask[None, :]
    return z, s, pair_mask, seq_mask


def rel_frobenius(a, b) -> float:
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))
