"""Torch-facing wrappers of the C ABI: weight packing (the counterpart of the reference's
``load_xsmm_params`` methods) and one Python function per fused operator (the counterpart of
``xsmm_kernels/prototypes/*.py``).  Tensors must live on an sm_100 GPU; nothing here computes on
the CPU and nothing falls back to eager PyTorch.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional

import torch

from . import _cabi
from ._cabi import (PairformerWeights, TransitionWeights, TriAttnWeights, TriMulWeights, check, ctx, load)

State = Dict[str, torch.Tensor]
BF16 = torch.bfloat16


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise _cabi.XfoldError("xfold_b200 operators run on a B200 GPU only: got a CPU tensor (no CPU fallback)")


def _dev(t: torch.Tensor) -> int:
    return t.device.index if t.device.index is not None else torch.cuda.current_device()


class _Workspace:
    """Grow-only scratch buffer per device, reused by every operator call on that device."""
    _bufs: Dict[int, torch.Tensor] = {}

    @classmethod
    def get(cls, device: int, nbytes: int) -> torch.Tensor:
        b = cls._bufs.get(device)
        if b is None or b.numel() < nbytes:
            cls._bufs[device] = None
            b = torch.empty(int(nbytes), dtype=torch.uint8, device=f"cuda:{device}")
            cls._bufs[device] = b
        return b


def synchronize_and_check(device: Optional[int] = None) -> None:
    """Synchronises the current stream and raises if a kernel reported a bounded-wait time-out."""
    device = torch.cuda.current_device() if device is None else device
    rc = load().xfold_check_status(ctx(device), _stream(device))
    check(rc, device, "xfold_check_status")


# ---------------------------------------------------------------------------------------------
# weight packing
# ---------------------------------------------------------------------------------------------
def _f32(t, device):
    return None if t is None else t.detach().to(device=device, dtype=torch.float32).contiguous()


def _b16(t, device):
    return t.detach().to(device=device, dtype=BF16).contiguous()


class PackedTriMul:
    """De-interleaves a/b (even/odd rows, nn/d_triangle_multiplication.py:128-129) and stacks
    projection, gate and gating_linear into one [640, 128] matrix."""

    def __init__(self, state: State, prefix: str, device):
        p, g = state[prefix + "projection.weight"], state[prefix + "gate.weight"]
        w_in = torch.cat([p[0::2], g[0::2], p[1::2], g[1::2], state[prefix + "gating_linear.weight"]], 0)
        self.w_in = _b16(w_in, device)
        self.w_out = _b16(state[prefix + "output_projection.weight"], device)
        self.ln_in_g = _f32(state.get(prefix + "left_norm_input.weight"), device)
        self.ln_in_b = _f32(state.get(prefix + "left_norm_input.bias"), device)
        self.ln_c_g = _f32(state.get(prefix + "center_norm.weight"), device)
        self.ln_c_b = _f32(state.get(prefix + "center_norm.bias"), device)
        self.c = TriMulWeights(_ptr(self.ln_in_g), _ptr(self.ln_in_b), _ptr(self.w_in), _ptr(self.ln_c_g),
                               _ptr(self.ln_c_b), _ptr(self.w_out))


class PackedTriAttn:
    def __init__(self, state: State, prefix: str, device, num_head: int = 4):
        c = state[prefix + "q_projection.weight"].shape[0]
        d = c // num_head
        w = torch.cat([state[prefix + n + ".weight"] for n in ("q_projection", "k_projection", "v_projection",
                                                               "gating_query")], 0)
        self.w_qkvg = _b16(w, device)
        scale = torch.ones(4 * c)
        scale[:c] = d ** -0.5
        self.scale = _f32(scale, device)
        self.w_bias = _f32(state[prefix + "pair_bias_projection.weight"], device)
        self.w_out = _b16(state[prefix + "output_projection.weight"], device)
        self.ln_g = _f32(state.get(prefix + "act_norm.weight"), device)
        self.ln_b = _f32(state.get(prefix + "act_norm.bias"), device)
        self.c = TriAttnWeights(_ptr(self.ln_g), _ptr(self.ln_b), _ptr(self.w_bias), _ptr(self.w_qkvg),
                                _ptr(self.scale), _ptr(self.w_out))


def pack_swiglu_weight(w1: torch.Tensor) -> torch.Tensor:
    """[2F, C] (rows 0..F-1 feed SiLU, rows F..2F-1 are the linear half, kernel_test/transition.py:40-42)
    -> 256-row tiles [128 SiLU rows | 128 linear rows] so both halves of an output meet in one tile."""
    f = w1.shape[0] // 2
    assert f % 128 == 0
    a, b = w1[:f].reshape(f // 128, 128, -1), w1[f:].reshape(f // 128, 128, -1)
    return torch.cat([a, b], 1).reshape(2 * f, -1)


class PackedTransition:
    def __init__(self, state: State, prefix: str, device):
        w1 = state[prefix + "transition1.weight"]
        self.C = w1.shape[1]
        self.F = w1.shape[0] // 2
        self.w1 = _b16(pack_swiglu_weight(w1), device)
        self.w2 = _b16(state[prefix + "transition2.weight"], device)
        self.ln_g = _f32(state.get(prefix + "input_layer_norm.weight"), device)
        self.ln_b = _f32(state.get(prefix + "input_layer_norm.bias"), device)
        self.c = TransitionWeights(_ptr(self.ln_g), _ptr(self.ln_b), _ptr(self.w1), _ptr(self.w2))


def _pad_heads_rows(w: torch.Tensor, num_head: int, dp: int) -> torch.Tensor:
    """[H*d, C] -> [H*dp, C] with zero rows after each head's d rows."""
    hd, cdim = w.shape
    d = hd // num_head
    out = torch.zeros(num_head, dp, cdim, dtype=w.dtype)
    out[:, :d] = w.reshape(num_head, d, cdim).cpu()
    return out.reshape(num_head * dp, cdim)


class PackedSelfAttention:
    """AttentionPairBias weights with the head dimension padded to 32 or 64 (zero rows/columns)."""

    def __init__(self, state: State, prefix: str, device, num_head: int = 16):
        q = state[prefix + "q_projection.weight"].detach().float().cpu()
        c = q.shape[0]
        d = c // num_head
        self.H, self.C, self.d = num_head, c, d
        self.Dp = 32 if d <= 32 else 64
        assert d <= 64
        ws = [_pad_heads_rows(state[prefix + n + ".weight"].detach().float().cpu(), num_head, self.Dp)
              for n in ("q_projection", "k_projection", "v_projection", "gating_query")]
        self.w_qkvg = _b16(torch.cat(ws, 0), device)
        wd = num_head * self.Dp
        bias = torch.zeros(4 * wd)
        qb = state.get(prefix + "q_projection.bias")
        if qb is not None:
            bias[:wd] = _pad_heads_rows(qb.detach().float().cpu()[:, None], num_head, self.Dp)[:, 0]
        scale = torch.ones(4 * wd)
        scale[:wd] = d ** -0.5
        self.bias, self.scale = _f32(bias, device), _f32(scale, device)
        t2 = state[prefix + "adaptive_zero_init.transition2.weight"].detach().float().cpu()  # [c_out, H*d]
        self.w_out = _b16(_pad_heads_rows(t2.T.contiguous(), num_head, self.Dp).T.contiguous(), device)  # [c_out, H*Dp]


class PackedPairformerBlock:
    def __init__(self, state: State, prefix: str, device, with_single: bool = True):
        self.tri_out = PackedTriMul(state, prefix + "triangle_multiplication_outgoing.", device)
        self.tri_in = PackedTriMul(state, prefix + "triangle_multiplication_incoming.", device)
        self.att_start = PackedTriAttn(state, prefix + "pair_attention1.", device)
        self.att_end = PackedTriAttn(state, prefix + "pair_attention2.", device)
        self.pair_transition = PackedTransition(state, prefix + "pair_transition.", device)
        self.with_single = with_single
        w = PairformerWeights()
        w.tri_out, w.tri_in = self.tri_out.c, self.tri_in.c
        w.att_start, w.att_end = self.att_start.c, self.att_end.c
        w.pair_transition = self.pair_transition.c
        if with_single:
            self.spl_g = _f32(state.get(prefix + "single_pair_logits_norm.weight"), device)
            self.spl_b = _f32(state.get(prefix + "single_pair_logits_norm.bias"), device)
            self.spl_w = _f32(state[prefix + "single_pair_logits_projection.weight"], device)
            self.sa = PackedSelfAttention(state, prefix + "single_attention_.", device, 16)
            self.sa_ln_g = _f32(state.get(prefix + "single_attention_.adaptive_layernorm.layer_norm.weight"), device)
            self.sa_ln_b = _f32(state.get(prefix + "single_attention_.adaptive_layernorm.layer_norm.bias"), device)
            self.single_transition = PackedTransition(state, prefix + "single_transition.", device)
            w.spl_ln_gamma, w.spl_ln_beta, w.spl_w = _ptr(self.spl_g), _ptr(self.spl_b), _ptr(self.spl_w)
            w.sa_ln_gamma, w.sa_ln_beta = _ptr(self.sa_ln_g), _ptr(self.sa_ln_b)
            w.sa_w_qkvg, w.sa_qkvg_bias, w.sa_qkvg_scale = _ptr(self.sa.w_qkvg), _ptr(self.sa.bias), _ptr(self.sa.scale)
            w.sa_w_out = _ptr(self.sa.w_out)
            w.single_transition = self.single_transition.c
        self.c = w


# ---------------------------------------------------------------------------------------------
# operators
# ---------------------------------------------------------------------------------------------
def layernorm(x: torch.Tensor, gamma=None, beta=None, eps: float = 1e-5, proj_w: Optional[torch.Tensor] = None,
              want_y: bool = True, mod_scale=None, mod_shift=None):
    """LayerNorm over the last dim of a bf16 tensor (width 128 / 384 / 768).  With ``proj_w`` [H, C]
    (float32) also returns proj [H, rows] float32.  ``mod_scale`` / ``mod_shift`` [rows_mod, C] bf16
    apply the AdaLN modulation sigmoid(scale) * y + shift, broadcast over leading dims."""
    _need_cuda(x, gamma, beta, proj_w)
    assert x.dtype == BF16 and x.is_contiguous()
    dev = _dev(x)
    cdim = x.shape[-1]
    rows = x.numel() // cdim
    y = torch.empty_like(x) if want_y else None
    h = 0 if proj_w is None else proj_w.shape[0]
    proj = torch.empty(h, rows, dtype=torch.float32, device=x.device) if h else None
    mod_rows = 0 if mod_scale is None else mod_scale.numel() // cdim
    rc = load().xfold_layernorm_fwd(ctx(dev), _ptr(x), cdim, _ptr(y), cdim, rows, cdim, _ptr(gamma), _ptr(beta), eps, h,
                                    _ptr(proj_w), _ptr(proj), rows, _ptr(mod_scale), _ptr(mod_shift), mod_rows,
                                    _stream(dev))
    check(rc, dev, "xfold_layernorm_fwd")
    return (y, proj) if h else y


def swiglu(x: torch.Tensor) -> torch.Tensor:
    _need_cuda(x)
    assert x.dtype == BF16 and x.is_contiguous()
    dev = _dev(x)
    f = x.shape[-1] // 2
    out = torch.empty(*x.shape[:-1], f, dtype=BF16, device=x.device)
    rc = load().xfold_swiglu_fwd(ctx(dev), _ptr(x), _ptr(out), x.numel() // (2 * f), f, _stream(dev))
    check(rc, dev, "xfold_swiglu_fwd")
    return out


def linear(x: torch.Tensor, w: torch.Tensor, bias=None, scale=None) -> torch.Tensor:
    """x [..., K] bf16, w [N, K] bf16 -> [..., N] bf16 ((x w^T + bias) * scale)."""
    _need_cuda(x, w, bias, scale)
    assert x.dtype == BF16 and w.dtype == BF16 and x.is_contiguous() and w.is_contiguous()
    dev = _dev(x)
    k, n = x.shape[-1], w.shape[0]
    m = x.numel() // k
    out = torch.empty(*x.shape[:-1], n, dtype=BF16, device=x.device)
    rc = load().xfold_linear_fwd(ctx(dev), _ptr(x), k, m, k, _ptr(w), n, _ptr(bias), _ptr(scale), _ptr(out), n, _stream(dev))
    check(rc, dev, "xfold_linear_fwd")
    return out


def linear_gate_residual(x, w, gate=None, resid=None, row_gate_mod: int = 0, out=None):
    _need_cuda(x, w, gate, resid)
    dev = _dev(x)
    k, n = x.shape[-1], w.shape[0]
    m = x.numel() // k
    if out is None:
        out = torch.empty(*x.shape[:-1], n, dtype=BF16, device=x.device)
    rc = load().xfold_linear_gate_residual_fwd(ctx(dev), _ptr(x), k, m, k, _ptr(w), n, _ptr(gate), n, row_gate_mod,
                                               _ptr(resid), n, _ptr(out), n, _stream(dev))
    check(rc, dev, "xfold_linear_gate_residual_fwd")
    return out


def linear_swiglu(x, w_packed):
    _need_cuda(x, w_packed)
    dev = _dev(x)
    k, f = x.shape[-1], w_packed.shape[0] // 2
    m = x.numel() // k
    out = torch.empty(*x.shape[:-1], f, dtype=BF16, device=x.device)
    rc = load().xfold_linear_swiglu_fwd(ctx(dev), _ptr(x), k, m, k, _ptr(w_packed), f, _ptr(out), f, _stream(dev))
    check(rc, dev, "xfold_linear_swiglu_fwd")
    return out


def batched_contract(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """out[c, i, j] = sum_k a[c, i, k] * b[c, j, k]; the last dim must be a multiple of 8."""
    _need_cuda(a, b)
    assert a.dtype == BF16 and b.dtype == BF16 and a.is_contiguous() and b.is_contiguous()
    dev = _dev(a)
    ch, mi, kk = a.shape
    nj = b.shape[1]
    ldo = (nj + 7) // 8 * 8
    out = torch.empty(ch, mi, ldo, dtype=BF16, device=a.device)
    rc = load().xfold_batched_contract_fwd(ctx(dev), _ptr(a), _ptr(b), _ptr(out), ch, mi, nj, kk, kk, mi * kk, nj * kk,
                                           ldo, mi * ldo, _stream(dev))
    check(rc, dev, "xfold_batched_contract_fwd")
    return out[:, :, :nj]


def triangle_multiplication_(z: torch.Tensor, mask: Optional[torch.Tensor], w: PackedTriMul, outgoing: bool):
    """In place: z += TriangleMultiplication(z, mask).  z bf16 [N, N, 128]; mask float32 [N, N]."""
    _need_cuda(z, mask)
    assert z.dtype == BF16 and z.is_contiguous() and z.shape[0] == z.shape[1] and z.shape[2] == 128
    dev = _dev(z)
    n = z.shape[0]
    lib = load()
    nb = lib.xfold_trimul_workspace_bytes(n)
    ws = _Workspace.get(dev, nb)
    if mask is not None:
        mask = mask.to(torch.float32).contiguous()
    rc = lib.xfold_triangle_multiplication_fwd(ctx(dev), _ptr(z), _ptr(mask), n, int(outgoing), C.byref(w.c), _ptr(ws),
                                               ws.numel(), _stream(dev))
    check(rc, dev, "xfold_triangle_multiplication_fwd")
    return z


def triangle_attention_(z: torch.Tensor, mask: Optional[torch.Tensor], w: PackedTriAttn, transpose: bool):
    """In place: z += TriangleAttention(z, mask) (starting node, or ending node when ``transpose``)."""
    _need_cuda(z, mask)
    assert z.dtype == BF16 and z.is_contiguous() and z.shape[0] == z.shape[1] and z.shape[2] == 128
    dev = _dev(z)
    n = z.shape[0]
    lib = load()
    ws = _Workspace.get(dev, lib.xfold_triattn_workspace_bytes(n))
    if mask is not None:
        mask = mask.to(torch.float32).contiguous()
    rc = lib.xfold_triangle_attention_fwd(ctx(dev), _ptr(z), _ptr(mask), n, int(transpose), C.byref(w.c), _ptr(ws),
                                          ws.numel(), _stream(dev))
    check(rc, dev, "xfold_triangle_attention_fwd")
    return z


def transition_(x: torch.Tensor, w: PackedTransition):
    """In place: x += Transition(x) over the last dim (128 or 384)."""
    _need_cuda(x)
    assert x.dtype == BF16 and x.is_contiguous() and x.shape[-1] == w.C
    dev = _dev(x)
    rows = x.numel() // w.C
    lib = load()
    ws = _Workspace.get(dev, lib.xfold_transition_workspace_bytes(rows, w.C, w.F))
    rc = lib.xfold_transition_fwd(ctx(dev), _ptr(x), rows, w.C, w.F, C.byref(w.c), _ptr(ws), ws.numel(), _stream(dev))
    check(rc, dev, "xfold_transition_fwd")
    return x


def prepare_pair_bias(pair_bias: torch.Tensor) -> torch.Tensor:
    """float32 [H, S, S] -> the operand the attention kernel reads: float16 [H, S, pad8(S)] holding bias * log2(e)
    (``xfold_pair_bias_prepare_fwd``).  Worth doing once when the same bias serves many calls (the diffusion
    transformer's pair logits, the same for every denoising step)."""
    _need_cuda(pair_bias)
    assert pair_bias.dtype == torch.float32 and pair_bias.is_contiguous() and pair_bias.dim() == 3
    h, s, s2 = pair_bias.shape
    assert s == s2
    dev = _dev(pair_bias)
    out = torch.empty(h, s, (s + 7) // 8 * 8, dtype=torch.float16, device=pair_bias.device)
    check(load().xfold_pair_bias_prepare_fwd(ctx(dev), _ptr(pair_bias), h, s, _ptr(out), _stream(dev)), dev,
          "xfold_pair_bias_prepare_fwd")
    return out


def attention_pair_bias_core(xn: torch.Tensor, w: PackedSelfAttention, pair_bias: torch.Tensor,
                             mask: Optional[torch.Tensor]) -> torch.Tensor:
    """xn bf16 [B, S, C] (normalised input), pair_bias float32 [H, S, S] or the float16 [H, S, pad8(S)] tensor of
    ``prepare_pair_bias``, mask float32 [S] -> gated attention output bf16 [B, S, H * Dp] (head dim padded to Dp)."""
    _need_cuda(xn, pair_bias, mask)
    assert xn.dtype == BF16 and xn.is_contiguous() and pair_bias.is_contiguous()
    dev = _dev(xn)
    b, s, cdim = xn.shape
    lib = load()
    ws = _Workspace.get(dev, lib.xfold_apb_workspace_bytes(b, s, w.H, w.Dp))
    out = torch.empty(b, s, w.H * w.Dp, dtype=BF16, device=xn.device)
    if mask is not None:
        mask = mask.to(torch.float32).contiguous()
    if pair_bias.dtype == torch.float16:
        assert tuple(pair_bias.shape) == (w.H, s, (s + 7) // 8 * 8)
        fn, name = lib.xfold_attention_pair_bias_core_prepared_fwd, "xfold_attention_pair_bias_core_prepared_fwd"
    else:
        assert pair_bias.dtype == torch.float32 and tuple(pair_bias.shape) == (w.H, s, s)
        fn, name = lib.xfold_attention_pair_bias_core_fwd, "xfold_attention_pair_bias_core_fwd"
    rc = fn(ctx(dev), _ptr(xn), b, s, cdim, w.H, w.Dp, _ptr(w.w_qkvg), _ptr(w.bias), _ptr(w.scale), _ptr(pair_bias),
            _ptr(mask), _ptr(out), _ptr(ws), ws.numel(), _stream(dev))
    check(rc, dev, name)
    return out


class PackedCrossAttention:
    """Weights of the gated cross attention in the reference's op layout (query_w / gating_w [a, H, D], query_b [1, H, D],
    key_w / value_w [m, H, D]; prototypes/Batched_DiffusionCrossAttention.py) stacked into the two projection matrices of
    ``xfold_cross_attention_fwd``."""

    def __init__(self, query_w, query_b, key_w, value_w, gating_w, device):
        a, h, d = query_w.shape
        m = key_w.shape[0]
        self.H, self.D, self.Ca, self.Cm = h, d, a, m
        flat = lambda w: w.detach().float().reshape(w.shape[0], h * d).T          # [H*D, in]
        self.w_qg = _b16(torch.cat([flat(query_w), flat(gating_w)], 0), device)
        self.w_kv = _b16(torch.cat([flat(key_w), flat(value_w)], 0), device)
        bias = torch.zeros(2 * h * d)
        if query_b is not None:
            bias[: h * d] = query_b.detach().float().reshape(-1).cpu()
        scale = torch.ones(2 * h * d)
        scale[: h * d] = d ** -0.5
        self.bias, self.scale = _f32(bias, device), _f32(scale, device)


def cross_attention(q_data: torch.Tensor, m_data: torch.Tensor, batched_bias: torch.Tensor, w: PackedCrossAttention):
    """q_data bf16 [B, S, a], m_data bf16 [B, K, m], batched_bias float32 [B, H, S, K] -> bf16 [B, S, H, D]."""
    _need_cuda(q_data, m_data, batched_bias)
    assert q_data.dtype == BF16 and m_data.dtype == BF16 and batched_bias.dtype == torch.float32
    q_data, m_data, batched_bias = q_data.contiguous(), m_data.contiguous(), batched_bias.contiguous()
    dev = _dev(q_data)
    b, s_, _ = q_data.shape
    k = m_data.shape[1]
    assert tuple(batched_bias.shape) == (b, w.H, s_, k)
    lib = load()
    ws = _Workspace.get(dev, lib.xfold_cross_attention_workspace_bytes(b, s_, k, w.H, w.D))
    out = torch.empty(b, s_, w.H, w.D, dtype=BF16, device=q_data.device)
    rc = lib.xfold_cross_attention_fwd(ctx(dev), _ptr(q_data), _ptr(m_data), b, s_, k, w.Ca, w.Cm, w.H, w.D, _ptr(w.w_qg),
                                       _ptr(w.bias), _ptr(w.scale), _ptr(w.w_kv), _ptr(batched_bias), _ptr(out), _ptr(ws),
                                       ws.numel(), _stream(dev))
    check(rc, dev, "xfold_cross_attention_fwd")
    return out


def pairformer_block_(z: torch.Tensor, s: Optional[torch.Tensor], pair_mask, seq_mask, w: PackedPairformerBlock):
    """In place: one Pairformer block on z bf16 [N, N, 128] and s bf16 [N, 384]."""
    _need_cuda(z, s, pair_mask, seq_mask)
    assert z.dtype == BF16 and z.is_contiguous()
    dev = _dev(z)
    n = z.shape[0]
    lib = load()
    ws = _Workspace.get(dev, lib.xfold_pairformer_workspace_bytes(n))
    pm = None if pair_mask is None else pair_mask.to(torch.float32).contiguous()
    sm = None if seq_mask is None else seq_mask.to(torch.float32).contiguous()
    rc = lib.xfold_pairformer_block_fwd(ctx(dev), _ptr(z), _ptr(s), _ptr(pm), _ptr(sm), n, C.byref(w.c), _ptr(ws),
                                        ws.numel(), _stream(dev))
    check(rc, dev, "xfold_pairformer_block_fwd")
    return z, s


class PackedPairformerStack:
    """The blocks of a trunk (``trunk_pairformer.{i}.`` in the model's state dict, d_alphafold3.py:160-166) packed
    into one contiguous array of weight structs, so that the whole loop is one C-ABI call."""

    def __init__(self, blocks):
        self.blocks = list(blocks)
        self.c = (PairformerWeights * len(self.blocks))(*[b.c for b in self.blocks])

    @classmethod
    def from_state(cls, state: State, num_blocks: int, device, prefix: str = "trunk_pairformer.", with_single: bool = True):
        return cls(PackedPairformerBlock(state, f"{prefix}{i}.", device, with_single) for i in range(num_blocks))

    def __len__(self):
        return len(self.blocks)

    def __iter__(self):
        return iter(self.blocks)


def pairformer_stack_(z: torch.Tensor, s: Optional[torch.Tensor], pair_mask, seq_mask, w: PackedPairformerStack):
    """In place: the trunk loop of d_alphafold3.py:242-244, every block of ``w`` applied in order to z and s."""
    _need_cuda(z, s, pair_mask, seq_mask)
    assert z.dtype == BF16 and z.is_contiguous() and (s is None or (s.dtype == BF16 and s.is_contiguous()))
    dev = _dev(z)
    n = z.shape[0]
    lib = load()
    ws = _Workspace.get(dev, lib.xfold_pairformer_workspace_bytes(n))
    pm = None if pair_mask is None else pair_mask.to(torch.float32).contiguous()
    sm = None if seq_mask is None else seq_mask.to(torch.float32).contiguous()
    rc = lib.xfold_pairformer_stack_fwd(ctx(dev), _ptr(z), _ptr(s), _ptr(pm), _ptr(sm), n, w.c, len(w), _ptr(ws),
                                        ws.numel(), _stream(dev))
    check(rc, dev, "xfold_pairformer_stack_fwd")
    return z, s


# ---------------------------------------------------------------------------------------------
# fp32 validation build: float32 weights in the reference's own layouts, float32 z and s
# ---------------------------------------------------------------------------------------------
class PackedPairformerBlockF32:
    """Float32 weights of one block for ``xfold_pairformer_stack_f32_fwd``: nothing is re-laid-out except that the
    four attention projections are stacked into one matrix."""

    def __init__(self, state: State, prefix: str, device, with_single: bool = True):
        self._keep = []

        def f(name):
            t = state.get(prefix + name)
            if t is None:
                return None
            t = t.detach().to(device=device, dtype=torch.float32).contiguous()
            self._keep.append(t)
            return t.data_ptr()

        def cat(names):
            t = torch.cat([state[prefix + n].detach().float() for n in names], 0).to(device).contiguous()
            self._keep.append(t)
            return t.data_ptr()

        def trimul(p):
            return _cabi.TriMulWeightsF32(f(p + "left_norm_input.weight"), f(p + "left_norm_input.bias"), f(p + "projection.weight"),
                                          f(p + "gate.weight"), f(p + "center_norm.weight"), f(p + "center_norm.bias"),
                                          f(p + "output_projection.weight"), f(p + "gating_linear.weight"))

        def triattn(p):
            return _cabi.TriAttnWeightsF32(f(p + "act_norm.weight"), f(p + "act_norm.bias"), f(p + "pair_bias_projection.weight"),
                                           cat([p + n + ".weight" for n in ("q_projection", "k_projection", "v_projection", "gating_query")]),
                                           f(p + "output_projection.weight"))

        def transition(p):
            return _cabi.TransitionWeightsF32(f(p + "input_layer_norm.weight"), f(p + "input_layer_norm.bias"),
                                              f(p + "transition1.weight"), f(p + "transition2.weight"))

        w = _cabi.PairformerWeightsF32()
        w.tri_out, w.tri_in = trimul("triangle_multiplication_outgoing."), trimul("triangle_multiplication_incoming.")
        w.att_start, w.att_end = triattn("pair_attention1."), triattn("pair_attention2.")
        w.pair_transition = transition("pair_transition.")
        if with_single:
            sa = "single_attention_."
            w.spl_ln_gamma, w.spl_ln_beta = f("single_pair_logits_norm.weight"), f("single_pair_logits_norm.bias")
            w.spl_w = f("single_pair_logits_projection.weight")
            w.sa_ln_gamma, w.sa_ln_beta = f(sa + "adaptive_layernorm.layer_norm.weight"), f(sa + "adaptive_layernorm.layer_norm.bias")
            w.sa_qkvg = cat([sa + n + ".weight" for n in ("q_projection", "k_projection", "v_projection", "gating_query")])
            c = state[prefix + sa + "q_projection.weight"].shape[0]
            b = torch.zeros(4 * c)
            if prefix + sa + "q_projection.bias" in state:
                b[:c] = state[prefix + sa + "q_projection.bias"].detach().float().cpu()
            b = b.to(device)
            self._keep.append(b)
            w.sa_qkvg_bias = b.data_ptr()
            w.sa_out = f(sa + "adaptive_zero_init.transition2.weight")
            w.single_transition = transition("single_transition.")
        self.c = w


def pairformer_stack_f32_(z: torch.Tensor, s: Optional[torch.Tensor], pair_mask, seq_mask, blocks):
    """In place, float32: the blocks of ``blocks`` (PackedPairformerBlockF32) applied in order to z [N, N, 128] and s [N, 384]."""
    _need_cuda(z, s, pair_mask, seq_mask)
    assert z.dtype == torch.float32 and z.is_contiguous() and (s is None or (s.dtype == torch.float32 and s.is_contiguous()))
    dev = _dev(z)
    n = z.shape[0]
    lib = load()
    ws = _Workspace.get(dev, lib.xfold_pairformer_f32_workspace_bytes(n))
    pm = None if pair_mask is None else pair_mask.to(torch.float32).contiguous()
    sm = None if seq_mask is None else seq_mask.to(torch.float32).contiguous()
    arr = (_cabi.PairformerWeightsF32 * len(blocks))(*[b.c for b in blocks])
    rc = lib.xfold_pairformer_stack_f32_fwd(ctx(dev), _ptr(z), _ptr(s), _ptr(pm), _ptr(sm), n, arr, len(blocks), _ptr(ws),
                                            ws.numel(), _stream(dev))
    check(rc, dev, "xfold_pairformer_stack_f32_fwd")
    return z, s


# ---------------------------------------------------------------------------------------------
# row-shard stages (the multi-GPU block composes these with collectives in between)
# ---------------------------------------------------------------------------------------------
def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


def stage_trimul_project(z: torch.Tensor, mask_shard: Optional[torch.Tensor], w: PackedTriMul):
    """z [R, N, 128] -> a, b [R, 128, ld] (row-interleaved channel-major) and g [R, N, 128]."""
    _need_cuda(z, mask_shard)
    dev = _dev(z)
    r, n, _ = z.shape
    ld = _pad8(n)
    x = torch.empty_like(z)
    a = torch.zeros(r, 128, ld, dtype=BF16, device=z.device) if ld != n else torch.empty(r, 128, ld, dtype=BF16, device=z.device)
    b = torch.zeros_like(a) if ld != n else torch.empty_like(a)
    g = torch.empty_like(z)
    m = None if mask_shard is None else mask_shard.to(torch.float32).contiguous()
    rc = load().xfold_trimul_project_fwd(ctx(dev), _ptr(z), _ptr(m), r, n, C.byref(w.c), _ptr(x), _ptr(a), _ptr(b),
                                         _ptr(g), ld, _stream(dev))
    check(rc, dev, "xfold_trimul_project_fwd")
    return a, b, g


def stage_trimul_contract(a: torch.Tensor, b_full: torch.Tensor, n: int) -> torch.Tensor:
    """o[i, c, j] = sum_k a[i, c, k] * b_full[j, c, k] over the first n entries of k."""
    _need_cuda(a, b_full)
    dev = _dev(a)
    r, _, ld = a.shape
    nj = b_full.shape[0]
    ldo = _pad8(nj)
    o = torch.empty(r, 128, ldo, dtype=BF16, device=a.device)
    rc = load().xfold_trimul_contract_fwd(ctx(dev), _ptr(a), _ptr(b_full.contiguous()), r, nj, n, ld, _ptr(o), ldo,
                                          _stream(dev))
    check(rc, dev, "xfold_trimul_contract_fwd")
    return o


def stage_trimul_contract_planes(a: torch.Tensor, b: torch.Tensor, n: int) -> torch.Tensor:
    """Channel-major planes: o[c, i, j] = sum_k a[c, i, k] * b[c, j, k] over the first n entries of k."""
    _need_cuda(a, b)
    dev = _dev(a)
    ch, ni, ld = a.shape
    nj = b.shape[1]
    ldo = _pad8(nj)
    o = torch.empty(ch, ni, ldo, dtype=BF16, device=a.device)
    rc = load().xfold_trimul_contract_planes_fwd(ctx(dev), _ptr(a), _ptr(b), ch, ni, nj, n, ld, _ptr(o), ldo, _stream(dev))
    check(rc, dev, "xfold_trimul_contract_planes_fwd")
    return o


def stage_trimul_contract_planes_incoming(a: torch.Tensor, b: torch.Tensor, n: int) -> torch.Tensor:
    """The incoming-edges product on the same channel planes: o[c, i, j] = sum_k a[c, k, j] * b[c, k, i] over the first n
    rows k; a, b [channels, n, ld] -> o [channels, n, pad8(n)].  Nothing is transposed: the tensor-core operands are
    read MN-major."""
    _need_cuda(a, b)
    dev = _dev(a)
    ch, nk, ld = a.shape
    assert b.shape == a.shape and a.is_contiguous() and b.is_contiguous() and nk >= n
    ldo = _pad8(n)
    o = torch.empty(ch, n, ldo, dtype=BF16, device=a.device)
    rc = load().xfold_trimul_contract_planes_incoming_fwd(ctx(dev), _ptr(a), _ptr(b), ch, nk, n, n, ld, _ptr(o), ldo,
                                                          _stream(dev))
    check(rc, dev, "xfold_trimul_contract_planes_incoming_fwd")
    return o


def stage_trimul_output(o: torch.Tensor, g: torch.Tensor, z: torch.Tensor, w: PackedTriMul) -> None:
    _need_cuda(o, g, z)
    dev = _dev(z)
    r, n, _ = z.shape
    x = torch.empty_like(z)
    rc = load().xfold_trimul_output_fwd(ctx(dev), _ptr(o), o.shape[2], _ptr(g), r, n, C.byref(w.c), _ptr(x), _ptr(z),
                                        _stream(dev))
    check(rc, dev, "xfold_trimul_output_fwd")


def stage_triattn_bias(z: torch.Tensor, w: PackedTriAttn, rows_are_keys: bool):
    """x = act_norm(z) and this shard's part of the pair bias [head, query, key] (bf16):
    [4, R, pad8(N)] when the shard's rows are query rows, [4, N, R] when they are key rows."""
    _need_cuda(z)
    dev = _dev(z)
    r, n, _ = z.shape
    x = torch.empty_like(z)
    if rows_are_keys:
        pitch = _pad8(r)
        bias = torch.zeros(4, n, pitch, dtype=BF16, device=z.device)
        plane = n * pitch
    else:
        pitch = _pad8(n)
        bias = torch.zeros(4, r, pitch, dtype=BF16, device=z.device)
        plane = r * pitch
    rc = load().xfold_triattn_bias_fwd(ctx(dev), _ptr(z), r, n, C.byref(w.c), _ptr(x), _ptr(bias), pitch, plane,
                                       int(rows_are_keys), _stream(dev))
    check(rc, dev, "xfold_triattn_bias_fwd")
    return x, (bias[..., :r] if rows_are_keys else bias)


def stage_triattn_core(x: torch.Tensor, bias_t: torch.Tensor, mask_shard: Optional[torch.Tensor], w: PackedTriAttn,
                       z: torch.Tensor) -> None:
    _need_cuda(x, bias_t, mask_shard, z)
    dev = _dev(z)
    r, n, _ = z.shape
    lib = load()
    mext_bytes = C.c_size_t()
    qkvg_bytes = lib.xfold_triattn_core_scratch_bytes(r, n, C.byref(mext_bytes))
    qkvg = torch.empty(qkvg_bytes, dtype=torch.uint8, device=z.device)
    mext = torch.empty(mext_bytes.value, dtype=torch.uint8, device=z.device)
    m = None if mask_shard is None else mask_shard.to(torch.float32).contiguous()
    bias_t = bias_t.contiguous()
    assert bias_t.shape[0] == 4 and bias_t.shape[1] == n and bias_t.shape[2] % 8 == 0
    rc = lib.xfold_triattn_core_fwd(ctx(dev), _ptr(x), _ptr(bias_t), bias_t.shape[2], _ptr(m), n, r, n, C.byref(w.c),
                                    _ptr(qkvg), _ptr(mext), _ptr(z), _stream(dev))
    check(rc, dev, "xfold_triattn_core_fwd")


def stage_transition(x: torch.Tensor, w: PackedTransition) -> None:
    transition_(x, w)


def stage_pair_logits(z: torch.Tensor, w: PackedPairformerBlock) -> torch.Tensor:
    """Pair logits [head, query, key] contributed by this shard's (query) rows: bf16 [16, R, pad8(N)]."""
    _need_cuda(z)
    dev = _dev(z)
    r, n, _ = z.shape
    pitch = _pad8(n)
    out = torch.zeros(16, r, pitch, dtype=BF16, device=z.device)
    rc = load().xfold_pair_logits_fwd(ctx(dev), _ptr(z), r, n, _ptr(w.spl_g), _ptr(w.spl_b), _ptr(w.spl_w), _ptr(out),
                                      pitch, r * pitch, 0, _stream(dev))
    check(rc, dev, "xfold_pair_logits_fwd")
    return out


def stage_single_update(s: torch.Tensor, pl_t: torch.Tensor, seq_mask: Optional[torch.Tensor],
                        w: PackedPairformerBlock) -> None:
    _need_cuda(s, pl_t, seq_mask)
    dev = _dev(s)
    n = s.shape[0]
    lib = load()
    nbytes = lib.xfold_single_update_workspace_bytes(n)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=s.device)
    pl_t = pl_t.contiguous()
    sm = None if seq_mask is None else seq_mask.to(torch.float32).contiguous()
    rc = lib.xfold_single_update_fwd(ctx(dev), _ptr(s), _ptr(pl_t), pl_t.shape[2], _ptr(sm), n, C.byref(w.c), _ptr(ws),
                                     nbytes, _stream(dev))
    check(rc, dev, "xfold_single_update_fwd")
