"""The reference's native operator interface on the GPU: ``torch.ops._alpha_attention.*``.

The reference defines six operator schemas in its C++ extension (``TORCH_LIBRARY(_alpha_attention)``,
xsmm_kernels/csrc/Alpha_Attention.cpp:181-211), implements five of them for the CPU dispatch key (:215-221) and registers
shape-only kernels for tracing (xsmm_kernels/prototypes/register_fake_kernels.py:12-125).  ``register()`` gives the same
five operators a CUDA implementation on this library's C ABI and Meta kernels with the same shape rules, so the
reference's own wrappers (``prototypes/*.py``) run unchanged on GPU tensors:

* arguments arrive exactly as those wrappers pass them (activations contiguous, weights in the op layouts
  ``[c, H, D]`` / ``[H, D, c]``, masks as float32 additive biases ``1e9 * (mask - 1)``);
* results are the PADDED tensors the wrappers expect and narrow themselves (TriangleMultiplication.py:54-58,
  GridSelfAttention.py:47-49): sequence axes rounded up to 64, TriangleMultiplication's two token axes to 32;
* the schemas are defined here only when no extension has defined them already.

Weights are re-packed into the kernel layouts on first use and cached per (storage, version).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from . import ops

TRI_BLOCKSIZE = 32   # prototypes/__init__.py:3
QKV_BLOCKSIZE = 64   # prototypes/__init__.py:5
BF16 = torch.bfloat16

SCHEMAS = {
    "grid_self_attn_forward": "(Tensor q_data, Tensor bias, Tensor nonbatched_bias, Tensor query_w, Tensor key_w, "
                              "Tensor value_w, Tensor gating_w, Tensor output_w, int key_dim, int value_dim) -> Tensor",
    "transition_forward": "(Tensor act, Tensor transition1, Tensor transition2, Tensor layernorm_weight, "
                          "Tensor layernorm_bias) -> Tensor",
    "batch_diffusion_self_attention_forward": "(Tensor q_data, Tensor bias, Tensor nonbatched_bias, Tensor query_w, "
                                              "Tensor query_b, Tensor key_w, Tensor value_w, Tensor gating_w, int key_dim, "
                                              "int value_dim) -> Tensor",
    "diffusion_self_attention_forward": "(Tensor q_data, Tensor bias, Tensor nonbatched_bias, Tensor query_w, "
                                        "Tensor query_b, Tensor key_w, Tensor value_w, Tensor gating_w, int key_dim, "
                                        "int value_dim) -> Tensor",
    "batch_diffusion_cross_attention_forward": "(Tensor q_data, Tensor m_data, Tensor batched_bias, Tensor query_w, "
                                               "Tensor query_b, Tensor key_w, Tensor value_w, Tensor gating_w, int key_dim, "
                                               "int value_dim) -> Tensor",
    "traingle_multiplication_forward": "(Tensor act, Tensor mask, int equation_flag, Tensor left_norm_input_weight, "
                                       "Tensor left_norm_input_bias, Tensor projection_weight, Tensor gate_weight, "
                                       "Tensor center_norm_weight, Tensor center_norm_bias, "
                                       "Tensor output_projection_weight, Tensor gating_linear_weight) -> Tensor",
}

_LIBS = []      # torch.library.Library objects must stay referenced, or their registrations vanish
_CACHE: Dict[Tuple, object] = {}


def _pad_to(n: int, block: int) -> int:
    return (n + block - 1) // block * block


def _key(*ts) -> Tuple:
    return tuple((t.data_ptr(), t._version, tuple(t.shape)) for t in ts)


def _cached(name, tensors, make):
    k = (name,) + _key(*tensors)
    v = _CACHE.get(k)
    if v is None:
        if len(_CACHE) > 4096:
            _CACHE.clear()
        v = _CACHE[k] = make()
    return v


def _mask_from_bias(bias: torch.Tensor, rows: int, s: int) -> torch.Tensor:
    """The wrappers pass the token mask as the additive bias 1e9 * (mask - 1) (nn/d_attention.py:63); the kernels take the
    mask itself (and floor the bias they derive from it so that fully masked rows stay finite)."""
    return (bias.reshape(-1, s)[:rows].float() * 1e-9 + 1.0).clamp_(0.0, 1.0).contiguous()


# ---------------------------------------------------------------------------------------------------------------
# CUDA implementations
# ---------------------------------------------------------------------------------------------------------------
def _grid_self_attn(q_data, bias, nonbatched_bias, query_w, key_w, value_w, gating_w, output_w, key_dim, value_dim):
    import ctypes as C
    from ._cabi import check, ctx, load
    b, s, c = q_data.shape
    _, h, d = query_w.shape
    if d > 32:
        raise ops._cabi.XfoldError("grid_self_attn_forward: head dimension up to 32")
    dev = q_data.device

    def pack():
        flat = lambda w: w.detach().float().reshape(c, h * d).T                      # [H*D, c]
        pad = lambda w: ops._pad_heads_rows(flat(w).cpu(), h, 32)
        w_qkvg = ops._b16(torch.cat([pad(query_w), pad(key_w), pad(value_w), pad(gating_w)], 0), dev)
        scale = torch.ones(4 * h * 32)
        scale[: h * 32] = d ** -0.5
        w_out = output_w.detach().float().reshape(h * d, -1).T                       # [c_out, H*D]
        w_out = ops._b16(ops._pad_heads_rows(w_out.T.contiguous().cpu(), h, 32).T.contiguous(), dev)   # [c_out, H*32]
        return w_qkvg, ops._f32(scale, dev), w_out

    w_qkvg, scale, w_out = _cached("gsa", (query_w, key_w, value_w, gating_w, output_w), pack)
    x = q_data.to(BF16).contiguous()
    mask = _mask_from_bias(bias, b, s)
    nb = nonbatched_bias.float().contiguous() if nonbatched_bias.numel() else torch.zeros(h, s, s, device=dev)
    lib = load()
    di = dev.index if dev.index is not None else torch.cuda.current_device()
    ws = ops._Workspace.get(di, lib.xfold_apb_workspace_bytes(b, s, h, 32))
    att = torch.empty(b, s, h * 32, dtype=BF16, device=dev)
    rc = lib.xfold_gated_attention_core_fwd(ctx(di), x.data_ptr(), b, s, c, h, 32, w_qkvg.data_ptr(), None, scale.data_ptr(),
                                            nb.data_ptr(), mask.data_ptr(), s if mask.shape[0] == b else 0, att.data_ptr(),
                                            ws.data_ptr(), ws.numel(), torch.cuda.current_stream(di).cuda_stream)
    check(rc, di, "xfold_gated_attention_core_fwd")
    out = ops.linear(att, w_out)                                                     # [B, S, c_out]
    sp = _pad_to(s, QKV_BLOCKSIZE)
    if sp != s:
        out = torch.nn.functional.pad(out, (0, 0, 0, sp - s))
    return out.to(q_data.dtype)


def _batch_diffusion_self_attention(q_data, bias, nonbatched_bias, query_w, query_b, key_w, value_w, gating_w, key_dim,
                                    value_dim):
    b, s, c = q_data.shape
    _, h, d = query_w.shape
    dev = q_data.device

    def pack():
        flat = lambda w: w.detach().float().reshape(w.shape[0], h * d).T
        state = {"q_projection.weight": flat(query_w), "k_projection.weight": flat(key_w),
                 "v_projection.weight": flat(value_w), "gating_query.weight": flat(gating_w),
                 "q_projection.bias": query_b.detach().float().reshape(-1),
                 "adaptive_zero_init.transition2.weight": torch.zeros(1, h * d)}
        return ops.PackedSelfAttention(state, "", dev, h)

    w = _cached("bdsa", (query_w, query_b, key_w, value_w, gating_w), pack)
    mask = _mask_from_bias(bias, 1, s)[0]
    out = ops.attention_pair_bias_core(q_data.to(BF16).contiguous(), w, nonbatched_bias.float().contiguous(), mask)
    out = out.view(b, s, h, w.Dp)[..., :d]
    sp = _pad_to(s, QKV_BLOCKSIZE)
    if sp != s:
        out = torch.nn.functional.pad(out, (0, 0, 0, 0, 0, sp - s))
    return out.contiguous().to(q_data.dtype)


def _batch_diffusion_cross_attention(q_data, m_data, batched_bias, query_w, query_b, key_w, value_w, gating_w, key_dim,
                                     value_dim):
    s = q_data.shape[1]
    w = _cached("bdca", (query_w, query_b, key_w, value_w, gating_w),
                lambda: ops.PackedCrossAttention(query_w, query_b, key_w, value_w, gating_w, q_data.device))
    out = ops.cross_attention(q_data.to(BF16), m_data.to(BF16), batched_bias.float(), w)
    sp = _pad_to(s, QKV_BLOCKSIZE)
    if sp != s:
        out = torch.nn.functional.pad(out, (0, 0, 0, 0, 0, sp - s))
    return out.to(q_data.dtype)


def _transition(act, transition1, transition2, layernorm_weight, layernorm_bias):
    c = act.shape[-1]

    def pack():   # the op takes the matrices as [in, out] (kernel_test/transition.py:31-36)
        state = {"transition1.weight": transition1.detach().float().T, "transition2.weight": transition2.detach().float().T,
                 "input_layer_norm.weight": layernorm_weight.detach().float(),
                 "input_layer_norm.bias": layernorm_bias.detach().float()}
        return ops.PackedTransition(state, "", act.device)

    w = _cached("tr", (transition1, transition2, layernorm_weight, layernorm_bias), pack)
    import ctypes as C
    from ._cabi import check, ctx, load
    x = act.to(BF16).contiguous()
    upd = torch.empty_like(x)
    di = act.device.index if act.device.index is not None else torch.cuda.current_device()
    rows = x.numel() // c
    lib = load()
    ws = ops._Workspace.get(di, lib.xfold_transition_workspace_bytes(rows, w.C, w.F))
    rc = lib.xfold_transition_update_fwd(ctx(di), x.data_ptr(), upd.data_ptr(), rows, w.C, w.F, C.byref(w.c), ws.data_ptr(),
                                         ws.numel(), torch.cuda.current_stream(di).cuda_stream)
    check(rc, di, "xfold_transition_update_fwd")
    return upd.to(act.dtype)


def _traingle_multiplication(act, mask, equation_flag, left_norm_input_weight, left_norm_input_bias, projection_weight,
                             gate_weight, center_norm_weight, center_norm_bias, output_projection_weight,
                             gating_linear_weight):
    import ctypes as C
    from ._cabi import check, ctx, load
    n, n2, c = act.shape
    if n != n2 or c != 128:
        raise ops._cabi.XfoldError("traingle_multiplication_forward: a square [N, N, 128] pair representation is expected")
    dev = act.device

    def pack():
        # projection / gate arrive de-interleaved by load_xsmm_params: rows [0, c) are a, rows [c, 2c) are b
        # (nn/d_triangle_multiplication.py:128-129); PackedTriMul wants the checkpoint's interleaved order back
        def interleave(w):
            w = w.detach().float()
            out = torch.empty_like(w)
            out[0::2], out[1::2] = w[:c], w[c:]
            return out
        state = {"projection.weight": interleave(projection_weight), "gate.weight": interleave(gate_weight),
                 "gating_linear.weight": gating_linear_weight, "output_projection.weight": output_projection_weight,
                 "left_norm_input.weight": left_norm_input_weight, "left_norm_input.bias": left_norm_input_bias,
                 "center_norm.weight": center_norm_weight, "center_norm.bias": center_norm_bias}
        return ops.PackedTriMul(state, "", dev)

    w = _cached("tm", (left_norm_input_weight, left_norm_input_bias, projection_weight, gate_weight, center_norm_weight,
                       center_norm_bias, output_projection_weight, gating_linear_weight), pack)
    z = act.to(BF16).contiguous()
    m = mask.reshape(n, n).float().contiguous()
    upd = torch.empty_like(z)
    di = dev.index if dev.index is not None else torch.cuda.current_device()
    lib = load()
    ws = ops._Workspace.get(di, lib.xfold_trimul_workspace_bytes(n))
    outgoing = 1 if int(equation_flag) == 0 else 0   # flag 0: "ikc,jkc->ijc" (TriangleMultiplication.py:37-41)
    rc = lib.xfold_triangle_multiplication_update_fwd(ctx(di), z.data_ptr(), upd.data_ptr(), m.data_ptr(), n, outgoing,
                                                      C.byref(w.c), ws.data_ptr(), ws.numel(),
                                                      torch.cuda.current_stream(di).cuda_stream)
    check(rc, di, "xfold_triangle_multiplication_update_fwd")
    np_ = _pad_to(n, TRI_BLOCKSIZE)
    if np_ != n:
        upd = torch.nn.functional.pad(upd, (0, 0, 0, np_ - n, 0, np_ - n))
    return upd.to(act.dtype)


# ---------------------------------------------------------------------------------------------------------------
# Meta kernels: the shape rules of prototypes/register_fake_kernels.py:12-125
# ---------------------------------------------------------------------------------------------------------------
def _meta_grid(q_data, bias, nonbatched_bias, query_w, key_w, value_w, gating_w, output_w, key_dim, value_dim):
    b, s, c = q_data.shape
    return q_data.new_empty((b, _pad_to(s, QKV_BLOCKSIZE), c))


def _meta_transition(act, transition1, transition2, layernorm_weight, layernorm_bias):
    return act.new_empty(act.shape)


def _meta_heads(q_data, second, third, query_w, query_b, key_w, value_w, gating_w, key_dim, value_dim):
    b, s = q_data.shape[:2]
    return q_data.new_empty((b, _pad_to(s, QKV_BLOCKSIZE), query_w.shape[-2], query_w.shape[-1]))


def _meta_trimul(act, mask, equation_flag, *weights):
    b, s, c = act.shape
    return act.new_empty((_pad_to(b, TRI_BLOCKSIZE), _pad_to(s, TRI_BLOCKSIZE), c))


_CUDA = {"grid_self_attn_forward": _grid_self_attn, "transition_forward": _transition,
         "batch_diffusion_self_attention_forward": _batch_diffusion_self_attention,
         "batch_diffusion_cross_attention_forward": _batch_diffusion_cross_attention,
         "traingle_multiplication_forward": _traingle_multiplication}
_META = {"grid_self_attn_forward": _meta_grid, "transition_forward": _meta_transition,
         "batch_diffusion_self_attention_forward": _meta_heads, "batch_diffusion_cross_attention_forward": _meta_heads,
         "traingle_multiplication_forward": _meta_trimul}


def register() -> None:
    """Defines the schemas (unless an extension already did) and registers the CUDA and Meta kernels.  Idempotent."""
    if _LIBS:
        return
    have = True
    try:
        torch.ops._alpha_attention.grid_self_attn_forward  # noqa: B018  (AttributeError when the schema is unknown)
    except (AttributeError, RuntimeError):
        have = False
    if not have:
        d = torch.library.Library("_alpha_attention", "DEF")
        for name, sig in SCHEMAS.items():
            d.define(name + sig)
        _LIBS.append(d)
    impl = torch.library.Library("_alpha_attention", "IMPL")
    _LIBS.append(impl)
    for name, fn in _CUDA.items():
        impl.impl(name, fn, "CUDA")
    for name, fn in _META.items():
        try:
            impl.impl(name, fn, "Meta")
        except RuntimeError:
            pass  # the reference's own fake kernels are registered already
