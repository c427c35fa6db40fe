"""ctypes binding of ``libxfold_b200.so`` (the C ABI declared in ``include/xfold_b200.h``).

This is the only place the package touches the shared library.  It takes the place of the
reference's ``import tpp_pytorch_extension._C`` (xsmm_kernels/prototypes/__init__.py:1): loading it
makes the fused operators available; if the library is missing the import fails loudly; there is
no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libxfold_b200.so")

XFOLD_OK, XFOLD_ERR_ARG, XFOLD_ERR_LAUNCH, XFOLD_ERR_DEVICE, XFOLD_ERR_TIMEOUT = range(5)

vp, ll, ci, cf, sz = C.c_void_p, C.c_longlong, C.c_int, C.c_float, C.c_size_t


class TriMulWeights(C.Structure):
    _fields_ = [("ln_in_gamma", vp), ("ln_in_beta", vp), ("w_in", vp), ("ln_c_gamma", vp), ("ln_c_beta", vp),
                ("w_out", vp)]


class TriAttnWeights(C.Structure):
    _fields_ = [("ln_gamma", vp), ("ln_beta", vp), ("w_bias", vp), ("w_qkvg", vp), ("qkvg_scale", vp), ("w_out", vp)]


class TransitionWeights(C.Structure):
    _fields_ = [("ln_gamma", vp), ("ln_beta", vp), ("w1_packed", vp), ("w2", vp)]


class PairformerWeights(C.Structure):
    _fields_ = [("tri_out", TriMulWeights), ("tri_in", TriMulWeights), ("att_start", TriAttnWeights),
                ("att_end", TriAttnWeights), ("pair_transition", TransitionWeights),
                ("spl_ln_gamma", vp), ("spl_ln_beta", vp), ("spl_w", vp), ("sa_ln_gamma", vp), ("sa_ln_beta", vp),
                ("sa_w_qkvg", vp), ("sa_qkvg_bias", vp), ("sa_qkvg_scale", vp), ("sa_w_out", vp),
                ("single_transition", TransitionWeights)]


class TriMulWeightsF32(C.Structure):
    _fields_ = [(n, vp) for n in ("ln_in_gamma", "ln_in_beta", "projection", "gate", "ln_c_gamma", "ln_c_beta",
                                  "output_projection", "gating_linear")]


class TriAttnWeightsF32(C.Structure):
    _fields_ = [(n, vp) for n in ("ln_gamma", "ln_beta", "pair_bias_projection", "qkvg", "output_projection")]


class TransitionWeightsF32(C.Structure):
    _fields_ = [(n, vp) for n in ("ln_gamma", "ln_beta", "transition1", "transition2")]


class PairformerWeightsF32(C.Structure):
    _fields_ = [("tri_out", TriMulWeightsF32), ("tri_in", TriMulWeightsF32), ("att_start", TriAttnWeightsF32),
                ("att_end", TriAttnWeightsF32), ("pair_transition", TransitionWeightsF32),
                ("spl_ln_gamma", vp), ("spl_ln_beta", vp), ("spl_w", vp), ("sa_ln_gamma", vp), ("sa_ln_beta", vp),
                ("sa_qkvg", vp), ("sa_qkvg_bias", vp), ("sa_out", vp), ("single_transition", TransitionWeightsF32)]


class ShardDesc(C.Structure):
    _fields_ = [("world", ci), ("rank", ci), ("n_tokens", ci), ("row_starts", C.POINTER(ci)),
                ("zbuf0", C.POINTER(vp)), ("zbuf1", C.POINTER(vp)), ("plane_a", C.POINTER(vp)), ("plane_b", C.POINTER(vp)),
                ("plane_o", C.POINTER(vp)), ("bias", C.POINTER(vp)), ("flags", C.POINTER(vp))]


# name -> (restype, argtypes); every symbol include/xfold_b200.h declares
SIGNATURES = {
    "xfold_ctx_create": (ci, [ci, C.POINTER(vp)]),
    "xfold_ctx_destroy": (None, [vp]),
    "xfold_last_error": (C.c_char_p, [vp]),
    "xfold_check_status": (ci, [vp, vp]),
    "xfold_version": (C.c_char_p, []),
    "xfold_launch_count": (ll, [vp]),
    "xfold_profile_enable": (ci, [vp, ci]),
    "xfold_profile_read": (ci, [vp, ci, C.POINTER(cf), C.POINTER(ci)]),
    "xfold_layernorm_fwd": (ci, [vp, vp, ll, vp, ll, ll, ci, vp, vp, cf, ci, vp, vp, ll, vp, vp, ci, vp]),
    "xfold_swiglu_fwd": (ci, [vp, vp, vp, ll, ci, vp]),
    "xfold_linear_fwd": (ci, [vp, vp, ll, ll, ci, vp, ci, vp, vp, vp, ll, vp]),
    "xfold_linear_gate_residual_fwd": (ci, [vp, vp, ll, ll, ci, vp, ci, vp, ll, ci, vp, ll, vp, ll, vp]),
    "xfold_linear_swiglu_fwd": (ci, [vp, vp, ll, ll, ci, vp, ci, vp, ll, vp]),
    "xfold_batched_contract_fwd": (ci, [vp, vp, vp, vp, ci, ci, ci, ci, ll, ll, ll, ll, ll, vp]),
    "xfold_trimul_workspace_bytes": (sz, [ci]),
    "xfold_triangle_multiplication_fwd": (ci, [vp, vp, vp, ci, ci, C.POINTER(TriMulWeights), vp, sz, vp]),
    "xfold_triattn_workspace_bytes": (sz, [ci]),
    "xfold_triangle_attention_fwd": (ci, [vp, vp, vp, ci, ci, C.POINTER(TriAttnWeights), vp, sz, vp]),
    "xfold_transition_workspace_bytes": (sz, [ll, ci, ci]),
    "xfold_transition_fwd": (ci, [vp, vp, ll, ci, ci, C.POINTER(TransitionWeights), vp, sz, vp]),
    "xfold_apb_workspace_bytes": (sz, [ci, ci, ci, ci]),
    "xfold_attention_pair_bias_core_fwd": (ci, [vp, vp, ci, ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
    "xfold_trimul_project_fwd": (ci, [vp, vp, vp, ci, ci, C.POINTER(TriMulWeights), vp, vp, vp, vp, ci, vp]),
    "xfold_trimul_contract_fwd": (ci, [vp, vp, vp, ci, ci, ci, ci, vp, ci, vp]),
    "xfold_trimul_contract_planes_fwd": (ci, [vp, vp, vp, ci, ci, ci, ci, ci, vp, ci, vp]),
    "xfold_trimul_output_fwd": (ci, [vp, vp, ci, vp, ci, ci, C.POINTER(TriMulWeights), vp, vp, vp]),
    "xfold_triattn_bias_fwd": (ci, [vp, vp, ci, ci, C.POINTER(TriAttnWeights), vp, vp, ci, ll, ci, vp]),
    "xfold_triattn_core_scratch_bytes": (sz, [ci, ci, C.POINTER(sz)]),
    "xfold_triattn_core_fwd": (ci, [vp, vp, vp, ci, vp, ll, ci, ci, C.POINTER(TriAttnWeights), vp, vp, vp, vp]),
    "xfold_pair_logits_fwd": (ci, [vp, vp, ci, ci, vp, vp, vp, vp, ci, ll, ci, vp]),
    "xfold_single_update_workspace_bytes": (sz, [ci]),
    "xfold_single_update_fwd": (ci, [vp, vp, vp, ci, vp, ci, C.POINTER(PairformerWeights), vp, sz, vp]),
    "xfold_triangle_multiplication_update_fwd": (ci, [vp, vp, vp, vp, ci, ci, C.POINTER(TriMulWeights), vp, sz, vp]),
    "xfold_triangle_attention_update_fwd": (ci, [vp, vp, vp, vp, ci, ci, C.POINTER(TriAttnWeights), vp, sz, vp]),
    "xfold_transition_update_fwd": (ci, [vp, vp, vp, ll, ci, ci, C.POINTER(TransitionWeights), vp, sz, vp]),
    "xfold_transpose_scatter_fwd": (ci, [vp, vp, ci, ci, ci, C.POINTER(vp), C.POINTER(ci), ci, vp]),
    "xfold_trimul_scatter_channels_fwd": (ci, [vp, vp, vp, ci, ci, ci, ci, C.POINTER(vp), C.POINTER(vp), ci, vp]),
    "xfold_trimul_scatter_rows_fwd": (ci, [vp, vp, ci, ci, ci, ci, C.POINTER(vp), C.POINTER(ci), ci, vp]),
    "xfold_peer_allgather_fwd": (ci, [vp, vp, ll, ll, C.POINTER(vp), ci, vp]),
    "xfold_peer_barrier": (ci, [vp, C.POINTER(vp), ci, ci, ci, vp]),
    "xfold_shard_ctx_create": (ci, [vp, C.POINTER(ShardDesc), C.POINTER(vp)]),
    "xfold_shard_ctx_destroy": (None, [vp]),
    "xfold_shard_workspace_bytes": (sz, [vp]),
    "xfold_shard_ctx_set_overlap": (ci, [vp, ci, ci]),
    "xfold_pairformer_stack_sharded_fwd": (ci, [vp, vp, ci, vp, vp, vp, C.POINTER(PairformerWeights), ci, vp, sz, vp,
                                                C.POINTER(ci)]),
    "xfold_trimul_contract_planes_incoming_fwd": (ci, [vp, vp, vp, ci, ci, ci, ci, ci, vp, ci, vp]),
    "xfold_gated_attention_core_fwd": (ci, [vp, vp, ci, ci, ci, ci, ci, vp, vp, vp, vp, vp, ll, vp, vp, sz, vp]),
    "xfold_pair_bias_prepare_fwd": (ci, [vp, vp, ci, ci, vp, vp]),
    "xfold_attention_pair_bias_core_prepared_fwd": (ci, [vp, vp, ci, ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
    "xfold_cross_attention_workspace_bytes": (sz, [ci, ci, ci, ci, ci]),
    "xfold_cross_attention_fwd": (ci, [vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, vp, vp, vp, vp, vp, vp, vp, sz, vp]),
    "xfold_pairformer_f32_workspace_bytes": (sz, [ci]),
    "xfold_pairformer_stack_f32_fwd": (ci, [vp, vp, vp, vp, vp, ci, C.POINTER(PairformerWeightsF32), ci, vp, sz, vp]),
    "xfold_transition_static_max_bytes": (sz, []),
    "xfold_transition_static_fwd": (ci, [vp, vp, ll, ci, ci, C.POINTER(TransitionWeights), vp]),
    "xfold_pairformer_workspace_bytes": (sz, [ci]),
    "xfold_pairformer_block_fwd": (ci, [vp, vp, vp, vp, vp, ci, C.POINTER(PairformerWeights), vp, sz, vp]),
    "xfold_pairformer_stack_fwd": (ci, [vp, vp, vp, vp, vp, ci, C.POINTER(PairformerWeights), ci, vp, sz, vp]),
}

_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    """Loads the shared library (once) and sets the prototypes. Raises if it was not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python __graft_entry__.py` "
                          "(nvcc, sm_100a); this package has no CPU or eager fallback")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class XfoldError(RuntimeError):
    """Raised for a non-zero status of a C-ABI call (the reference's ops surface C++ exceptions
    as RuntimeError in the same way)."""


_ctxs = {}


def ctx(device: int) -> int:
    """Per-device context handle (created on first use; needs an sm_100 GPU)."""
    h = _ctxs.get(device)
    if h is None:
        lib = load()
        out = vp()
        rc = lib.xfold_ctx_create(device, C.byref(out))
        if rc != XFOLD_OK or not out.value:
            raise XfoldError(f"xfold_ctx_create(device={device}) failed with status {rc}: an sm_100 (B200) GPU "
                             "and a CUDA 12.x driver are required")
        h = out.value
        _ctxs[device] = h
    return h


def check(rc: int, device: int, what: str) -> None:
    if rc != XFOLD_OK:
        msg = load().xfold_last_error(_ctxs.get(device))
        raise XfoldError(f"{what}: status {rc}: {msg.decode() if msg else ''}")
