"""Shared plumbing of the module classes: update-returning calls into the C ABI."""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from .. import ops
from .._cabi import check, ctx, load

BF16 = torch.bfloat16


def _as_bf16(x: torch.Tensor) -> torch.Tensor:
    ops._need_cuda(x)
    return x.to(BF16).contiguous()


def _mask(m: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    return None if m is None else m.to(torch.float32).contiguous()


def trimul_update(pair: torch.Tensor, mask, w: ops.PackedTriMul, outgoing: bool) -> torch.Tensor:
    z = _as_bf16(pair)
    dev = ops._dev(z)
    n = z.shape[0]
    lib = load()
    ws = ops._Workspace.get(dev, lib.xfold_trimul_workspace_bytes(n))
    out = torch.empty_like(z)
    m = _mask(mask)
    rc = lib.xfold_triangle_multiplication_update_fwd(ctx(dev), z.data_ptr(), out.data_ptr(), ops._ptr(m), n, int(outgoing),
                                                      C.byref(w.c), ws.data_ptr(), ws.numel(), ops._stream(dev))
    check(rc, dev, "xfold_triangle_multiplication_update_fwd")
    return out.to(pair.dtype)


def triattn_update(pair: torch.Tensor, mask, w: ops.PackedTriAttn, transpose: bool) -> torch.Tensor:
    z = _as_bf16(pair)
    dev = ops._dev(z)
    n = z.shape[0]
    lib = load()
    ws = ops._Workspace.get(dev, lib.xfold_triattn_workspace_bytes(n))
    out = torch.empty_like(z)
    m = _mask(mask)
    rc = lib.xfold_triangle_attention_update_fwd(ctx(dev), z.data_ptr(), out.data_ptr(), ops._ptr(m), n, int(transpose),
                                                 C.byref(w.c), ws.data_ptr(), ws.numel(), ops._stream(dev))
    check(rc, dev, "xfold_triangle_attention_update_fwd")
    return out.to(pair.dtype)


def transition_update(x: torch.Tensor, w: ops.PackedTransition) -> torch.Tensor:
    xb = _as_bf16(x)
    dev = ops._dev(xb)
    rows = xb.numel() // w.C
    lib = load()
    ws = ops._Workspace.get(dev, lib.xfold_transition_workspace_bytes(rows, w.C, w.F))
    out = torch.empty_like(xb)
    rc = lib.xfold_transition_update_fwd(ctx(dev), xb.data_ptr(), out.data_ptr(), rows, w.C, w.F, C.byref(w.c),
                                         ws.data_ptr(), ws.numel(), ops._stream(dev))
    check(rc, dev, "xfold_transition_update_fwd")
    return out.to(x.dtype)
