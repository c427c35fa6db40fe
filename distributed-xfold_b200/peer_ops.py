"""ctypes wrappers of the peer-memory kernels (``xfold_transpose_scatter_fwd``, ``xfold_peer_barrier``)."""
from __future__ import annotations

import ctypes as C
from typing import List

import torch

from ._cabi import check, ctx, load


def transpose_scatter(z: torch.Tensor, row0: int, peer_ptrs: List[int], col_starts: List[int]) -> None:
    """Stores every token z[i, j, :] of this rank's rows into the buffer of the rank owning column j."""
    assert z.is_cuda and z.dtype == torch.bfloat16 and z.is_contiguous() and z.shape[-1] == 128
    dev = z.device.index
    world = len(peer_ptrs)
    ptrs = (C.c_void_p * world)(*peer_ptrs)
    starts = (C.c_int * (world + 1))(*col_starts)
    rc = load().xfold_transpose_scatter_fwd(ctx(dev), z.data_ptr(), z.shape[0], z.shape[1], row0, ptrs, starts, world,
                                            torch.cuda.current_stream(dev).cuda_stream)
    check(rc, dev, "xfold_transpose_scatter_fwd")


def peer_barrier(flag_ptrs: List[int], me: int, world: int, epoch: int, device) -> None:
    dev = torch.device(device).index
    ptrs = (C.c_void_p * world)(*flag_ptrs)
    rc = load().xfold_peer_barrier(ctx(dev), ptrs, me, world, epoch, torch.cuda.current_stream(dev).cuda_stream)
    check(rc, dev, "xfold_peer_barrier")
