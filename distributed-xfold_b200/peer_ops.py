"""ctypes wrappers of the peer-memory kernels (``xfold_transpose_scatter_fwd``, ``xfold_trimul_scatter_channels_fwd``,
``xfold_trimul_scatter_rows_fwd``, ``xfold_peer_barrier``)."""
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


def scatter_channels(a: torch.Tensor, b: torch.Tensor, n: int, row0: int, peer_a: List[int], peer_b: List[int]) -> None:
    """a, b [R, 128, ld] of this rank's rows -> the planes [128 / world, N, ld] of the rank that takes each channel."""
    assert a.is_cuda and a.dtype == torch.bfloat16 and a.is_contiguous() and b.is_contiguous() and a.shape == b.shape
    dev = a.device.index
    world = len(peer_a)
    pa, pb = (C.c_void_p * world)(*peer_a), (C.c_void_p * world)(*peer_b)
    rc = load().xfold_trimul_scatter_channels_fwd(ctx(dev), a.data_ptr(), b.data_ptr(), a.shape[0], n, a.shape[2], row0, pa, pb,
                                                  world, torch.cuda.current_stream(dev).cuda_stream)
    check(rc, dev, "xfold_trimul_scatter_channels_fwd")


def scatter_rows(o: torch.Tensor, chan0: int, peer_o: List[int], row_starts: List[int]) -> None:
    """o [channels, N, ldo] of this rank's channels -> [R_p, 128, ldo] on the rank p that owns each row."""
    assert o.is_cuda and o.dtype == torch.bfloat16 and o.is_contiguous()
    dev = o.device.index
    world = len(peer_o)
    po = (C.c_void_p * world)(*peer_o)
    starts = (C.c_int * (world + 1))(*row_starts)
    rc = load().xfold_trimul_scatter_rows_fwd(ctx(dev), o.data_ptr(), o.shape[0], chan0, o.shape[1], o.shape[2], po, starts,
                                              world, torch.cuda.current_stream(dev).cuda_stream)
    check(rc, dev, "xfold_trimul_scatter_rows_fwd")


def peer_allgather(src: torch.Tensor, offset_bytes: int, peer_dst: List[int]) -> None:
    """Copies this rank's contiguous block to byte offset ``offset_bytes`` of every rank's destination buffer."""
    assert src.is_cuda and src.is_contiguous()
    dev = src.device.index
    world = len(peer_dst)
    pd = (C.c_void_p * world)(*peer_dst)
    rc = load().xfold_peer_allgather_fwd(ctx(dev), src.data_ptr(), src.numel() * src.element_size(), offset_bytes, pd, world,
                                         torch.cuda.current_stream(dev).cuda_stream)
    check(rc, dev, "xfold_peer_allgather_fwd")
