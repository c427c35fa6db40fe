"""Process-grid and sharding helpers with the reference's names and meanings
(src/distributed_xfold/distribute_utils.py): ``DeviceMesh``, ``init_dist_info``, ``ShardInfo``,
``shard_linear``, ``all_gather_into_tensor``, ``all_to_all``, ``setup_gloo``.

One process drives one GPU; ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests) is the
plumbing.  Collectives that the kernels do not fuse go through the two helpers at the bottom.
"""
from __future__ import annotations

import math
import os
import socket
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn


def find_free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def setup_gloo(rank: int, world_size: int, port: int) -> None:
    """Single-node gloo rendezvous on 127.0.0.1 (reference: distribute_utils.py:38-45)."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world_size)


def setup_dist_env(backend: Optional[str] = None) -> None:
    """env:// rendezvous as launched by torchrun; NCCL when a GPU is present, else gloo."""
    if dist.is_initialized():
        return
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group(backend)


def cleanup() -> None:
    if dist.is_initialized():
        dist.destroy_process_group()


class DeviceMesh:
    """Ranks 0..world-1 laid out row-major as a [dp, tp] grid (reference :53-81).  In the trunk
    'dp' is the pair-row shard axis and tp is 1."""

    def __init__(self, world_size: int, dp_size: int = 1, tp_size: int = 1):
        if dp_size * tp_size != world_size:
            raise ValueError(f"dp_size * tp_size ({dp_size} * {tp_size}) must equal world_size ({world_size})")
        self.world_size, self.dp_size, self.tp_size = world_size, dp_size, tp_size
        self.device_mesh = torch.arange(world_size, dtype=torch.long).reshape(dp_size, tp_size)
        self._groups = {}

    def get_rank_coords(self, rank: int) -> torch.Tensor:
        return (self.device_mesh == rank).nonzero()

    def _coords(self, rank: int):
        return divmod(int(rank), self.tp_size)

    def _group(self, ranks: List[int]):
        key = tuple(ranks)
        if key not in self._groups:
            self._groups[key] = dist.new_group(list(ranks))
        return self._groups[key]

    def get_dp_group(self, rank: int):
        return self._group(self.device_mesh[:, self._coords(rank)[1]].tolist())

    def get_tp_group(self, rank: int):
        return self._group(self.device_mesh[self._coords(rank)[0]].tolist())

    def get_dp_shard_num(self, rank: int) -> int:
        return self._coords(rank)[0]

    def get_tp_shard_num(self, rank: int) -> int:
        return self._coords(rank)[1]

    def get_all_device(self):
        return self._group(self.device_mesh.flatten().tolist())


def init_dist_info(module, device_mesh: DeviceMesh) -> None:
    """Sets the attributes every ``Distribute*`` module carries (reference :83-99)."""
    module.device_mesh = device_mesh
    module.dp_size, module.tp_size = device_mesh.dp_size, device_mesh.tp_size
    module.use_dp, module.use_tp = device_mesh.dp_size > 1, device_mesh.tp_size > 1
    if dist.is_initialized():
        module.rank = dist.get_rank()
        module.dp_shard_group = device_mesh.get_dp_group(module.rank)
        module.tp_shard_group = device_mesh.get_tp_group(module.rank)
    else:
        module.rank = 0
        module.dp_shard_group = module.tp_shard_group = None
    module.dp_shard_num = device_mesh.get_dp_shard_num(module.rank)
    module.tp_shard_num = device_mesh.get_tp_shard_num(module.rank)


class ShardInfo:
    """Row partition: ceil(size / shards) per shard, the last one takes what is left
    (reference :101-128; 764 rows over 8 ranks -> 7 x 96 + 92)."""

    def __init__(self, tensor_size: int, num_shard: int):
        if num_shard > tensor_size:
            raise ValueError("more shards than rows")
        self.tensor_size, self.num_shard = tensor_size, num_shard
        if tensor_size % num_shard:
            self.per_chunk_size = math.ceil(tensor_size / num_shard)
            self.remain_chunk_size = tensor_size % self.per_chunk_size
            self.shard_size_list = [self.per_chunk_size] * (num_shard - 1) + [self.remain_chunk_size]
        else:
            self.per_chunk_size = tensor_size // num_shard
            self.remain_chunk_size = 0
            self.shard_size_list = [self.per_chunk_size] * num_shard
        starts = [0]
        for sz in self.shard_size_list:
            starts.append(starts[-1] + sz)
        self.shard_slice_list = [slice(starts[i], starts[i + 1]) for i in range(num_shard)]

    def get_shard_size_list(self): return self.shard_size_list
    def get_shard_slice_list(self): return self.shard_slice_list
    def get_per_chunk_size(self): return self.per_chunk_size
    def get_remain_chunk_size(self): return self.remain_chunk_size
    def get_num_shard(self): return self.num_shard
    def get_tensor_size(self): return self.tensor_size


def shard_linear(fnn: nn.Linear, rank: int, device_mesh: DeviceMesh, out: bool = True) -> nn.Linear:
    """Column-parallel (``out=True``: contiguous chunk of output rows, bias chunked with it) or
    row-parallel (``out=False``: chunk of input columns, full bias) slice of a Linear for this
    rank's tp coordinate (reference :130-206)."""
    if not isinstance(fnn, nn.Linear):
        raise TypeError("Input 'fnn' must be a torch.nn.Linear layer.")
    tp, tp_rank = device_mesh.tp_size, device_mesh.get_tp_shard_num(rank)
    w, b = fnn.weight, fnn.bias
    if out:
        if fnn.out_features % tp:
            raise ValueError(f"Output dimension ({fnn.out_features}) not divisible by TP size ({tp})")
        w = w.chunk(tp, dim=0)[tp_rank]
        b = None if b is None else b.chunk(tp, dim=0)[tp_rank]
    else:
        if fnn.in_features % tp:
            raise ValueError(f"Input dimension ({fnn.in_features}) not divisible by TP size ({tp})")
        w = w.chunk(tp, dim=1)[tp_rank]
    new = nn.Linear(w.shape[1], w.shape[0], bias=b is not None, dtype=w.dtype, device=w.device)
    new.weight = nn.Parameter(w.detach().clone())
    if b is not None:
        new.bias = nn.Parameter(b.detach().clone())
    return new


def all_gather_into_tensor(output_tensor: torch.Tensor, input_tensor: torch.Tensor, group=None,
                           async_op: bool = False, shard_dim: Optional[int] = None):
    """Gathers the ranks' shards along the one dim in which ``output_tensor`` and ``input_tensor``
    differ (reference :229-262).  Shards may be ragged in that dim (ShardInfo's short last shard):
    they are padded to the largest for the collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    x = input_tensor.contiguous()
    if shard_dim is None:
        diff = [d for d in range(x.dim()) if output_tensor.shape[d] != x.shape[d]]
        if len(diff) > 1:
            raise ValueError("Could not determine shard dimension")
        shard_dim = diff[0] if diff else 0
    sizes = ShardInfo(output_tensor.shape[shard_dim], world).shard_size_list if world > 1 else [x.shape[shard_dim]]
    if async_op:
        bufs = [torch.empty_like(x) for _ in range(world)]
        return bufs, dist.all_gather(bufs, x, group=group, async_op=True)
    biggest = max(sizes)
    if x.shape[shard_dim] < biggest:
        pad_shape = list(x.shape)
        pad_shape[shard_dim] = biggest - x.shape[shard_dim]
        x = torch.cat([x, x.new_zeros(pad_shape)], shard_dim)
    bufs = [torch.empty_like(x) for _ in range(world)]
    dist.all_gather(bufs, x, group=group)
    torch.cat([b.narrow(shard_dim, 0, sz) for b, sz in zip(bufs, sizes)], dim=shard_dim, out=output_tensor)
    return output_tensor


def all_to_all(input_tensor: torch.Tensor, shard_dim: int, unshard_dim: int, group=None, async_op: bool = False):
    """Re-shards: splits ``shard_dim`` across the ranks and concatenates what arrives along
    ``unshard_dim`` (reference :209-227, equal chunks)."""
    world = dist.get_world_size(group)
    send = [c.contiguous() for c in torch.chunk(input_tensor, world, dim=shard_dim)]
    recv = [torch.empty_like(send[0]) for _ in range(world)]
    work = dist.all_to_all(recv, send, group=group, async_op=async_op)
    if async_op:
        return work
    return torch.cat(recv, dim=unshard_dim)
