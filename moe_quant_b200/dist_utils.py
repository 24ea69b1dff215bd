"""The torch.distributed wrappers that GPTQ and its driver call (src/dist_utils.py:20-65)."""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.distributed as dist
import torch.nn as nn


def is_dist_available_and_initialized() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_world_size() -> int:
    return dist.get_world_size() if is_dist_available_and_initialized() else 1


def get_rank() -> int:
    return dist.get_rank() if is_dist_available_and_initialized() else 0


def is_main() -> bool:
    return get_rank() == 0


def barrier(device_ids=None) -> None:
    if is_dist_available_and_initialized():
        dist.barrier(device_ids=device_ids)


def broadcast_parameters(module: nn.Module, src: Any = 0, group: Optional[Any] = None) -> None:
    for param in module.parameters():
        dist.broadcast(param.data, src=src, group=group)


def gather_into_tensor(tensor: torch.Tensor, dim: int = 0):
    world = get_world_size()
    out = chunks = None
    if is_main():
        shape = list(tensor.shape)
        shape[dim] *= world
        out = torch.empty(shape, device=tensor.device, dtype=tensor.dtype)
        chunks = list(out.chunk(world, dim=dim))
    dist.gather(tensor, chunks)
    return out


def print_on_main(*args, **kwargs) -> None:
    if is_main():
        print(*args, **kwargs)
