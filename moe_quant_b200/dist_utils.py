"""The torch.distributed queries that the GPTQ handle and the block loop use (src/dist_utils.py:20-41).
The reference module's parameter broadcast, gather and printing helpers serve its model-loading
driver, which is not part of this path."""
from __future__ import annotations

import torch.distributed as dist


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
