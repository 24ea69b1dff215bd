"""pack_weight / pack_to_int32 of pack_quantized_model.py:57-75 on the CUDA packer."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import ops
from ._lib import MoeQuantError


def pack_to_int32(value: Tensor, num_bits: int = 4, packed_dim: int = 1) -> Tensor:
    """compressed-tensors compatible packer for signed int8 values in [-8, 7] (R, C)."""
    if value.dtype is not torch.int8:
        raise ValueError("Tensor must be quantized to torch.int8 before packing")
    if num_bits != 4 or packed_dim != 1:
        raise MoeQuantError("only 4-bit packing along the input dimension is implemented")
    codes = (value + 8).to(torch.uint8)
    return ops.pack_int4(codes)


def pack_weight(weight: dict, bits: int, sym: bool, group_size: Optional[int] = None) -> dict:
    """{'qweight','scale','zero'} -> {'weight_packed','weight_shape','weight_scale'[, 'weight_zero_point']}.

    The reference runs this on CPU tensors loaded from quantized_weight.pt
    (pack_quantized_model.py:186-191); here the codes are moved to the current CUDA
    device if needed, packed there, and the words returned on the input's device.
    """
    if bits != 4:
        raise MoeQuantError("only 4-bit packing is implemented")
    q, scale, zero = weight["qweight"], weight["scale"], weight["zero"]
    g = group_size or q.shape[-1]
    home = q.device
    dev = home if q.is_cuda else torch.device("cuda", torch.cuda.current_device())
    qd = q.to(dev)
    if sym:
        packed = ops.pack_int4(qd)
    else:
        packed = ops.pack_int4(qd, zero.to(dev).to(torch.int8), g)
    out = {
        "weight_packed": packed.to(home),
        "weight_shape": torch.tensor(q.shape),
        "weight_scale": scale,
    }
    if not sym:
        out["weight_zero_point"] = zero
    return out
