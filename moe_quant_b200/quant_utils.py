"""The helpers quant.py and GPTQ import from src.quant_utils, on the CUDA kernels
(src/quant_utils.py:57-101, 195-264).  Symmetric grids only: the reference's
asymmetric branch is broken (swapped min/max, src/quant_utils.py:91-99) and its
README supports 4-bit symmetric only."""
from __future__ import annotations

from enum import Enum
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import ops
from ._lib import MoeQuantError


class QuantizationScale(Enum):
    ABSMAX = "absmax"
    MSE = "mse"


def round_fp(x: Tensor, dtype: Optional[torch.dtype] = None) -> Tensor:
    return x if dtype is None else x.to(dtype).to(x.dtype)


def quantize(x: Tensor, scale: Tensor, qzero: Tensor, maxq: Tensor) -> Tensor:
    """Element-wise grid projection (src/quant_utils.py:61-62), torch ops on the tensors' device."""
    return (x / scale + qzero).round().clamp(torch.zeros_like(maxq), maxq)


def dequantize(qx: Tensor, scale: Tensor, qzero: Tensor, dtype: Optional[torch.dtype] = None) -> Tensor:
    return round_fp((qx - qzero) * scale, dtype)


def get_quantization_grid(weight: Tensor, group_size: int, bits: int, symmetric: bool = False,
                          dtype: Optional[torch.dtype] = None, quantization_scale="absmax",
                          **_unused) -> Tuple[Tensor, Tensor, Tensor]:
    """(scale, zero, maxq) replicated to the weight's shape like the reference
    (src/quant_utils.py:195-240).  GPTQ.quantize does not call this: the fused
    entry point never materialises the replicated tensors."""
    if not symmetric:
        raise MoeQuantError("only the symmetric grid is implemented")
    W = weight.float().contiguous()
    scale = ops.absmax_scales(W, group_size, bits, dtype if dtype is not None else torch.float32)
    # Like the reference, the search runs only for the Enum member: a plain string "mse" (what
    # GPTQ stores when quant.py passes its command-line value) compares unequal and gives absmax.
    if quantization_scale == QuantizationScale.MSE:
        ops.mse_scales(W, scale, group_size, bits, dtype if dtype is not None else torch.float32,
                       _unused.get("quant_max_shrink", 0.2), _unused.get("quant_n_grid", 100),
                       _unused.get("quant_norm", 2.4))
    maxq = torch.tensor(2 ** bits - 1, dtype=W.dtype, device=W.device)
    zero = torch.full_like(scale, (2 ** bits) / 2)
    return scale.repeat_interleave(group_size, dim=-1), zero.repeat_interleave(group_size, dim=-1), maxq


def dequantize_linear_weight(qweight: Tensor, scale: Tensor, zero: Tensor, perm: Optional[Tensor] = None) -> Tensor:
    """(q - zero) * scale per group, in the dtype of scale (src/quant_utils.py:243-256)."""
    R, C = qweight.shape
    G = scale.numel() // R
    out = ops.dequantize(qweight, scale.reshape(R, G), zero.reshape(R, G), C // G, 4, scale.dtype)
    if perm is not None:
        out = out[:, perm.argsort()]
    return out


def get_relative_mse_error(q: Tensor, w: Tensor, H: Optional[Tensor] = None) -> Tensor:
    """mean((q-w) H o (q-w)) / (mean(w H o w) + 1e-6) (src/quant_utils.py:259-264).  Both
    quadratic forms run on the engine (`mq_quadratic_form`); the result is an fp32 scalar on the
    device like the reference's."""
    delta = (q - w).float()
    if H is None:
        return delta.pow(2).mean() / w.pow(2).mean()
    n = float(w.numel())
    num = ops.quadratic_form(delta, H.float()) / n
    den = ops.quadratic_form(w.float(), H.float()) / n
    return (num / (den + 1e-6)).float()
