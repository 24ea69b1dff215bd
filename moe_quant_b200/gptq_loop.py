"""Drop-in for src.gptq_loop.gptq_loop (src/gptq_loop.py:193-225) on the CUDA sweep."""
from __future__ import annotations

import torch
from torch import Tensor

from . import ops


def gptq_loop(weight: Tensor, hessian_inv: Tensor, scale: Tensor, qzero: Tensor, maxq: Tensor, dtype: torch.dtype,
              gptq_block_size: int = 128) -> Tensor:
    """Same contract as the reference seam: `weight` is the TRANSPOSED weight (C, R) fp32 and
    is overwritten with the dequantized values; `scale`/`qzero` are (C, R) per-element grids;
    returns the codes as an fp32 (C, R) tensor.

    The kernels work on the (R, C) orientation, so this seam pays two transposes that
    GPTQ.quantize (which calls the fused entry point) never does.  The block size only
    changes the order of fp32 additions in the reference; the kernels always use 128-column
    tiles, so `gptq_block_size` is accepted and ignored.
    """
    C, R = weight.shape
    bits = int(round(float(torch.log2(maxq.float() + 1).item()))) if isinstance(maxq, Tensor) else int(maxq + 1).bit_length() - 1
    W = weight.t().contiguous().float()
    U = hessian_inv.contiguous().float()
    s = scale.contiguous().float()   # element (r, c) at c*R + r
    z = qzero.contiguous().float()
    codes, deq = ops.gptq_sweep(W, U, s, z, group=1, row_stride=1, group_stride=R, bits=bits,
                                dtype=dtype if dtype is not None else torch.float32, want_dequantized=True)
    weight.copy_(deq.t())
    return codes.t().float()
