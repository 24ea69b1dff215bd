"""Replacement for src/linalg_utils.py on top of the CUDA factorisation kernels."""
from __future__ import annotations

import torch
from torch import Tensor

from . import ops

__all__ = ["inv_sym", "hessian_inverse_factor"]


def hessian_inverse_factor(H: Tensor, precision=None):
    """Row-normalised upper Cholesky factor of H^-1 (what GPTQ._get_hessian_inverse returns,
    src/gptq.py:236-243) for an H that is already masked and damped.  H is left intact.
    Returns (Uhat, flags)."""
    U, flags, _ = ops.hinv_upper(H.clone(), precision)
    return U, flags


def inv_sym(X: Tensor, precision=None) -> Tensor:
    """Inverse of a symmetric positive-definite matrix (src/linalg_utils.py:8-12).

    The engine never needs H^-1 itself; this seam rebuilds it from the factor:
    X = T T^T,  Uhat = diag(T) T^-1  =>  X^-1 = Uhat^T diag(T)^-2 Uhat.
    """
    U, _, d = ops.hinv_upper(X.clone().float(), precision, want_diag=True)
    V = U / d[:, None]
    return torch.mm(V.t(), V)
