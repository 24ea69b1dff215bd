"""CPU restatement of the MoE-Quant GPTQ hot path.  TEST INFRASTRUCTURE ONLY.

This module is the checker that the CUDA path is compared against.  Nothing in
the product package imports it; only the test-suite, the smoke entry and the
CPU-baseline leg of the benchmark do.

Every function names the reference lines it restates (paths are relative to the
MoE-Quant project root).  The restatement is plain torch on CPU tensors in
fp32, so it follows the reference's own arithmetic type.

Parity status
-------------
* Hessian update, pre-step, grid, Hessian inverse, the tail of ``_quantize``,
  ``dequantize_linear_weight``, ``get_relative_mse_error`` and ``pack_weight``
  are PINNED: the golden fixtures under ``tests/golden`` were produced by the
  reference's own code imported unchanged (``tests/golden/make_golden.py``).
* The column sweep (``src/gptq_loop.py:141-148``) is Triton-only in the
  reference and cannot execute without a GPU.  It is PINNED by
  ``tests/golden/sweep_triton.npz``: codes produced on a B200 by the reference's
  own ``gptq_loop`` (Triton kernels + ``addmm_``) and by its whole ``GPTQ`` handle,
  imported unchanged (``tests/golden/make_golden_sweep_gpu.py``).  The sweep
  restated here reproduces them (``tests/test_triton_pin.py``).  The codes inside
  the CPU fixtures of ``make_golden.py`` come from this restatement patched into
  the reference's pipeline; the device run showed them identical to the Triton
  loop's on every fixture.
* ``compressed_tensors.pack_to_int32`` (third-party, unpinned by the reference;
  0.15.0.1 here) is restated in :func:`pack_to_int32`; the fixtures hold the
  installed library's words.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import Tensor

EPS = 1e-12  # src/quant_utils.py:88


# ----------------------------------------------------------------------------
# Hessian accumulation                                     src/gptq.py:74-105
# ----------------------------------------------------------------------------
def hessian_update(H: Optional[Tensor], n_seen: int, x: Tensor) -> Tuple[Tensor, int]:
    """Running mean ``H <- n/(n+m) H + 2/(n+m) X^T X`` in fp32 (src/gptq.py:97-105)."""
    x = x.reshape(-1, x.shape[-1]).float()
    m = x.shape[0]
    if H is None:
        H = torch.zeros(x.shape[1], x.shape[1], dtype=torch.float32)
    beta = n_seen / (n_seen + m)
    alpha = 2.0 / (n_seen + m)
    H.addmm_(x.T, x, beta=beta, alpha=alpha)
    return H, n_seen + m


# ----------------------------------------------------------------------------
# pre-step                                                src/gptq.py:122-154
# ----------------------------------------------------------------------------
def pre_step(H: Optional[Tensor], weight: Tensor):
    """Returns (H, W_fp32, issue_zero_samples, issue_nan).  src/gptq.py:127-152."""
    d_col = weight.shape[1]
    zero_samples = nan = False
    if H is None:
        H = torch.eye(d_col, dtype=torch.float32)
        zero_samples = True
    if torch.isnan(H).any().item():
        H = torch.eye(d_col, dtype=torch.float32)
        nan = True
    dead = torch.diag(H) == 0
    H[dead, dead] = 1
    W = weight.clone().float()
    W[:, dead] = 0
    return H, W, zero_samples, nan


# ----------------------------------------------------------------------------
# grid                                  src/quant_utils.py:75-101 and 195-240
# ----------------------------------------------------------------------------
def round_fp(x: Tensor, dtype: Optional[torch.dtype]) -> Tensor:
    """Round through the layer dtype, RTNE (src/quant_utils.py:57-58)."""
    return x if dtype is None else x.to(dtype).to(x.dtype)


def symmetric_grid(W: Tensor, group_size: int, bits: int, dtype: Optional[torch.dtype]):
    """Per (row, group) absmax scale, zero = (maxq+1)/2.  Returns the
    de-replicated (R, G) fp32 scale and zero plus python maxq.

    src/quant_utils.py:89-97: scale = round_fp((2/maxq) * max(|amax|,|amin|) + 1e-12).
    The reference then replicates to (R, C) (``:234-235``); the replication
    carries no information and is left to the caller.
    """
    R, C = W.shape
    maxq = torch.tensor(2 ** bits - 1, dtype=W.dtype)
    wg = W.unflatten(-1, (-1, group_size))
    hi = wg.amax(dim=-1)
    lo = wg.amin(dim=-1)
    scale = (2.0 / maxq) * torch.maximum(hi.abs(), lo.abs())
    scale = round_fp(scale + EPS, dtype)
    zero = torch.full_like(scale, ((maxq + 1.0) * 0.5).item())
    return scale, zero, float(maxq)


def mse_scale(Wg: Tensor, scale: Tensor, zero: Tensor, maxq: float, dtype: Optional[torch.dtype],
              max_shrink: float = 0.2, n_grid: int = 100, norm: float = 2.4) -> Tensor:
    """Shrink-factor search of ``mse_scale_triton_kernel`` (src/quant_utils.py:104-139) with the
    candidates of ``get_quantization_grid`` (``:219``).  Wg (R, G, g) fp32; scale, zero (R, G).

    Per candidate p_i: s_i = round_fp(scale * p_i); the group is quantized with the Triton
    rounding (floor(x/s + z + 0.5), ``:30-34``) and dequantized through the dtype; the loss is
    sum |q - x|^norm with the power taken as exp(norm * log|.|) (``tl_pow``, ``:25-27``); the scale
    becomes round_fp(scale * p_argmin).  The reference pads the candidate axis to 128 with an
    unmasked load of unspecified values; only the real candidates are searched here."""
    p = torch.linspace(1, max_shrink, n_grid, dtype=Wg.dtype)
    best = torch.full_like(scale, float("inf"))
    best_i = torch.zeros_like(scale, dtype=torch.long)
    for i in range(n_grid):
        s = round_fp(scale * p[i], dtype)[..., None]
        q = torch.clamp(torch.floor((Wg / s + zero[..., None]) + 0.5), 0.0, maxq)
        y = round_fp((q - zero[..., None]) * s, dtype)
        loss = ((y - Wg).abs().log() * norm).exp().sum(-1)
        better = loss < best
        best = torch.where(better, loss, best)
        best_i = torch.where(better, torch.full_like(best_i, i), best_i)
    return round_fp(scale * p[best_i], dtype)


# ----------------------------------------------------------------------------
# Hessian inverse              src/gptq.py:220-243, src/linalg_utils.py:8-12
# ----------------------------------------------------------------------------
def hessian_inverse(H: Tensor, W: Tensor, rel_damp: float):
    """Masks all-zero weight columns, damps, and returns the row-normalised upper
    Cholesky factor of H^-1 (mutating H like the reference), plus a flag telling
    whether the factorisation failed (the reference silently substitutes I)."""
    d_col = H.shape[0]
    zero_cols = torch.nonzero(W.eq(0).all(dim=0))
    H[zero_cols, :] = 0
    H[:, zero_cols] = 0
    H[zero_cols, zero_cols] = 1
    damp = rel_damp * torch.diag(H).mean()
    H[range(d_col), range(d_col)] += damp
    failed = False
    try:
        Hinv = torch.cholesky_inverse(torch.linalg.cholesky(H))
        U = torch.linalg.cholesky(Hinv, upper=True)
    except Exception:  # noqa: BLE001 - the reference uses a bare except (src/gptq.py:239)
        U = torch.eye(d_col, dtype=torch.float32)
        failed = True
    U = U.div(U.diag()[:, None]).contiguous()
    return U, failed


# ----------------------------------------------------------------------------
# column sweep                                        src/gptq_loop.py:141-148
# ----------------------------------------------------------------------------
def _quantize_col(x: Tensor, scale: Tensor, zero: Tensor, maxq: float) -> Tensor:
    """clamp(floor(x/scale + zero + 0.5), 0, maxq): src/quant_utils.py:30-34,43-44."""
    return torch.clamp(torch.floor((x / scale + zero) + 0.5), 0.0, maxq)


def _fma(a: Tensor, b: Tensor, c: Tensor) -> Tensor:
    """Single-rounding a*b+c as tl.fma does (src/gptq_loop.py:85): the product of two
    fp32 numbers is exact in fp64, so one fp64 add followed by a cast is an FMA up
    to measure-zero double-rounding cases."""
    return (a.double() * b.double() + c.double()).float()


def gptq_sweep(
    Wt: Tensor,
    Uhat: Tensor,
    scale_t: Tensor,
    zero_t: Tensor,
    maxq: float,
    dtype: Optional[torch.dtype],
    block: int = 128,
):
    """The body captured by the reference's CUDA graph (src/gptq_loop.py:141-148).

    Wt (C, R) fp32 is mutated in place (ends up holding the dequantized values),
    Uhat (C, C) row-normalised upper factor, scale_t/zero_t (C, R) fp32.
    Returns codes (C, R) fp32 with integer values 0..maxq.

    Per column j: quantize_error_triton_kernel (``:28-40``) then the rank-1
    ``addvv`` (``:83-88``) on the rest of the block; per block: ``addmm_`` on every
    later column (``:148``).
    """
    C, R = Wt.shape
    if block <= 0:
        block = C
    Q = torch.empty_like(Wt)
    err = torch.empty(block, R, dtype=Wt.dtype)
    for i1 in range(0, C, block):
        i2 = min(i1 + block, C)
        for j in range(i1, i2):
            x = Wt[j]
            q = _quantize_col(x, scale_t[j], zero_t[j], maxq)
            y = round_fp((q - zero_t[j]) * scale_t[j], dtype)
            e = y - x
            Wt[j] = y
            Q[j] = q
            err[j - i1] = e
            if j + 1 < i2:
                Wt[j + 1:i2] = _fma(Uhat[j, j + 1:i2, None], e[None, :], Wt[j + 1:i2])
        if i2 < C:
            Wt[i2:].addmm_(Uhat[i1:i2, i2:].t(), err[: i2 - i1], beta=1, alpha=1)
    return Q


# ----------------------------------------------------------------------------
# whole layer                                             src/gptq.py:156-218
# ----------------------------------------------------------------------------
def quantize_layer(
    weight: Tensor,
    H: Optional[Tensor],
    *,
    bits: int = 4,
    group_size: Optional[int] = None,
    rel_damp: float = 1e-2,
    block_size: Optional[int] = None,
    act_order: bool = False,
    mse: bool = False,
):
    """``GPTQ.quantize(bits)`` for a symmetric, non-distributed, untied handle.

    Returns dict(qweight uint8 (R,C), scale (R,G) layer dtype, zero (R,G) layer
    dtype, H (the damped Hessian, mutated as in the reference), Uhat, flags).
    """
    dtype = weight.dtype
    R, C = weight.shape
    g = group_size or C
    block = block_size or C
    H, W, zero_samples, nan = pre_step(H, weight)
    scale, zero, maxq = symmetric_grid(W, g, bits, dtype)
    if mse:
        scale = mse_scale(W.unflatten(-1, (-1, g)), scale, zero, maxq, dtype)
    if act_order:
        perm = torch.argsort(H.diag(), descending=True)
    else:
        perm = torch.arange(C)
    perm_inv = torch.argsort(perm)
    H = H[perm][:, perm]
    Uhat, failed = hessian_inverse(H, W, rel_damp)
    scale_full = scale.repeat_interleave(g, dim=-1)
    zero_full = zero.repeat_interleave(g, dim=-1)
    Wt = W.t()[perm].contiguous()
    Q = gptq_sweep(
        Wt, Uhat, scale_full.t()[perm].contiguous(), zero_full.t()[perm].contiguous(), maxq, dtype, block
    )
    qweight = Q[perm_inv].t().contiguous().to(torch.uint8)
    return {
        "qweight": qweight,
        "scale": scale.to(dtype),
        "zero": zero.to(dtype),
        "H": H,
        "Uhat": Uhat,
        "issue_zero_samples": zero_samples,
        "issue_nan_hessian": nan,
        "issue_non_invertible": failed,
    }


# ----------------------------------------------------------------------------
# consumers                               src/quant_utils.py:65-66 and 243-264
# ----------------------------------------------------------------------------
def dequantize_linear_weight(qweight: Tensor, scale: Tensor, zero: Tensor) -> Tensor:
    R = qweight.shape[0]
    s = scale.view(R, -1, 1)
    z = zero.view(R, -1, 1)
    G = s.shape[1]
    return ((qweight.view(R, G, -1) - z) * s).view_as(qweight)


def relative_mse_error(q: Tensor, w: Tensor, H: Optional[Tensor] = None) -> Tensor:
    d = q - w
    if H is None:
        return d.pow(2).mean() / w.pow(2).mean()
    return d.mm(H).mul(d).mean() / (w.mm(H).mul(w).mean() + 1e-6)


# ----------------------------------------------------------------------------
# packing       pack_quantized_model.py:57-75 -> compressed_tensors pack_to_int32
# ----------------------------------------------------------------------------
def pack_to_int32(value: Tensor, num_bits: int = 4) -> Tensor:
    """Published algorithm of compressed-tensors' ``pack_to_int32`` with
    ``packed_dim=1``: add 2^(bits-1), zero-pad the row to a multiple of
    32/bits entries, and put entry i of every run of 32/bits at bit i*bits."""
    assert value.dtype is torch.int8 and value.ndim == 2
    per = 32 // num_bits
    u = (value + (1 << (num_bits - 1))).to(torch.uint8)
    R, C = u.shape
    pad = math.ceil(C / per) * per - C
    if pad:
        u = torch.nn.functional.pad(u, (0, pad))
    u = u.view(R, -1, per).to(torch.int64)
    shifts = torch.arange(per, dtype=torch.int64) * num_bits
    words = (u << shifts).sum(dim=2)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)  # wrap like int32 arithmetic
    return words.to(torch.int32)


def pack_weight(weight: dict, bits: int, sym: bool, group_size: Optional[int] = None) -> dict:
    """pack_quantized_model.py:57-75."""
    q, scale, zero = weight["qweight"], weight["scale"], weight["zero"]
    g = group_size or q.shape[-1]
    shifted = q.to(torch.int8) - zero.repeat_interleave(g, dim=-1).to(torch.int8)
    out = {
        "weight_packed": pack_to_int32(shifted, bits),
        "weight_shape": torch.tensor(q.shape),
        "weight_scale": scale,
    }
    if not sym:
        out["weight_zero_point"] = zero
    return out


# ----------------------------------------------------------------------------
# parity metrics used by the tests and the benchmark
# ----------------------------------------------------------------------------
def reconstruction_error(W: Tensor, Wq: Tensor, H_raw: Tensor) -> float:
    """||WX - QX||^2 / ||WX||^2 expressed through the undamped H = (2/N) X^T X."""
    d = (Wq - W).double()
    Hd = H_raw.double()
    Wd = W.double()
    return float((d @ Hd).mul(d).sum() / (Wd @ Hd).mul(Wd).sum())


def code_agreement(a: Tensor, b: Tensor) -> float:
    return float((a == b).double().mean())
