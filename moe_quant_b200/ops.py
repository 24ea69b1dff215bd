"""Tensor-level wrappers over the C ABI: one function per entry point of
include/moequant.h.  They validate devices/dtypes, size the workspace and pass
raw pointers plus the current CUDA stream.  No arithmetic happens here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import ctypes
import torch
from torch import Tensor

from . import _lib
from ._lib import MATH_COMPACT, MATH_FP32, MATH_TENSOR, MoeQuantError, check, dtype_code, lib, ptr, require_cuda, stream_ptr


@dataclass
class Precision:
    """Arithmetic of the dense contractions.

    math: MATH_TENSOR (tcgen05, fp32 accumulation in TMEM) or MATH_FP32 (CUDA cores).
    split_*: number of bf16 planes an fp32 operand is cut into on the tensor path
    (1, 2 or 3 planes -> 1, 3 or 6 products).  bf16/fp16 activations always enter the
    Hessian exactly with one product.
    compact: several layers are in flight on different streams (quantize_many sets it): the sweep
    uses launch shapes that occupy few SMs (MQ_MATH_COMPACT); the results do not change.
    """

    math: int = MATH_TENSOR
    split_hessian: int = 3
    split_hinv: int = 3
    split_sweep: int = 3
    compact: bool = False

    @property
    def sweep_math(self) -> int:
        """The `math` argument of the sweep and of the whole-layer entry point."""
        return self.math | (MATH_COMPACT if self.compact else 0)


DEFAULT_PRECISION = Precision()


def set_default_precision(p: Precision) -> None:
    global DEFAULT_PRECISION
    DEFAULT_PRECISION = p


def _prec(p: Optional[Precision]) -> Precision:
    return DEFAULT_PRECISION if p is None else p


def _flags_tensor(device) -> Tensor:
    return torch.zeros(4, dtype=torch.int32, device=device)


def hessian_accum(H: Tensor, x: Tensor, beta: float, alpha: float, precision: Optional[Precision] = None) -> None:
    """H <- beta*H + alpha*x^T x in place.  x is (m, C) fp32/bf16/fp16, H (C, C) fp32."""
    p = _prec(precision)
    require_cuda(H, "H")
    require_cuda(x, "x")
    if H.dtype != torch.float32 or H.dim() != 2 or H.shape[0] != H.shape[1] or H.stride(1) != 1:
        raise MoeQuantError("H must be a square fp32 matrix with unit column stride")
    if x.dim() != 2 or x.shape[1] != H.shape[0]:
        raise MoeQuantError(f"x of shape {tuple(x.shape)} does not match H of shape {tuple(H.shape)}")
    if x.stride(1) != 1 and x.shape[0] > 0:
        x = x.contiguous()
    m, C = x.shape
    code = dtype_code(x.dtype)
    L = lib()
    nbytes = L.mq_hessian_accum_workspace_bytes(code, m, C, p.math, p.split_hessian)
    ws = _lib.workspace(H.device, nbytes)
    with torch.cuda.device(H.device):
        check(L.mq_hessian_accum(ptr(x) if m else None, code, m, C, x.stride(0) if m else C, ptr(H), H.stride(0),
                                 beta, alpha, p.math, p.split_hessian, ptr(ws), ws.numel(), stream_ptr(H.device)))


def gemm(A: Tensor, B: Tensor, C: Tensor, alpha: float = 1.0, beta: float = 0.0, upper_tiles_only: bool = False,
         precision: Optional[Precision] = None, split: Optional[int] = None) -> None:
    """C <- alpha * A @ B + beta * C in place.  A (M,K), B (K,N) fp32 with any strides (views and
    transposes are fine), C (M,N) fp32 with unit column stride."""
    p = _prec(precision)
    for t, n in ((A, "A"), (B, "B"), (C, "C")):
        require_cuda(t, n)
        if t.dtype != torch.float32 or t.dim() != 2:
            raise MoeQuantError(f"{n} must be a 2-D fp32 tensor")
    M, K = A.shape
    K2, N = B.shape
    if K2 != K or C.shape != (M, N) or C.stride(1) != 1:
        raise MoeQuantError("gemm: shape mismatch")
    sp = p.split_hinv if split is None else split
    L = lib()
    ws = _lib.workspace(C.device, L.mq_gemm_workspace_bytes(M, N, K, p.math, sp))
    with torch.cuda.device(C.device):
        check(L.mq_gemm(ptr(A), A.stride(0), A.stride(1), ptr(B), B.stride(0), B.stride(1), ptr(C), C.stride(0), M, N, K,
                        alpha, beta, int(upper_tiles_only), p.math, sp, ptr(ws), ws.numel(), stream_ptr(C.device)))


def hessian_prepare(H: Tensor, W: Optional[Tensor], rel_damp: float) -> Tensor:
    """In-place NaN guard, dead-channel fix, zero-column masking and damping.
    Returns the int32[4] flag tensor (nan, dead, zero columns, not-positive)."""
    require_cuda(H, "H")
    C = H.shape[0]
    L = lib()
    flags = _flags_tensor(H.device)
    nbytes = L.mq_hessian_prepare_workspace_bytes(C)
    ws = _lib.workspace(H.device, nbytes)
    if W is not None:
        require_cuda(W, "W")
        if W.dtype != torch.float32 or W.stride(1) != 1:
            raise MoeQuantError("W must be the fp32 working copy with unit column stride")
    with torch.cuda.device(H.device):
        check(L.mq_hessian_prepare(ptr(H), C, H.stride(0), ptr(W), 0 if W is None else W.shape[0],
                                   0 if W is None else W.stride(0), rel_damp, ptr(flags), ptr(ws), ws.numel(),
                                   stream_ptr(H.device)))
    return flags


def hessian_prepare_noalloc(H: Tensor, W: Optional[Tensor], rel_damp: float, flags: Tensor) -> None:
    """hessian_prepare for hosts that cannot provide scratch: the channel lists live in a static
    array inside the library (C <= 32768).  Even the 16-byte flag word is the caller's (`flags`,
    int32[4] on H's device), so this call allocates nothing at all.  Calls on one device must
    not overlap on the GPU: they share the array."""
    require_cuda(H, "H")
    require_cuda(flags, "flags")
    with torch.cuda.device(H.device):
        check(lib().mq_hessian_prepare_noalloc(ptr(H), H.shape[0], H.stride(0), ptr(W), 0 if W is None else W.shape[0],
                                               0 if W is None else W.stride(0), rel_damp, ptr(flags),
                                               stream_ptr(H.device)))


def hinv_upper(H: Tensor, precision: Optional[Precision] = None, flags: Optional[Tensor] = None,
               want_diag: bool = False) -> Tuple[Tensor, Tensor, Optional[Tensor]]:
    """Row-normalised upper Cholesky factor of H^-1.  H (damped) is DESTROYED.
    Returns (Uhat, flags, diag(T) or None)."""
    p = _prec(precision)
    require_cuda(H, "H")
    C = H.shape[0]
    L = lib()
    U = torch.empty(C, C, dtype=torch.float32, device=H.device)
    diag = torch.empty(C, dtype=torch.float32, device=H.device) if want_diag else None
    if flags is None:
        flags = _flags_tensor(H.device)
    nbytes = L.mq_hinv_upper_workspace_bytes(C, p.math, p.split_hinv)
    ws = _lib.workspace(H.device, nbytes)
    with torch.cuda.device(H.device):
        check(L.mq_hinv_upper(ptr(H), C, H.stride(0), ptr(U), C, ptr(diag), p.math, p.split_hinv, ptr(flags), ptr(ws),
                              ws.numel(), stream_ptr(H.device)))
    return U, flags, diag


def absmax_scales(W: Tensor, group: int, bits: int, dtype: torch.dtype) -> Tensor:
    """(R, C/group) fp32 scales of the symmetric grid, already rounded through `dtype`."""
    require_cuda(W, "W")
    if W.dtype != torch.float32 or W.stride(1) != 1:
        raise MoeQuantError("W must be fp32 with unit column stride")
    R, C = W.shape
    out = torch.empty(R, C // group, dtype=torch.float32, device=W.device)
    with torch.cuda.device(W.device):
        check(lib().mq_absmax_scales(ptr(W), R, C, W.stride(0), group, bits, dtype_code(dtype), ptr(out),
                                     stream_ptr(W.device)))
    return out


def mse_scales(W: Tensor, scale: Tensor, group: int, bits: int, dtype: torch.dtype, max_shrink: float = 0.2,
               n_grid: int = 100, norm: float = 2.4) -> Tensor:
    """Refines absmax scales (R, C/group) in place by the reference's shrink-factor search and returns them."""
    require_cuda(W, "W")
    require_cuda(scale, "scale")
    if W.dtype != torch.float32 or W.stride(1) != 1 or scale.dtype != torch.float32 or not scale.is_contiguous():
        raise MoeQuantError("W must be fp32 with unit column stride, scale contiguous fp32")
    R, C = W.shape
    shrink = torch.linspace(1, max_shrink, n_grid, dtype=torch.float32, device=W.device)   # src/quant_utils.py:219
    with torch.cuda.device(W.device):
        check(lib().mq_mse_scales(ptr(W), R, C, W.stride(0), group, bits, dtype_code(dtype), ptr(shrink), n_grid, norm,
                                  ptr(scale), stream_ptr(W.device)))
    return scale


def chol_unit_factor(H: Tensor, precision: Optional[Precision] = None, flags: Optional[Tensor] = None):
    """In place: damped H -> Utilde = T diag(T)^-1 (unit upper), H = T T^T.  Returns (flags, diag(T))."""
    p = _prec(precision)
    require_cuda(H, "H")
    C = H.shape[0]
    L = lib()
    diag = torch.empty(C, dtype=torch.float32, device=H.device)
    if flags is None:
        flags = _flags_tensor(H.device)
    nbytes = L.mq_chol_unit_factor_workspace_bytes(C, p.math, p.split_hinv)
    ws = _lib.workspace(H.device, nbytes)
    with torch.cuda.device(H.device):
        check(L.mq_chol_unit_factor(ptr(H), C, H.stride(0), ptr(diag), p.math, p.split_hinv, ptr(flags), ptr(ws),
                                    ws.numel(), stream_ptr(H.device)))
    return flags, diag


def gptq_sweep(W: Tensor, Uhat: Tensor, scale: Tensor, zero: Optional[Tensor], group: int, row_stride: int,
               group_stride: int, bits: int, dtype: torch.dtype, want_dequantized: bool = False,
               precision: Optional[Precision] = None, W_original: Optional[Tensor] = None,
               packed_out: Optional[Tensor] = None) -> Tuple[Tensor, Optional[Tensor]]:
    """Column sweep over the fp32 working copy W (R, C), which is destroyed.
    With W_original (a second fp32 copy of the weights) `Uhat` must be the unit factor from
    chol_unit_factor and the inverse-free recurrence is used.
    packed_out: optional (R, C/8) int32 tensor that receives the compressed-tensors words.
    Returns (codes uint8 (R, C), dequantized (R, C) of `dtype` or None)."""
    p = _prec(precision)
    for t, n in ((W, "W"), (Uhat, "Uhat"), (scale, "scale")):
        require_cuda(t, n)
        if t.dtype != torch.float32:
            raise MoeQuantError(f"{n} must be fp32")
    R, C = W.shape
    L = lib()
    codes = torch.empty(R, C, dtype=torch.uint8, device=W.device)
    deq = torch.empty(R, C, dtype=dtype, device=W.device) if want_dequantized else None
    nbytes = L.mq_gptq_sweep_workspace_bytes(R, C, p.math, p.split_sweep)
    ws = _lib.workspace(W.device, nbytes)
    with torch.cuda.device(W.device):
        check(L.mq_gptq_sweep(ptr(W), R, C, W.stride(0), ptr(Uhat), Uhat.stride(0), ptr(scale), ptr(zero), group,
                              row_stride, group_stride, bits, dtype_code(dtype), ptr(codes), ptr(packed_out), ptr(deq),
                              ptr(W_original), 0 if W_original is None else W_original.stride(0), p.sweep_math,
                              p.split_sweep, ptr(ws), ws.numel(), stream_ptr(W.device)))
    return codes, deq


def quantize_layer(weights: Sequence[Tensor], H: Tensor, group: int, bits: int, rel_damp: float,
                   want_dequantized: bool = False, precision: Optional[Precision] = None, want_packed: bool = False):
    """GPTQ.quantize for one layer or for several layers that share H.

    weights: (R, C) tensors of one dtype; H (C, C) fp32 is damped in place.
    Returns (list of codes uint8 (R, C), list of scales fp32 (R, C/group),
             list of dequantized or None, flags int32[4] on the device); with want_packed a fifth
    element, the list of (R, C/8) int32 compressed-tensors words written by the sweep itself.
    """
    p = _prec(precision)
    require_cuda(H, "H")
    n = len(weights)
    R, C = weights[0].shape
    dtype = weights[0].dtype
    ws_list = []
    for w in weights:
        require_cuda(w, "weight")
        if w.shape != (R, C) or w.dtype != dtype:
            raise MoeQuantError("layers that share a Hessian must share shape and dtype")
        ws_list.append(w if w.is_contiguous() else w.contiguous())
    dev = H.device
    codes = [torch.empty(R, C, dtype=torch.uint8, device=dev) for _ in range(n)]
    scales = [torch.empty(R, C // group, dtype=torch.float32, device=dev) for _ in range(n)]
    deqs = [torch.empty(R, C, dtype=dtype, device=dev) for _ in range(n)] if want_dequantized else None
    packed = [torch.empty(R, C // 8, dtype=torch.int32, device=dev) for _ in range(n)] if want_packed else None
    flags = _flags_tensor(dev)
    L = lib()
    nbytes = L.mq_quantize_layer_workspace_bytes(n, R, C, p.math, p.split_hinv, p.split_sweep)
    ws = _lib.workspace(dev, nbytes)
    arr = ctypes.c_void_p * n
    w_arr = arr(*[t.data_ptr() for t in ws_list])
    c_arr = arr(*[t.data_ptr() for t in codes])
    s_arr = arr(*[t.data_ptr() for t in scales])
    d_arr = arr(*[t.data_ptr() for t in deqs]) if deqs is not None else None
    p_arr = arr(*[t.data_ptr() for t in packed]) if packed is not None else None
    with torch.cuda.device(dev):
        check(L.mq_quantize_layer(w_arr, dtype_code(dtype), n, R, C, ptr(H), H.stride(0), group, bits, rel_damp, c_arr,
                                  p_arr, s_arr, d_arr, ptr(flags), p.sweep_math, p.split_hinv, p.split_sweep, ptr(ws), ws.numel(),
                                  stream_ptr(dev)))
    if want_packed:
        return codes, scales, deqs, flags, packed
    return codes, scales, deqs, flags


def dequantize(codes: Tensor, scale: Tensor, zero: Optional[Tensor], group: int, bits: int,
               dtype: torch.dtype) -> Tensor:
    require_cuda(codes, "codes")
    R, C = codes.shape
    out = torch.empty(R, C, dtype=dtype, device=codes.device)
    codes = codes.contiguous()
    scale = scale.to(torch.float32).contiguous()
    zero = None if zero is None else zero.to(torch.float32).contiguous()
    with torch.cuda.device(codes.device):
        check(lib().mq_dequantize(ptr(codes), R, C, ptr(scale), ptr(zero), group, bits, dtype_code(dtype), ptr(out),
                                  stream_ptr(codes.device)))
    return out


def quadratic_form(A: Tensor, H: Tensor, precision: Optional[Precision] = None) -> Tensor:
    """sum((A @ H) * A) as a 0-d float64 tensor on the device.  A (R, C) fp32, H (C, C) fp32."""
    p = _prec(precision)
    require_cuda(A, "A")
    require_cuda(H, "H")
    if A.dtype != torch.float32 or H.dtype != torch.float32 or A.dim() != 2 or H.shape != (A.shape[1], A.shape[1]):
        raise MoeQuantError("quadratic_form: A must be (R, C) fp32 and H (C, C) fp32")
    A = A if A.stride(1) == 1 else A.contiguous()
    H = H if H.stride(1) == 1 else H.contiguous()
    R, C = A.shape
    out = torch.empty((), dtype=torch.float64, device=A.device)
    L = lib()
    ws = _lib.workspace(A.device, L.mq_quadratic_form_workspace_bytes(R, C, p.math, p.split_hinv))
    with torch.cuda.device(A.device):
        check(L.mq_quadratic_form(ptr(A), R, C, A.stride(0), ptr(H), H.stride(0), ptr(out), p.math, p.split_hinv,
                                  ptr(ws), ws.numel(), stream_ptr(A.device)))
    return out


def pack_int4(codes: Tensor, zero_i8: Optional[Tensor] = None, group: int = 0) -> Tensor:
    """(R, C) uint8 codes -> (R, ceil(C/8)) int32 words in the compressed-tensors layout."""
    require_cuda(codes, "codes")
    if codes.dtype != torch.uint8 or codes.dim() != 2:
        raise MoeQuantError("codes must be a 2-D uint8 tensor")
    codes = codes.contiguous()
    R, C = codes.shape
    out = torch.empty(R, (C + 7) // 8, dtype=torch.int32, device=codes.device)
    if zero_i8 is not None:
        zero_i8 = zero_i8.to(torch.int8).contiguous()
    with torch.cuda.device(codes.device):
        check(lib().mq_pack_int4(ptr(codes), R, C, ptr(zero_i8), group, ptr(out), stream_ptr(codes.device)))
    return out
