"""ctypes binding of libmoequant_sm100.so (the C ABI declared in include/moequant.h).

The library is the only implementation of the GPTQ path in this package: there
is no torch or CPU fallback.  If it cannot be loaded, every operation raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmoequant_sm100.so")

MQ_F32, MQ_BF16, MQ_F16 = 0, 1, 2
MATH_FP32, MATH_TENSOR = 0, 1
MATH_COMPACT = 0x100   # MQ_MATH_COMPACT: flag OR-ed into the math argument of the sweep / whole-layer calls

_DTYPES = {torch.float32: MQ_F32, torch.bfloat16: MQ_BF16, torch.float16: MQ_F16}

# every exported symbol with (restype, argtypes); tests check the library against this table
SIGNATURES = {
    "mq_abi_version": (c_int, []),
    "mq_last_error": (c_char_p, []),
    "mq_launch_count": (ctypes.c_longlong, []),
    "mq_engine_fault": (c_int, [ctypes.POINTER(c_int)]),
    "mq_engine_fault_clear": (c_int, []),
    "mq_profile_begin": (c_int, []),
    "mq_profile_end": (c_int, [ctypes.POINTER(c_int64), ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double),
                               ctypes.POINTER(ctypes.c_double)]),
    "mq_hessian_accum": (c_int, [c_void_p, c_int, c_int64, c_int64, c_int64, c_void_p, c_int64, c_float, c_float,
                                 c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "mq_hessian_accum_workspace_bytes": (c_size_t, [c_int, c_int64, c_int64, c_int, c_int]),
    "mq_gemm": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int64,
                        c_int64, c_float, c_float, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "mq_gemm_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int64, c_int, c_int]),
    "mq_hessian_prepare": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_float, c_void_p,
                                   c_void_p, c_size_t, c_void_p]),
    "mq_hessian_prepare_workspace_bytes": (c_size_t, [c_int64]),
    "mq_hessian_prepare_noalloc": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_float, c_void_p,
                                           c_void_p]),
    "mq_hinv_upper": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p,
                              c_void_p, c_size_t, c_void_p]),
    "mq_hinv_upper_workspace_bytes": (c_size_t, [c_int64, c_int, c_int]),
    "mq_absmax_scales": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "mq_mse_scales": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_int, c_float,
                              c_void_p, c_void_p]),
    "mq_gptq_sweep": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64,
                              c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int,
                              c_void_p, c_size_t, c_void_p]),
    "mq_chol_unit_factor": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int, c_int, c_void_p, c_void_p, c_size_t,
                                    c_void_p]),
    "mq_chol_unit_factor_workspace_bytes": (c_size_t, [c_int64, c_int, c_int]),
    "mq_gptq_sweep_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int, c_int]),
    "mq_quantize_layer": (c_int, [c_void_p, c_int, c_int, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int,
                                  c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p,
                                  c_size_t, c_void_p]),
    "mq_quantize_layer_workspace_bytes": (c_size_t, [c_int, c_int64, c_int64, c_int, c_int, c_int]),
    "mq_dequantize": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p,
                              c_void_p]),
    "mq_quadratic_form": (c_int, [c_void_p, c_int64, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int, c_int,
                                  c_void_p, c_size_t, c_void_p]),
    "mq_quadratic_form_workspace_bytes": (c_size_t, [c_int64, c_int64, c_int, c_int]),
    "mq_pack_int4": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p]),
}

_lib: Optional[ctypes.CDLL] = None


class MoeQuantError(RuntimeError):
    """A non-zero mq_status from the library."""


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise MoeQuantError(
                f"{LIB_PATH} is missing: the sm_100a GPTQ engine has not been built "
                "(run `python -m moe_quant_b200.build`). There is no fallback implementation."
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status != 0:
        msg = lib().mq_last_error().decode(errors="replace")
        raise MoeQuantError(f"mq_status {status}: {msg}")


def engine_fault_clear() -> None:
    """Resets the current device's fault code once the caller has dropped the affected results."""
    check(lib().mq_engine_fault_clear())


def engine_fault() -> int:
    """Device-side status of the tensor-core kernels on the current device (0 = healthy).  Synchronises."""
    out = c_int(0)
    check(lib().mq_engine_fault(ctypes.byref(out)))
    return out.value


PROFILE_KINDS = ["umma_gemm", "simt_gemm", "sweep_tile", "chol_diag", "trsm_rows", "split_planes", "pack_int4", "other", "umma_deep"]


def profile_begin() -> None:
    check(lib().mq_profile_begin())


def profile_end() -> dict:
    """{kind: dict(launches, ms, work, work2)} for the launches since profile_begin()."""
    n = len(PROFILE_KINDS)
    launches = (c_int64 * n)()
    ms = (ctypes.c_double * n)()
    work = (ctypes.c_double * n)()
    work2 = (ctypes.c_double * n)()
    check(lib().mq_profile_end(launches, ms, work, work2))
    return {k: dict(launches=int(launches[i]), ms=float(ms[i]), work=float(work[i]), work2=float(work2[i]))
            for i, k in enumerate(PROFILE_KINDS)}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise MoeQuantError(f"unsupported dtype {dtype}: the engine takes float32, bfloat16 and float16") from None


def require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise MoeQuantError(f"{what} must live on a CUDA device (got {t.device}); this engine has no CPU path")


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_workspaces: dict = {}


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """A scratch buffer per (device, current stream).  Work is stream-ordered, so consecutive
    calls on one stream may share it; calls on different streams may overlap on the GPU and
    therefore get different buffers.  The buffer grows on demand; one of more than 1 GB is
    replaced by a smaller one when a call needs less than a quarter of it (a single very wide
    layer would otherwise pin gigabytes on every stream it ever ran on).  The caching allocator
    keeps the old block alive until the stream's queued work has used it."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (index, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    oversized = buf is not None and buf.numel() > (1 << 30) and 4 * max(int(nbytes), 1) < buf.numel()
    if buf is None or buf.numel() < nbytes or oversized:
        _workspaces[key] = None
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def release_workspaces() -> None:
    _workspaces.clear()
