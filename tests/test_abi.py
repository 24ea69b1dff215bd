"""The shared library loads on a machine without a GPU and exports what the header declares."""
import ctypes
import os
import re

import pytest
import torch

from moe_quant_b200 import _lib, ops
from moe_quant_b200._lib import MoeQuantError

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols(headers=("moequant.h", "moequant_bench.h")):
    names = set()
    for header in headers:
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(mq_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_product_header_holds_no_measurement_hooks():
    product = _declared_symbols(("moequant.h",))
    assert not [n for n in product if "profile" in n or "launch_count" in n]


def test_library_exports_every_declared_symbol():
    handle = ctypes.CDLL(_lib.LIB_PATH)
    declared = _declared_symbols()
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(handle, name), f"{name} is declared in moequant.h but not exported"


def test_binding_table_matches_header():
    assert sorted(_lib.SIGNATURES) == _declared_symbols()


def test_abi_version_and_error_text():
    L = _lib.lib()
    assert L.mq_abi_version() == 2
    # argument validation happens on the host, before any CUDA call
    assert L.mq_pack_int4(None, 4, 8, None, 0, None, None) == 1
    assert b"null pointer" in L.mq_last_error()
    assert L.mq_pack_int4(None, -1, 8, None, 0, None, None) == 1
    assert L.mq_absmax_scales(None, 4, 8, 8, 8, 4, 0, None, None) == 1


def test_workspace_sizes_are_monotone_and_cover_the_big_shapes():
    L = _lib.lib()
    small = L.mq_quantize_layer_workspace_bytes(1, 2048, 7168, 1, 3, 3)
    tied = L.mq_quantize_layer_workspace_bytes(2, 2048, 7168, 1, 3, 3)
    fp32 = L.mq_quantize_layer_workspace_bytes(1, 2048, 7168, 0, 3, 3)
    big = L.mq_quantize_layer_workspace_bytes(1, 7168, 16384, 1, 3, 3)
    assert 0 < fp32 < small < tied < big < 40 * 2 ** 30
    assert L.mq_hessian_prepare_workspace_bytes(7168) >= 2 * 7168 * 4


def test_no_cpu_fallback():
    with pytest.raises(MoeQuantError):
        ops.pack_int4(torch.zeros(2, 8, dtype=torch.uint8))
    with pytest.raises(MoeQuantError):
        ops.hessian_accum(torch.zeros(8, 8), torch.zeros(3, 8), 0.0, 1.0)


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libmoequant_sm100.so")
    with pytest.raises(MoeQuantError, match="no fallback"):
        _lib.lib()
