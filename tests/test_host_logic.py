"""Bookkeeping of the GPTQ handle that needs no device (src/gptq.py:22-136)."""
import pytest
import torch
import torch.nn as nn

from moe_quant_b200 import GPTQ, QuantizationOrder, model_utils
from moe_quant_b200._lib import MoeQuantError


def _layer(R=8, C=16, dtype=torch.bfloat16):
    return nn.Linear(C, R, bias=False, dtype=dtype)


def test_constructor_matches_reference_positional_order():
    layer = _layer()
    h = GPTQ(layer, 8, True, 0.05, 128, "activation", "absmax", is_distributed=True)
    assert (h.d_row, h.d_col) == (8, 16)
    assert h.group_size == 8 and h.sym and h.rel_damp == 0.05 and h.block_size == 128
    assert h.quantization_order is QuantizationOrder.ACTIVATION and h.is_distributed
    assert h.W_dtype == torch.bfloat16 and h.W_shape == (8, 16)
    assert h.H is None and h.tokens_collected == 0 and not h.has_hessian_issues()
    assert GPTQ(_layer(), None).block_size == 16      # block defaults to d_col (src/gptq.py:45)


def test_rejects_other_modules():
    with pytest.raises(AssertionError):
        GPTQ(nn.LayerNorm(4))


def test_tied_handle_reference_counting():
    gate = GPTQ(_layer(), 8, True)
    up = GPTQ(_layer(), 8, True, tied_gptq_handle=gate)
    assert gate.num_tied_handles == 1 and up.num_tied_handles == 0
    gate.H = torch.eye(16)
    gate.reset()
    assert gate.H is not None               # still needed by `up`
    up.quantization_pre_step()
    assert up.H is gate.H and not up.issue_zero_samples
    up.reset()
    assert gate.H is None and gate.num_tied_handles == 0


def test_zero_samples_falls_back_to_identity():
    h = GPTQ(_layer(), 8, True)
    h.quantization_pre_step()
    assert h.issue_zero_samples and torch.equal(h.H, torch.eye(16))


def test_update_on_cpu_raises():
    h = GPTQ(_layer(), 8, True)
    with pytest.raises(MoeQuantError):
        h.update(torch.zeros(4, 16, dtype=torch.bfloat16))


def test_asymmetric_is_refused():
    h = GPTQ(_layer(), 8, False)
    h.H = torch.eye(16)
    with pytest.raises(MoeQuantError, match="symmetric"):
        h.quantize(4)


def test_model_utils():
    conv = nn.Conv2d(3, 5, 3)
    assert model_utils.get_number_of_rows_and_cols(conv) == (5, 27)
    model = nn.Sequential(nn.Linear(4, 4), nn.ReLU(), nn.Sequential(nn.Linear(4, 2)))
    got = model_utils.select_layers(model, "", ".*", model_utils.LINEAR_LAYERS)
    assert sorted(got) == ["0", "2.0"]
    assert sorted(model_utils.select_layers(model, "2", ".*", nn.Linear)) == ["2.0"]


def test_expired_device_wait_is_reported_with_the_layer_flags(monkeypatch):
    """Reading a layer's status words is where an expired wait of the tensor-core kernels must
    surface: the codes of that layer are garbage and may not be saved as a result."""
    from moe_quant_b200 import _lib

    h = GPTQ(_layer(), 8, True)
    h._pending_flags = [torch.zeros(4, dtype=torch.int32)]
    monkeypatch.setattr(_lib, "engine_fault", lambda: 13)
    with pytest.raises(MoeQuantError, match="bounded wait"):
        h.has_hessian_issues()
    # once reported, the flags are consumed; a healthy device reads clean again
    monkeypatch.setattr(_lib, "engine_fault", lambda: 0)
    h._pending_flags = [torch.tensor([1, 0, 0, 5], dtype=torch.int32)]
    assert h.issue_nan_hessian and h.issue_non_invertible


def test_tied_groups_and_compact_launch_scope():
    """Host side of quantize_many: handles tied to one another form one group led by the owner of
    the Hessian (wherever they stand in the list), a tied handle whose owner is not in the list
    stands alone; inside `compact_launches` a handle asks for compact launch shapes and gets its
    own precision object back afterwards, also when the body raises."""
    from moe_quant_b200 import gptq, ops

    def lin():
        return nn.Linear(16, 8, bias=False)

    gate0, gate1 = GPTQ(lin(), 8, True, 1e-2, 128), GPTQ(lin(), 8, True, 1e-2, 128)
    up0 = GPTQ(lin(), 8, True, 1e-2, 128, tied_gptq_handle=gate0)
    up1 = GPTQ(lin(), 8, True, 1e-2, 128, tied_gptq_handle=gate1)
    down = GPTQ(lin(), 8, True, 1e-2, 128)
    outsider = GPTQ(lin(), 8, True, 1e-2, 128, tied_gptq_handle=GPTQ(lin(), 8, True, 1e-2, 128))
    handles = [up0, gate0, down, gate1, outsider, up1]
    assert gptq._tied_groups(handles) == [[1, 0], [2], [3, 5], [4]]

    assert down.precision is None
    with gptq.compact_launches(down):
        assert down.precision.compact and down.precision.sweep_math == ops.MATH_TENSOR | 0x100
    assert down.precision is None
    mine = ops.Precision(math=0)
    down.precision = mine
    with pytest.raises(RuntimeError):
        with gptq.compact_launches(down):
            assert down.precision.compact and down.precision.math == 0
            raise RuntimeError("body failed")
    assert down.precision is mine and not mine.compact
    with gptq.compact_launches(down, on=False):
        assert down.precision is mine
