"""The column sweep pinned by the reference's own Triton loop.

tests/golden/sweep_triton.npz was written on a B200 by tests/golden/make_golden_sweep_gpu.py:
the reference's `src.gptq_loop.gptq_loop` (Triton kernels plus `addmm_`, unchanged) and its whole
`src.gptq.GPTQ` handle on the device.  The CPU tests here hold the oracle's restated sweep to
those codes; the GPU tests hold the CUDA sweep and the engine's handle to them.
"""
import ast
import os

import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import gptq_oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
Z = np.load(os.path.join(HERE, "golden", "sweep_triton.npz"))
CPU_CASES = ["fp32_g128", "bf16_rankdef", "fp16_g32_dead", "bf16_perchannel", "fp16_ragged_block", "bf16_g64_fullblock"]
MID_CASES = ["mid_bf16_g128", "mid_fp16_g64"]


def _t(key, dtype=None):
    a = torch.from_numpy(np.array(Z[key]))
    return a.view(torch.bfloat16) if dtype == torch.bfloat16 and a.dtype == torch.int16 else a


def _fixture_inputs(name):
    """(Wf after the pre-step, Uhat, scale (R,G) fp32, group, dtype, block) of a CPU fixture."""
    from tests.conftest import Golden
    g = Golden(name)
    _, Wf, _, _ = O.pre_step(g.t("H_final").clone(), g.W)
    return Wf, g.t("Uhat"), g.t("scale", typed=True).float(), g.group, g.dtype, g.block or g.W.shape[1]


def _mid_inputs(name):
    meta = ast.literal_eval(str(Z[f"{name}.meta"]))
    dtype = getattr(torch, meta["dtype"])
    W = _t(f"{name}.W", dtype)
    return W, _t(f"{name}.X", dtype), _t(f"{name}.Uhat"), _t(f"{name}.scale", dtype).float(), meta["g"], dtype, meta["b"]


def _oracle_sweep(Wf, Uhat, scale, group, dtype, block):
    sf = scale.repeat_interleave(group, -1)
    zf = torch.full_like(sf, 8.0)
    Q = O.gptq_sweep(Wf.t().contiguous(), Uhat, sf.t().contiguous(), zf.t().contiguous(), 15.0, dtype, block)
    return Q.t().contiguous().to(torch.uint8)


# ---------------------------------------------------------------------------- CPU: the oracle
@pytest.mark.parametrize("name", CPU_CASES)
def test_oracle_sweep_equals_the_reference_triton_loop(name):
    """Same inputs, same fp32 operations: the only freedom left is the summation order of the
    block GEMM (cuBLAS there, the CPU BLAS here)."""
    got = _oracle_sweep(*_fixture_inputs(name))
    want = _t(f"{name}.sweep_codes")
    agree = O.code_agreement(got, want)
    if name == "bf16_g64_fullblock":          # a single GPTQ block: no GEMM at all
        assert torch.equal(got, want)
    assert agree >= 0.999, agree


@pytest.mark.parametrize("name", MID_CASES)
def test_oracle_sweep_equals_the_reference_triton_loop_mid(name):
    W, _X, Uhat, scale, g, dtype, block = _mid_inputs(name)
    got = _oracle_sweep(W.float(), Uhat, scale, g, dtype, block)
    assert O.code_agreement(got, _t(f"{name}.sweep_codes")) >= 0.999


@pytest.mark.parametrize("name", CPU_CASES)
def test_oracle_layer_equals_the_reference_handle_on_the_device(name):
    """Whole handle: the reference ran cuBLAS / cuSOLVER / Triton, the oracle runs torch on the CPU."""
    from tests.conftest import Golden
    g = Golden(name)
    out = O.quantize_layer(g.W, g.t("H_final").clone(), bits=4, group_size=g.group, rel_damp=1e-2, block_size=g.block)
    assert torch.equal(out["scale"].float(), _t(f"{name}.scale", g.dtype).float())
    assert O.code_agreement(out["qweight"], _t(f"{name}.qweight")) >= 0.999


@pytest.mark.parametrize("name", MID_CASES)
def test_oracle_layer_equals_the_reference_handle_on_the_device_mid(name):
    W, X, _U, scale, g, dtype, block = _mid_inputs(name)
    H, _ = O.hessian_update(None, 0, X)
    out = O.quantize_layer(W, H, bits=4, group_size=g, rel_damp=1e-2, block_size=block)
    assert torch.equal(out["scale"].float(), scale)
    assert O.code_agreement(out["qweight"], _t(f"{name}.qweight")) >= 0.995


# ---------------------------------------------------------------------------- GPU: the engine
@pytest.mark.gpu
@pytest.mark.parametrize("math", ["fp32", "tensor"])
@pytest.mark.parametrize("name", CPU_CASES + MID_CASES)
def test_cuda_sweep_equals_the_reference_triton_loop(cuda, name, math):
    from moe_quant_b200 import ops
    from moe_quant_b200._lib import MATH_FP32, MATH_TENSOR
    if name in MID_CASES:
        W, _X, Uhat, scale, g, dtype, _block = _mid_inputs(name)
        Wf = W.float()
    else:
        Wf, Uhat, scale, g, dtype, _block = _fixture_inputs(name)
    p = ops.Precision(math=MATH_FP32 if math == "fp32" else MATH_TENSOR)
    codes, _ = ops.gptq_sweep(Wf.clone().to(cuda), Uhat.to(cuda), scale.to(cuda), None, g, Wf.shape[1] // g, 1, 4, dtype,
                              precision=p)
    assert O.code_agreement(codes.cpu(), _t(f"{name}.sweep_codes")) >= 0.999


@pytest.mark.gpu
@pytest.mark.parametrize("name", MID_CASES)
def test_engine_handle_equals_the_reference_handle_on_the_device(cuda, name):
    from moe_quant_b200 import GPTQ
    W, X, _U, scale, g, dtype, block = _mid_inputs(name)
    layer = nn.Linear(W.shape[1], W.shape[0], bias=False, dtype=dtype, device=cuda)
    layer.weight.data = W.to(cuda)
    h = GPTQ(layer, g, True, 1e-2, block)
    h.update(X.to(cuda))
    q, s, _z = h.quantize(4)
    assert torch.equal(s.cpu().float(), scale)
    assert O.code_agreement(q.cpu(), _t(f"{name}.qweight")) >= 0.995


# ---------------------------------------------------------------------------- the MSE scale search
MSE_CASES = ["mse_bfloat16_g128", "mse_float16_g32", "mse_float32_g64"]


def _mse_inputs(name):
    meta = ast.literal_eval(str(Z[f"{name}.meta"]))
    dtype = getattr(torch, meta["dtype"])
    return _t(f"{name}.W", dtype), _t(f"{name}.scale").float(), _t(f"{name}.scale_absmax").float(), meta["g"], dtype


def _check_mse_scales(got, want, base, dtype):
    """The reference sums |.|^2.4 over a group in whatever order its device reduction takes, so a
    candidate next to the minimum may win in one implementation and lose in another: nearly all
    scales identical, and every scale one of the hundred candidates of its group."""
    assert got.shape == want.shape
    assert float((got == want).float().mean()) >= 0.97
    cands = O.round_fp(base[..., None] * torch.linspace(1, 0.2, 100), dtype)
    assert bool((cands == got[..., None]).any(-1).all())
    assert float(((got - want).abs() / want).max()) <= 0.02    # a neighbour at worst: the grid step is 0.8 %


@pytest.mark.parametrize("name", MSE_CASES)
def test_oracle_mse_scales_equal_the_reference_grid_search(name):
    """`get_quantization_grid(..., QuantizationScale.MSE)` of the reference, run on the device."""
    W, want, base, g, dtype = _mse_inputs(name)
    s0, zero, maxq = O.symmetric_grid(W.float(), g, 4, dtype)
    assert torch.equal(s0.float(), base)
    got = O.mse_scale(W.float().unflatten(-1, (-1, g)), s0, zero, maxq, dtype).float()
    _check_mse_scales(got, want, base, dtype)


@pytest.mark.gpu
@pytest.mark.parametrize("name", MSE_CASES)
def test_cuda_mse_scales_equal_the_reference_grid_search(cuda, name):
    from moe_quant_b200 import ops
    W, want, base, g, dtype = _mse_inputs(name)
    Wd = W.float().to(cuda)
    s0 = ops.absmax_scales(Wd, g, 4, dtype)
    assert torch.equal(s0.cpu().float(), base)
    got = ops.mse_scales(Wd, s0, g, 4, dtype).cpu().float()
    _check_mse_scales(got, want, base, dtype)
