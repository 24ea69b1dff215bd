"""The oracle against the fixtures produced by the reference's own code."""
import os

import numpy as np
import torch

from oracle import gptq_oracle as O


def _hessian(golden):
    H, n = None, 0
    steps = []
    for x in golden.batches:
        H, n = O.hessian_update(H, n, x)
        steps.append(H.clone())
    return H, n, steps


def test_hessian_update_matches_reference(golden):
    H, n, steps = _hessian(golden)
    assert n == int(golden.t("tokens"))
    torch.testing.assert_close(H, golden.t("H_final"), rtol=1e-5, atol=1e-6)
    if len(steps) > 1:
        torch.testing.assert_close(steps[0], golden.t("H_after0"), rtol=1e-5, atol=1e-6)


def test_layer_matches_reference(golden):
    out = O.quantize_layer(golden.W, golden.t("H_final").clone(), bits=4, group_size=golden.group, rel_damp=1e-2,
                           block_size=golden.block)
    # scales: same torch ops on the same inputs -> identical
    assert torch.equal(out["scale"].float(), golden.t("scale", typed=True).float())
    assert torch.equal(out["zero"].float(), golden.t("zero", typed=True).float())
    torch.testing.assert_close(out["H"], golden.t("H_damped"), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(out["Uhat"], golden.t("Uhat"), rtol=1e-3, atol=1e-5)
    # LAPACK may pick another code path on another CPU: allow a few boundary flips
    assert O.code_agreement(out["qweight"], golden.t("qweight")) >= 0.999


def test_sweep_given_reference_factor_is_exact(golden):
    """With the reference's own Uhat the restated sweep must give the fixture's codes
    exactly on any machine that rounds fp32 like IEEE (the only library call left is the
    block GEMM, whose summation order may differ: allow 1e-3 of the codes)."""
    W = golden.W
    H, Wf, _, _ = O.pre_step(golden.t("H_final").clone(), W)
    scale, zero, maxq = O.symmetric_grid(Wf, golden.group, 4, golden.dtype)
    sf = scale.repeat_interleave(golden.group, -1)
    zf = zero.repeat_interleave(golden.group, -1)
    Q = O.gptq_sweep(Wf.t().contiguous(), golden.t("Uhat"), sf.t().contiguous(), zf.t().contiguous(), maxq,
                     golden.dtype, golden.block or W.shape[1])
    q = Q.t().contiguous().to(torch.uint8)
    assert O.code_agreement(q, golden.t("qweight")) >= 0.999


def test_dequantize_and_error_match_reference(golden):
    q, s, z = golden.t("qweight"), golden.t("scale", typed=True), golden.t("zero", typed=True)
    deq = O.dequantize_linear_weight(q, s, z)
    assert torch.equal(deq.float(), golden.t("dequantized", typed=True).float())
    rel = O.relative_mse_error(deq.float(), golden.W.float(), golden.t("H_damped"))
    assert abs(float(rel) - float(golden.t("rel_error"))) <= 1e-4 * float(golden.t("rel_error"))


def test_pack_weight_matches_reference(golden):
    packed = O.pack_weight({"qweight": golden.t("qweight"), "scale": golden.t("scale", typed=True),
                            "zero": golden.t("zero", typed=True)}, 4, True, golden.group)
    assert torch.equal(packed["weight_packed"], golden.t("weight_packed"))
    assert packed["weight_packed"].dtype == torch.int32
    assert packed["weight_shape"].tolist() == golden.t("weight_shape").tolist()


def test_pack_to_int32_matches_library_vectors():
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "pack_int4.npz"))
    for key in z.files:
        if key.startswith("v_"):
            v = torch.from_numpy(z[key])
            assert torch.equal(O.pack_to_int32(v, 4), torch.from_numpy(z["p_" + key[2:]]))


def test_gptq_beats_round_to_nearest(golden):
    """Sanity of the fixtures themselves: error feedback must reduce the Hessian-weighted error."""
    W = golden.W.float()
    Hraw = golden.t("H_final")
    deq = golden.t("dequantized", typed=True).float()
    _, Wf, _, _ = O.pre_step(Hraw.clone(), golden.W)
    scale, zero, maxq = O.symmetric_grid(Wf, golden.group, 4, golden.dtype)
    sf, zf = scale.repeat_interleave(golden.group, -1), zero.repeat_interleave(golden.group, -1)
    rtn = (torch.clamp(torch.floor(Wf / sf + zf + 0.5), 0, maxq) - zf) * sf
    assert O.reconstruction_error(W, deq, Hraw) < O.reconstruction_error(W, rtn, Hraw)
