"""Parity at the benchmarked configuration: the 2048 x 7168 routed-expert gate_proj in the token
regimes the benchmark runs (ragged experts with far fewer tokens than input channels, and the
4096-token mean), the fp32 weight/activation configuration, and the 7168 x 16384 o_proj.

Rows are independent given the Hessian, so the CPU oracle runs on a slice of the rows with the
Hessian the device accumulated (the accumulation kernel has parity tests of its own) and every
gate is asserted on that slice:
    scales within 1e-3 relative, >= 99.5 % of the int4 codes equal, ||WX-QX||^2/||WX||^2 within
    1 % relative, packed words bit-exact given the codes.
With N << C the damped Hessian is so ill conditioned that any fp32 route, the reference's
included, differs from an exact inverse on a few codes per thousand: a code that sits on a
rounding boundary flips with the last bits of the factor, and one flip changes about a third
of the codes behind it in that row.  Two fp32 implementations (the reference on a CPU and on a
GPU, say) therefore disagree with each other by the sum of their own distances from exact
arithmetic, which at N = 1388 is already 0.3-0.4 % for the reference's route alone.  For these
cases the 99.5 % gate is asserted against the reference's algorithm in exact arithmetic (the
oracle with its factor computed in fp64), which is what both implementations approximate, and
the agreement with the fp32 oracle is required to stay within twice the oracle's own distance
from exact arithmetic (its noise plus an equal share for any other fp32 implementation).  All
three figures are printed.  Where N is of the order of C or larger the plain gate applies.
"""
import json
import os

import pytest
import torch
import torch.nn as nn

from moe_quant_b200 import GPTQ, ops, pack_weight, quant_utils
from oracle import gptq_oracle as O

pytestmark = pytest.mark.gpu

CODE_AGREEMENT = 0.995
SCALE_RTOL = 1e-3
RECON_RTOL = 0.01
ROWS = 128


def _layer(W):
    layer = nn.Linear(W.shape[1], W.shape[0], bias=False, dtype=W.dtype, device=W.device)
    layer.weight.data = W
    return layer


def _make(R, C, N, dtype, seed, cuda):
    g = torch.Generator(device="cuda").manual_seed(seed)
    W = (0.02 * torch.randn(R, C, generator=g, device=cuda)).to(dtype)
    chan = torch.exp(torch.randn(C, generator=g, device=cuda))
    X = (torch.randn(N, C, generator=g, device=cuda) * chan).to(dtype)
    return W, X


def _exact_factor_codes(W_rows, H_raw, group, rel_damp=1e-2):
    """Codes of the oracle's route with the factor computed in fp64 (then rounded to fp32): the
    reference's algorithm without the rounding noise of its fp32 factorisations."""
    H, Wf, _, _ = O.pre_step(H_raw.clone(), W_rows)
    Hd = H.double()
    Hd += rel_damp * torch.diag(Hd).mean() * torch.eye(Hd.shape[0], dtype=torch.float64)
    L = torch.linalg.cholesky(Hd)
    U = torch.linalg.cholesky(torch.cholesky_inverse(L), upper=True)
    U = (U / U.diag()[:, None]).float().contiguous()
    scale, zero, maxq = O.symmetric_grid(Wf, group, 4, W_rows.dtype)
    Q = O.gptq_sweep(Wf.t().contiguous(), U, scale.repeat_interleave(group, -1).t().contiguous(),
                     zero.repeat_interleave(group, -1).t().contiguous(), maxq, W_rows.dtype, 128)
    return Q.t().contiguous().to(torch.uint8)


def _report(name, **figures):
    line = json.dumps({"parity_case": name, **{k: round(float(v), 6) for k, v in figures.items()}})
    print(line)
    out = os.environ.get("MQ_PARITY_REPORT")
    if out:
        with open(out, "a") as f:
            f.write(line + "\n")


def _check_slice(name, W, H_raw, q, s, z, group, with_floor):
    rows = slice(0, ROWS)
    Wc, Hc = W[rows].cpu(), H_raw.cpu()
    want = O.quantize_layer(Wc, Hc.clone(), bits=4, group_size=group, rel_damp=1e-2, block_size=128)
    rel = ((s[rows].cpu().float() - want["scale"].float()).abs() / want["scale"].float().abs().clamp_min(1e-30)).max()
    agree = O.code_agreement(q[rows].cpu(), want["qweight"])
    got = O.dequantize_linear_weight(q[rows].cpu(), s[rows].cpu(), z[rows].cpu()).float()
    ref = O.dequantize_linear_weight(want["qweight"], want["scale"], want["zero"]).float()
    e_got, e_ref = O.reconstruction_error(Wc.float(), got, Hc), O.reconstruction_error(Wc.float(), ref, Hc)
    figures = dict(code_agreement=agree, scale_rel=rel, recon_error=e_got, recon_error_oracle=e_ref)
    if with_floor:
        exact = _exact_factor_codes(Wc, Hc, group)
        figures["code_agreement_with_exact_factor"] = O.code_agreement(q[rows].cpu(), exact)
        figures["oracle_fp32_vs_exact_factor"] = O.code_agreement(want["qweight"], exact)
    _report(name, **figures)
    assert float(rel) <= SCALE_RTOL
    if with_floor:
        assert figures["code_agreement_with_exact_factor"] >= CODE_AGREEMENT, figures
        assert 1.0 - agree <= 2.0 * (1.0 - figures["oracle_fp32_vs_exact_factor"]) + 1e-3, figures
    else:
        assert agree >= CODE_AGREEMENT, figures
    assert abs(e_got - e_ref) <= RECON_RTOL * e_ref, figures
    packed = pack_weight({"qweight": q[rows].contiguous(), "scale": s[rows].contiguous(), "zero": z[rows].contiguous()},
                         4, True, group)
    ref_packed = O.pack_weight({"qweight": q[rows].cpu(), "scale": s[rows].cpu(), "zero": z[rows].cpu()}, 4, True, group)
    assert torch.equal(packed["weight_packed"].cpu(), ref_packed["weight_packed"])


# 4096 = the mean routed expert of 32 x 4096 tokens over 256 experts with top-8 routing;
# 581 / 1388 / 1885 = token counts of the ragged experts the benchmark quantizes
@pytest.mark.parametrize("tokens", [4096, 1885, 1388, 581])
def test_gate_proj_bf16_matches_oracle(cuda, tokens):
    R, C = 2048, 7168
    W, X = _make(R, C, tokens, torch.bfloat16, 100 + tokens, cuda)
    h = GPTQ(_layer(W), 128, True, 1e-2, 128)
    h.update(X)
    H_raw = h.H.clone()
    q, s, z = h.quantize(4)
    assert not h.has_hessian_issues()
    _check_slice(f"gate_proj_2048x7168_bf16_N{tokens}", W, H_raw, q, s, z, 128, with_floor=tokens < 4096)


def test_gate_proj_fp32_weights_and_activations_match_oracle(cuda):
    """The fp32 configuration: fp32 layer, fp32 calibration activations (three-plane Hessian)."""
    R, C, N = 2048, 7168, 4096
    W, X = _make(R, C, N, torch.float32, 7, cuda)
    h = GPTQ(_layer(W), 128, True, 1e-2, 128)
    h.update(X[: N // 2])
    h.update(X[N // 2:])
    # the accumulated Hessian against fp64 arithmetic on a block of channels
    Xd = X[:, :512].double()
    want_H = (2.0 / N) * (Xd.t() @ Xd)
    torch.testing.assert_close(h.H[:512, :512].double(), want_H, rtol=2e-5, atol=1e-6 * float(want_H.abs().max()))
    H_raw = h.H.clone()
    q, s, z = h.quantize(4)
    assert not h.has_hessian_issues() and s.dtype == torch.float32
    _check_slice("gate_proj_2048x7168_fp32_N4096", W, H_raw, q, s, z, 128, with_floor=False)


def test_o_proj_matches_oracle_on_a_row_slice(cuda):
    """7168 x 16384 (the widest layer of the model: the Hessian alone is 1 GB)."""
    R, C, N = 7168, 16384, 16384
    W, X = _make(R, C, N, torch.bfloat16, 5, cuda)
    h = GPTQ(_layer(W), 128, True, 1e-2, 128)
    for part in X.split(4096):
        h.update(part)
    del X
    H_raw = h.H.clone()
    q, s, z = h.quantize(4)
    assert not h.has_hessian_issues()
    _check_slice("o_proj_7168x16384_bf16_N16384", W, H_raw, q, s, z, 128, with_floor=False)
    del H_raw
    ops._lib.release_workspaces()
    torch.cuda.empty_cache()
