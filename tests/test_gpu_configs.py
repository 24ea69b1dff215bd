"""The layer shapes of the other benchmark configurations: the MLA attention projections
(q_a 1536x7168, q_b 24576x1536, kv_a 576x7168, kv_b 32768x512, o 7168x16384) and the
group-size / packing sweep on the expert down_proj shape (7168x2048, g in {32, 64, 128, C}).

Where the CPU oracle finishes in seconds the codes are compared with it (rows are independent
given the Hessian, so a slice of the rows is compared when the layer is tall); o_proj
(C = 16384) is checked through size-independent properties only.
"""
import pytest
import torch
import torch.nn as nn

from moe_quant_b200 import GPTQ, ops, pack_weight, quant_utils, synthetic
from oracle import gptq_oracle as O

pytestmark = pytest.mark.gpu

CODE_AGREEMENT = 0.995
RECON_RTOL = 0.01


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


def _rtn_error_ratio(W, q, s, H_raw, group):
    Wf = W.float()
    deq = quant_utils.dequantize_linear_weight(q, s, torch.full_like(s, 8)).float()
    sf = s.float().repeat_interleave(group, dim=-1)
    rtn = (torch.clamp(torch.floor(Wf / sf + 8.5), 0, 15) - 8) * sf

    def err(Wq):
        d = Wq - Wf
        return float((d @ H_raw).mul(d).sum())

    return err(deq) / err(rtn)


# Tokens: the configuration calibrates these layers with 262144 tokens, far more than C, which
# makes H well conditioned.  N >= C keeps that property at test size.  (With N < C the damped H
# has thousands of near-null directions and even the reference's fp32 pipeline agrees with an
# exact-arithmetic inverse on only about 99.8 % of the codes: there the 99.5 % bar sits in the
# rounding noise of any implementation.)
@pytest.mark.parametrize("name,R,C,N,rows_checked", [
    ("q_a_proj", 1536, 7168, 8192, 256),
    ("q_b_proj", 24576, 1536, 4096, 512),
    ("kv_a_proj_with_mqa", 576, 7168, 8192, 576),
    ("kv_b_proj", 32768, 512, 2048, 2048),
])
def test_mla_projection_matches_oracle(cuda, name, R, C, N, rows_checked):
    W, X = _make(R, C, N, torch.bfloat16, sum(map(ord, name)), cuda)
    h = GPTQ(_layer(W), 128, True, 1e-2, 128)
    h.update(X[: N // 2])
    h.update(X[N // 2:])
    H_raw = h.H.clone()
    q, s, z = h.quantize(4)
    assert not h.has_hessian_issues()
    assert q.shape == (R, C) and s.shape == (R, C // 128) and int(q.max()) <= 15
    # oracle on a slice of the rows with the Hessian the device accumulated (that kernel has its
    # own parity tests): isolates prepare + factor + sweep
    rows = slice(0, rows_checked)
    want = O.quantize_layer(W[rows].cpu(), H_raw.cpu().clone(), bits=4, group_size=128, rel_damp=1e-2, block_size=128)
    assert torch.equal(s[rows].cpu().float(), want["scale"].float())
    assert O.code_agreement(q[rows].cpu(), want["qweight"]) >= CODE_AGREEMENT
    Wc, Hc = W[rows].cpu().float(), H_raw.cpu()
    got = O.dequantize_linear_weight(q[rows].cpu(), s[rows].cpu(), z[rows].cpu()).float()
    ref = O.dequantize_linear_weight(want["qweight"], want["scale"], want["zero"]).float()
    e_got, e_ref = O.reconstruction_error(Wc, got, Hc), O.reconstruction_error(Wc, ref, Hc)
    assert abs(e_got - e_ref) <= RECON_RTOL * e_ref


def test_o_proj_properties(cuda):
    """7168 x 16384: H alone is 1 GB; properties only."""
    R, C, N = 7168, 16384, 4096
    W, X = _make(R, C, N, torch.bfloat16, 5, cuda)
    h = GPTQ(_layer(W), 128, True, 1e-2, 128)
    h.update(X)
    H_raw = h.H.clone()
    q, s, z = h.quantize(4)
    assert not h.has_hessian_issues()
    assert int(q.max()) <= 15 and bool(torch.isfinite(s.float()).all())
    assert _rtn_error_ratio(W, q, s, H_raw, 128) < 0.7
    words = ops.pack_int4(q)
    shifts = torch.arange(8, device=cuda, dtype=torch.int32) * 4
    assert torch.equal(((words.unsqueeze(-1) >> shifts) & 0xF).reshape(R, C).to(torch.uint8), q)


@pytest.mark.parametrize("group", [32, 64, 128, 2048])
def test_down_proj_group_sweep_and_packing(cuda, group):
    """fp16 layer (fp16 scales), 8192 tokens; packed words bit-exact against the packer oracle."""
    R, C, N = 7168, 2048, 8192
    W, X = _make(R, C, N, torch.float16, 40 + group, cuda)
    h = GPTQ(_layer(W), group, True, 1e-2, 128)
    h.update(X)
    H_raw = h.H.clone()
    q, s, z = h.quantize(4)
    assert s.dtype == torch.float16 and s.shape == (R, C // group)
    rows = slice(0, 384)
    want = O.quantize_layer(W[rows].cpu(), H_raw.cpu().clone(), bits=4, group_size=group, rel_damp=1e-2, block_size=128)
    assert torch.equal(s[rows].cpu().float(), want["scale"].float())
    assert O.code_agreement(q[rows].cpu(), want["qweight"]) >= CODE_AGREEMENT
    packed = pack_weight({"qweight": q, "scale": s, "zero": z}, 4, True, group)
    ref = O.pack_weight({"qweight": q.cpu(), "scale": s.cpu(), "zero": z.cpu()}, 4, True, group)
    assert torch.equal(packed["weight_packed"].cpu(), ref["weight_packed"])
    assert packed["weight_packed"].shape == (R, C // 8) and packed["weight_shape"].tolist() == [R, C]
    assert _rtn_error_ratio(W, q, s, H_raw, group) < 1.0   # error feedback must not lose to plain rounding
