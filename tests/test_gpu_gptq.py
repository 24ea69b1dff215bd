"""The GPTQ handle (the reference's call surface) end to end on the device."""
import pytest
import torch
import torch.nn as nn

from moe_quant_b200 import GPTQ, ops, pack_weight, quant_utils, quantize_tied, synthetic
from moe_quant_b200._lib import MATH_FP32, MATH_TENSOR
from oracle import gptq_oracle as O

pytestmark = pytest.mark.gpu

CODE_AGREEMENT = 0.995   # >= 99.5 % of int4 codes equal to the reference path's
SCALE_RTOL = 1e-3        # scales within 1e-3 relative
RECON_RTOL = 0.01        # ||WX-QX||^2/||WX||^2 within 1 % relative


@pytest.fixture(params=["fp32", "tensor"])
def precision(request):
    math = MATH_FP32 if request.param == "fp32" else MATH_TENSOR
    return ops.Precision(math=math, split_hessian=3, split_hinv=3, split_sweep=3)


def _layer(W, device):
    layer = nn.Linear(W.shape[1], W.shape[0], bias=False, dtype=W.dtype, device=device)
    layer.weight.data = W.to(device)
    return layer


def _check_against(q, s, z, W, want_q, want_s, H_raw, dtype, group):
    assert q.dtype == torch.uint8 and q.shape == W.shape and q.is_contiguous()
    assert s.dtype == dtype and z.dtype == dtype and s.shape == (W.shape[0], W.shape[1] // group)
    assert torch.all(z.float() == 8)
    rel = ((s.float().cpu() - want_s.float()).abs() / want_s.float().abs().clamp_min(1e-30)).max()
    assert float(rel) <= SCALE_RTOL
    assert O.code_agreement(q.cpu(), want_q) >= CODE_AGREEMENT
    deq = O.dequantize_linear_weight(q.cpu(), s.cpu(), z.cpu()).float()
    want_deq = O.dequantize_linear_weight(want_q, want_s, torch.full_like(want_s, 8)).float()
    e_got = O.reconstruction_error(W.float(), deq, H_raw)
    e_want = O.reconstruction_error(W.float(), want_deq, H_raw)
    assert abs(e_got - e_want) <= RECON_RTOL * e_want


def test_handle_matches_reference_fixture(cuda, golden, precision):
    layer = _layer(golden.W, cuda)
    h = GPTQ(layer, golden.group, True, 1e-2, golden.block, "default", "absmax", precision=precision)
    for x in golden.batches:
        h.update(x.to(cuda))
    assert h.tokens_collected == int(golden.t("tokens"))
    q, s, z = h.quantize(4)
    _check_against(q, s, z, golden.W, golden.t("qweight"), golden.t("scale", typed=True), golden.t("H_final"),
                   golden.dtype, golden.group)
    # the handle keeps the damped Hessian, as the reference's does (quant.py:314-316)
    torch.testing.assert_close(h.H.cpu(), golden.t("H_damped"), rtol=2e-5, atol=1e-5)
    assert not h.has_hessian_issues()
    # packed words are bit-exact given the codes
    packed = pack_weight({"qweight": q, "scale": s, "zero": z}, 4, True, golden.group)
    want = O.pack_weight({"qweight": q.cpu(), "scale": s.cpu(), "zero": z.cpu()}, 4, True, golden.group)
    assert torch.equal(packed["weight_packed"].cpu(), want["weight_packed"])
    assert packed["weight_shape"].tolist() == list(golden.W.shape)
    deq = quant_utils.dequantize_linear_weight(q, s, z)
    assert torch.equal(deq.cpu().float(), O.dequantize_linear_weight(q.cpu(), s.cpu(), z.cpu()).float())
    h.reset()
    assert h.H is None and h.tokens_collected == 0


@pytest.mark.parametrize("R,C,N,dtype,g", [(256, 1024, 700, torch.bfloat16, 128), (96, 2048, 1200, torch.float32, 128),
                                           (192, 512, 2000, torch.float16, 64)])
def test_handle_matches_oracle_medium(cuda, precision, R, C, N, dtype, g):
    W = synthetic.layer_weight(R, C, 11, dtype)
    X = synthetic.activations(N, C, 11, dtype)
    H_raw, _ = O.hessian_update(None, 0, X)
    want = O.quantize_layer(W, H_raw.clone(), bits=4, group_size=g, rel_damp=1e-2, block_size=128)
    h = GPTQ(_layer(W, cuda), g, True, 1e-2, 128, precision=precision)
    half = N // 2
    h.update(X[:half].to(cuda))
    h.update(X[half:].reshape(-1, 1, C).to(cuda))   # extra leading dims are flattened like the reference
    q, s, z = h.quantize(4)
    _check_against(q, s, z, W, want["qweight"], want["scale"], H_raw, dtype, g)


def test_tied_handles_share_one_factorisation(cuda, precision):
    R, C, N = 64, 512, 600
    Wg = synthetic.layer_weight(R, C, 1, torch.bfloat16)
    Wu = synthetic.layer_weight(R, C, 2, torch.bfloat16)
    X = synthetic.activations(N, C, 5, torch.bfloat16)
    H_raw, _ = O.hessian_update(None, 0, X)
    want_g = O.quantize_layer(Wg, H_raw.clone(), bits=4, group_size=128, block_size=128)
    want_u = O.quantize_layer(Wu, H_raw.clone(), bits=4, group_size=128, block_size=128)

    def handles():
        gate = GPTQ(_layer(Wg, cuda), 128, True, 1e-2, 128, precision=precision)
        up = GPTQ(_layer(Wu, cuda), 128, True, 1e-2, 128, tied_gptq_handle=gate, precision=precision)
        gate.update(X.to(cuda))
        return gate, up

    gate, up = handles()
    (qg, sg, zg), (qu, su, zu) = quantize_tied([gate, up], 4)
    _check_against(qg, sg, zg, Wg, want_g["qweight"], want_g["scale"], H_raw, torch.bfloat16, 128)
    _check_against(qu, su, zu, Wu, want_u["qweight"], want_u["scale"], H_raw, torch.bfloat16, 128)
    # the reference driver's order: quantize + reset one handle at a time (quant.py:351-387)
    gate, up = handles()
    qg2, sg2, _ = gate.quantize(4)
    gate.reset()
    assert gate.H is not None, "the Hessian must outlive its owner while a tied handle is pending"
    qu2, su2, _ = up.quantize(4)
    up.reset()
    assert gate.H is None
    assert torch.equal(qg2, qg) and torch.equal(qu2, qu) and torch.equal(su2, su)


def test_zero_samples_and_nan_flags(cuda, precision):
    W = synthetic.layer_weight(32, 256, 3, torch.bfloat16)
    h = GPTQ(_layer(W, cuda), 128, True, 1e-2, 128, precision=precision)
    q, s, z = h.quantize(4)      # never updated: identity Hessian, plain rounding
    assert h.issue_zero_samples and h.has_hessian_issues()
    want = O.quantize_layer(W, None, bits=4, group_size=128, block_size=128)
    assert O.code_agreement(q.cpu(), want["qweight"]) >= 0.999
    h2 = GPTQ(_layer(W, cuda), 128, True, 1e-2, 128, precision=precision)
    h2.update(synthetic.activations(64, 256, 3, torch.bfloat16).to(cuda))
    h2.H[3, 4] = float("nan")
    q2, _, _ = h2.quantize(4)
    assert h2.issue_nan_hessian
    assert O.code_agreement(q2.cpu(), want["qweight"]) >= 0.999


def test_activation_order(cuda, precision):
    R, C, N = 48, 512, 700
    W = synthetic.layer_weight(R, C, 13, torch.bfloat16)
    X = synthetic.activations(N, C, 13, torch.bfloat16)
    H_raw, _ = O.hessian_update(None, 0, X)
    want = O.quantize_layer(W, H_raw.clone(), bits=4, group_size=128, block_size=128, act_order=True)
    h = GPTQ(_layer(W, cuda), 128, True, 1e-2, 128, "activation", precision=precision)
    h.update(X.to(cuda))
    q, s, z = h.quantize(4)
    _check_against(q, s, z, W, want["qweight"], want["scale"], H_raw, torch.bfloat16, 128)


def test_tied_handles_with_activation_order(cuda, precision):
    """gate_proj / up_proj tied under activation ordering: the shared Hessian is regularised once
    (by its owner), whichever handle is quantized first and through whichever call."""
    R, C, N = 48, 512, 700
    Wg = synthetic.layer_weight(R, C, 31, torch.bfloat16)
    Wu = synthetic.layer_weight(R, C, 32, torch.bfloat16)
    X = synthetic.activations(N, C, 33, torch.bfloat16)
    H_raw, _ = O.hessian_update(None, 0, X)
    want_g = O.quantize_layer(Wg, H_raw.clone(), bits=4, group_size=128, block_size=128, act_order=True)
    want_u = O.quantize_layer(Wu, H_raw.clone(), bits=4, group_size=128, block_size=128, act_order=True)
    damped = H_raw + 1e-2 * torch.diag(H_raw).mean() * torch.eye(C)

    def handles():
        gate = GPTQ(_layer(Wg, cuda), 128, True, 1e-2, 128, "activation", precision=precision)
        up = GPTQ(_layer(Wu, cuda), 128, True, 1e-2, 128, "activation", tied_gptq_handle=gate, precision=precision)
        gate.update(X.to(cuda))
        return gate, up

    gate, up = handles()
    qg, sg, zg = gate.quantize(4)
    qu, su, zu = up.quantize(4)
    tol = dict(rtol=2e-5, atol=1e-5 * float(damped.abs().max()))
    torch.testing.assert_close(gate.H.cpu(), damped, **tol)      # damped once, not twice
    _check_against(qg, sg, zg, Wg, want_g["qweight"], want_g["scale"], H_raw, torch.bfloat16, 128)
    _check_against(qu, su, zu, Wu, want_u["qweight"], want_u["scale"], H_raw, torch.bfloat16, 128)
    gate, up = handles()
    (qg2, _, _), (qu2, _, _) = quantize_tied([gate, up], 4)      # falls back to one call per handle
    torch.testing.assert_close(gate.H.cpu(), damped, **tol)
    assert torch.equal(qg2, qg) and torch.equal(qu2, qu)
    # the Hessian-inverse seam of a tied handle must not regularise again either
    up._get_hessian_inverse()
    torch.testing.assert_close(gate.H.cpu(), damped, **tol)


def test_engine_fault_clear_leaves_a_healthy_device_healthy(cuda):
    from moe_quant_b200 import _lib
    assert _lib.engine_fault() == 0
    _lib.engine_fault_clear()
    assert _lib.engine_fault() == 0


def test_full_size_layer_properties(cuda, precision):
    """2048 x 7168 (the expert gate_proj shape): too large for the oracle to finish in
    seconds, so check what must hold at any size: codes in range, finite dequantized
    weights, error feedback beats plain rounding, pack/unpack returns the codes."""
    R, C, N = 2048, 7168, 4096
    g = torch.Generator(device="cuda").manual_seed(0)
    W = (0.02 * torch.randn(R, C, generator=g, device=cuda)).to(torch.bfloat16)
    chan = torch.exp(torch.randn(C, generator=g, device=cuda))
    X = (torch.randn(N, C, generator=g, device=cuda) * chan).to(torch.bfloat16)
    h = GPTQ(_layer(W, cuda), 128, True, 1e-2, 128, precision=precision)
    h.update(X[: N // 2])
    h.update(X[N // 2:])
    H_raw = h.H.clone()
    q, s, z = h.quantize(4)
    assert not h.has_hessian_issues()
    assert int(q.max()) <= 15
    deq = quant_utils.dequantize_linear_weight(q, s, z).float()
    assert bool(torch.isfinite(deq).all())
    Wf = W.float()
    sf = s.float().repeat_interleave(128, dim=-1)
    rtn = (torch.clamp(torch.floor(Wf / sf + 8.5), 0, 15) - 8) * sf
    def err(Wq):
        d = Wq - Wf
        return float((d @ H_raw).mul(d).sum() / (Wf @ H_raw).mul(Wf).sum())
    assert err(deq) < 0.6 * err(rtn)
    words = ops.pack_int4(q)
    shifts = torch.arange(8, device=cuda, dtype=torch.int32) * 4
    assert torch.equal(((words.unsqueeze(-1) >> shifts) & 0xF).reshape(R, C).to(torch.uint8), q)


def test_quantize_many_streams_match_sequential(cuda, precision):
    from moe_quant_b200 import quantize_many
    R, C, N = 64, 512, 600
    Ws = [synthetic.layer_weight(R, C, 20 + i, torch.bfloat16) for i in range(5)]
    Xs = [synthetic.activations(N + 37 * i, C, 40 + i, torch.bfloat16) for i in range(5)]

    def handles():
        hs = []
        for W, X in zip(Ws, Xs):
            h = GPTQ(_layer(W, cuda), 128, True, 1e-2, 128, precision=precision)
            h.update(X.to(cuda))
            hs.append(h)
        return hs

    seq = [h.quantize(4) for h in handles()]
    par = quantize_many(handles(), 4, streams=3)
    torch.cuda.synchronize()
    for (q1, s1, z1), (q2, s2, z2) in zip(seq, par):
        assert torch.equal(q1, q2) and torch.equal(s1, s2) and torch.equal(z1, z2)


def test_quantize_many_groups_tied_handles(cuda, precision):
    """Handles of the list that are tied to another handle of the list (gate_proj / up_proj with
    --tie_gptq_handles) are quantized with it, one factorisation per group, side by side with
    the untied ones; every result equals what quantize_tied / quantize give for that group alone."""
    from moe_quant_b200 import quantize_many
    R, C, N = 72, 640, 700
    Ws = [synthetic.layer_weight(R, C, 60 + i, torch.bfloat16) for i in range(7)]
    Xs = [synthetic.activations(N + 11 * i, C, 80 + i, torch.bfloat16) for i in range(3)]

    def handles():
        hs = []
        for e in range(3):                                    # gate, up (tied to gate), and an untied layer per expert
            gate = GPTQ(_layer(Ws[2 * e], cuda), 128, True, 1e-2, 128, precision=precision)
            gate.update(Xs[e].to(cuda))
            up = GPTQ(_layer(Ws[2 * e + 1], cuda), 128, True, 1e-2, 128, precision=precision, tied_gptq_handle=gate)
            other = GPTQ(_layer(Ws[6], cuda), 128, True, 1e-2, 128, precision=precision)
            other.update(Xs[(e + 1) % 3].to(cuda))
            hs += [up, other, gate] if e == 1 else [gate, up, other]   # order inside the list does not matter
        return hs

    # one group at a time on the current stream: quantize_tied for a pair, quantize for a single handle
    from moe_quant_b200 import quantize_tied
    hs_seq = handles()
    want = [None] * len(hs_seq)
    for i, h in enumerate(hs_seq):
        if h.tied_gptq_handle is not None:
            continue
        tied = [j for j, t in enumerate(hs_seq) if t.tied_gptq_handle is h]
        if tied:
            for j, r in zip([i] + tied, quantize_tied([h] + [hs_seq[j] for j in tied], 4)):
                want[j] = r
        else:
            want[i] = h.quantize(4)
    got = quantize_many(handles(), 4, streams=4)
    torch.cuda.synchronize()
    assert len(got) == len(want)
    for (q1, s1, z1), (q2, s2, z2) in zip(want, got):
        assert torch.equal(q1, q2) and torch.equal(s1, s2) and torch.equal(z1, z2)


def test_conv_layer_goes_through_unfold(cuda, precision):
    """Convolutions are handled like the reference does: inputs unfolded to patches
    (src/gptq.py:87-96), weight flattened to (out, in*kh*kw)."""
    g = torch.Generator().manual_seed(2)
    conv = nn.Conv2d(8, 16, kernel_size=2, stride=1, padding=1, bias=False, dtype=torch.bfloat16)
    conv.weight.data = (0.05 * torch.randn(16, 8, 2, 2, generator=g)).to(torch.bfloat16)
    x = torch.randn(3, 8, 12, 12, generator=g).to(torch.bfloat16)
    h = GPTQ(conv.to(cuda), 32, True, 1e-2, 128, precision=precision)
    h.update(x.to(cuda))
    q, s, z = h.quantize(4)
    assert q.shape == (16, 32) and s.shape == (16, 1)
    patches = nn.Unfold(2, dilation=1, padding=1, stride=1)(x.float()).transpose(1, 2).flatten(0, 1).to(torch.bfloat16)
    assert h.tokens_collected == patches.shape[0]
    H, _ = O.hessian_update(None, 0, patches)
    want = O.quantize_layer(conv.weight.detach().cpu().flatten(1), H, bits=4, group_size=32, rel_damp=1e-2, block_size=128)
    assert torch.equal(s.cpu().float(), want["scale"].float())
    assert O.code_agreement(q.cpu(), want["qweight"]) >= CODE_AGREEMENT


def test_mse_scale_search_through_the_handle(cuda):
    """QuantizationScale.MSE (the Enum member) runs the search; the STRING "mse" gives the
    absmax grid, as in the reference, whose handle compares a string with the Enum
    (src/gptq.py:47, src/quant_utils.py:218)."""
    from moe_quant_b200.quant_utils import QuantizationScale
    R, C, N = 64, 512, 700
    W = synthetic.layer_weight(R, C, 71, torch.bfloat16)
    X = synthetic.activations(N, C, 72, torch.bfloat16)
    H_raw, _ = O.hessian_update(None, 0, X)
    want = O.quantize_layer(W, H_raw.clone(), bits=4, group_size=128, block_size=128, mse=True)
    plain = O.quantize_layer(W, H_raw.clone(), bits=4, group_size=128, block_size=128)

    def run(scale_arg):
        h = GPTQ(_layer(W, cuda), 128, True, 1e-2, 128, "default", scale_arg)
        h.update(X.to(cuda))
        return h.quantize(4)

    q, s, z = run(QuantizationScale.MSE)
    same = (s.cpu().float() == want["scale"].float())
    assert float(same.float().mean()) >= 0.97
    assert float((s.cpu().float() < plain["scale"].float()).float().mean()) > 0.5     # the search shrinks most groups
    rows_ok = same.all(-1)
    assert O.code_agreement(q.cpu()[rows_ok], want["qweight"][rows_ok]) >= CODE_AGREEMENT
    deq = O.dequantize_linear_weight(q.cpu(), s.cpu(), z.cpu()).float()
    ref = O.dequantize_linear_weight(want["qweight"], want["scale"], want["zero"]).float()
    e_got, e_ref = O.reconstruction_error(W.float(), deq, H_raw), O.reconstruction_error(W.float(), ref, H_raw)
    assert abs(e_got - e_ref) <= 0.02 * e_ref
    q2, s2, _ = run("mse")
    assert torch.equal(s2.cpu().float(), plain["scale"].float())
    assert O.code_agreement(q2.cpu(), plain["qweight"]) >= CODE_AGREEMENT


@pytest.mark.parametrize("R,C,g,dtype", [(96, 1024, 128, torch.bfloat16), (40, 264, 8, torch.float16), (2048, 2048, 64, torch.bfloat16)])
def test_quantize_packed_writes_the_words_in_the_sweep(cuda, R, C, g, dtype):
    """The fused route: same codes and scales as quantize(), and words bit-identical to what the
    packer (and compressed-tensors' pack_to_int32) makes of those codes."""
    W = synthetic.layer_weight(R, C, 81, dtype)
    X = synthetic.activations(600, C, 82, dtype)

    def handle():
        h = GPTQ(_layer(W, cuda), g, True, 1e-2, 128)
        h.update(X.to(cuda))
        return h

    q, s, z = handle().quantize(4)
    out = handle().quantize_packed(4)
    assert torch.equal(out["qweight"], q) and torch.equal(out["scale"], s) and torch.equal(out["zero"], z)
    assert out["weight_packed"].dtype == torch.int32 and out["weight_packed"].shape == (R, C // 8)
    assert out["weight_shape"].tolist() == [R, C] and out["weight_scale"] is out["scale"]
    want = O.pack_weight({"qweight": q.cpu(), "scale": s.cpu(), "zero": z.cpu()}, 4, True, g)
    assert torch.equal(out["weight_packed"].cpu(), want["weight_packed"])
    # a handle on another route (activation order) packs in a second pass: same contract
    h = GPTQ(_layer(W, cuda), g, True, 1e-2, 128, "activation")
    h.update(X.to(cuda))
    out2 = h.quantize_packed(4)
    want2 = O.pack_weight({"qweight": out2["qweight"].cpu(), "scale": out2["scale"].cpu(), "zero": out2["zero"].cpu()}, 4, True, g)
    assert torch.equal(out2["weight_packed"].cpu(), want2["weight_packed"])


def test_repeated_quantization_is_bit_identical_and_clean(cuda):
    """The same layer many times over, alone and on several streams at once: every run must give the
    same codes bit for bit and raise no Hessian flag (a race inside a kernel shows up as a rare
    non-positive pivot or a handful of different codes)."""
    from moe_quant_b200 import quantize_many
    R, C, N = 512, 2048, 1000
    g = torch.Generator(device="cuda").manual_seed(3)
    W = (0.02 * torch.randn(R, C, generator=g, device=cuda)).to(torch.bfloat16)
    X = (torch.randn(N, C, generator=g, device=cuda) * torch.exp(torch.randn(C, generator=g, device=cuda))).to(torch.bfloat16)
    H = torch.zeros(C, C, device=cuda)
    ops.hessian_accum(H, X, 0.0, 2.0 / N)

    def handles(n):
        out = []
        for _ in range(n):
            h = GPTQ(_layer(W, cuda), 128, True, 1e-2, 128)
            h.H, h.num_samples = H.clone(), N
            out.append(h)
        return out

    first = handles(1)[0].quantize(4)
    seq = handles(40)
    for h in seq:
        q, s, _ = h.quantize(4)
        assert torch.equal(q, first[0]) and torch.equal(s, first[1])
    par = handles(48)
    for q, s, _ in quantize_many(par, 4, streams=8):
        assert torch.equal(q, first[0]) and torch.equal(s, first[1])
    assert not any(h.has_hessian_issues() for h in seq + par)
