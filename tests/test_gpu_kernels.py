"""Parity of every CUDA entry point (called through the C ABI) with the oracle and
with the fixtures written by the reference's own code.

Tolerances (from the stated parity bar): packed words and dequantized values
bit-exact; scales exact (<= 1e-3 relative allowed); >= 99.5 % of the int4 codes equal;
Hessian-weighted reconstruction error within 1 % relative.
"""
import os

import numpy as np
import pytest
import torch

from moe_quant_b200 import ops, synthetic
from moe_quant_b200._lib import MATH_FP32, MATH_TENSOR, MoeQuantError
from oracle import gptq_oracle as O

pytestmark = pytest.mark.gpu

CODE_AGREEMENT = 0.995
SCALE_RTOL = 1e-3
RECON_RTOL = 0.01


@pytest.fixture(params=["fp32", "tensor"])
def precision(request):
    math = MATH_FP32 if request.param == "fp32" else MATH_TENSOR
    return ops.Precision(math=math, split_hessian=3, split_hinv=3, split_sweep=3)


# ------------------------------------------------------------------ packing
def test_pack_golden_vectors(cuda):
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "pack_int4.npz"))
    for key in z.files:
        if key.startswith("v_"):
            v = torch.from_numpy(z[key])
            got = ops.pack_int4((v + 8).to(torch.uint8).to(cuda)).cpu()
            assert torch.equal(got, torch.from_numpy(z["p_" + key[2:]])), key


@pytest.mark.parametrize("shape", [(1, 16), (7, 2048), (33, 264), (5, 13), (128, 7168), (3, 1), (0, 64), (4, 0)])
def test_pack_random_shapes(cuda, shape):
    g = torch.Generator().manual_seed(shape[0] * 131 + shape[1])
    codes = torch.randint(0, 16, shape, generator=g, dtype=torch.uint8)
    got = ops.pack_int4(codes.to(cuda)).cpu()
    want = O.pack_to_int32(codes.to(torch.int8) - 8, 4) if codes.numel() else torch.empty(shape[0], (shape[1] + 7) // 8, dtype=torch.int32)
    assert got.shape == want.shape and torch.equal(got, want)


def test_pack_with_zero_points(cuda):
    g = torch.Generator().manual_seed(5)
    codes = torch.randint(0, 16, (9, 64), generator=g, dtype=torch.uint8)
    zero = torch.randint(6, 10, (9, 2), generator=g, dtype=torch.int8)
    shifted = codes.to(torch.int8) - zero.repeat_interleave(32, dim=-1)
    shifted = shifted.clamp(-8, 7)
    codes = (shifted + zero.repeat_interleave(32, dim=-1)).to(torch.uint8)
    got = ops.pack_int4(codes.to(cuda), zero.to(cuda), 32).cpu()
    assert torch.equal(got, O.pack_to_int32(shifted, 4))


def test_pack_unpack_round_trip_full_size(cuda):
    """Property at the full down_proj size: unpacking the words gives the codes back."""
    g = torch.Generator(device="cuda").manual_seed(1)
    codes = torch.randint(0, 16, (7168, 2048), generator=g, dtype=torch.uint8, device=cuda)
    words = ops.pack_int4(codes)
    shifts = torch.arange(8, device=cuda, dtype=torch.int32) * 4
    back = ((words.unsqueeze(-1) >> shifts) & 0xF).reshape(7168, 2048).to(torch.uint8)
    assert torch.equal(back, codes)


def test_pack_golden_layers(cuda, golden):
    got = ops.pack_int4(golden.t("qweight").to(cuda)).cpu()
    assert torch.equal(got, golden.t("weight_packed"))


# ------------------------------------------------------------------ dequantize
def test_dequantize_golden(cuda, golden):
    q = golden.t("qweight").to(cuda)
    s = golden.t("scale", typed=True).to(cuda)
    zr = golden.t("zero", typed=True).to(cuda)
    got = ops.dequantize(q, s, zr, golden.group, 4, golden.dtype).cpu()
    assert torch.equal(got.float(), golden.t("dequantized", typed=True).float())
    got2 = ops.dequantize(q, s, None, golden.group, 4, golden.dtype).cpu()
    assert torch.equal(got2.float(), got.float())


def test_relative_error_golden(cuda, golden, precision):
    """get_relative_mse_error on the engine against the number the reference's own function
    returned for the fixture (src/quant_utils.py:259-264)."""
    from moe_quant_b200 import quant_utils
    ops.set_default_precision(precision)
    try:
        deq = golden.t("dequantized", typed=True).float().to(cuda)
        rel = quant_utils.get_relative_mse_error(deq, golden.W.float().to(cuda), golden.t("H_damped").to(cuda))
    finally:
        ops.set_default_precision(ops.Precision())
    want = float(golden.t("rel_error"))
    assert rel.dtype == torch.float32 and rel.dim() == 0
    assert abs(float(rel) - want) <= 2e-4 * want
    plain = quant_utils.get_relative_mse_error(deq, golden.W.float().to(cuda))
    d = deq.cpu() - golden.W.float()
    assert abs(float(plain) - float(d.pow(2).mean() / golden.W.float().pow(2).mean())) <= 1e-5 * float(plain)


# ------------------------------------------------------------------ Hessian
def test_hessian_accum_golden(cuda, golden, precision):
    C = golden.W.shape[1]
    H = torch.zeros(C, C, dtype=torch.float32, device=cuda)
    n = 0
    for k, x in enumerate(golden.batches):
        m = x.shape[0]
        ops.hessian_accum(H, x.to(cuda), n / (n + m), 2.0 / (n + m), precision)
        n += m
        if k == 0 and len(golden.batches) > 1:
            torch.testing.assert_close(H.cpu(), golden.t("H_after0"), rtol=2e-5, atol=1e-5)
    Hc = H.cpu()
    torch.testing.assert_close(Hc, golden.t("H_final"), rtol=2e-5, atol=1e-5)
    assert torch.equal(Hc, Hc.t()), "both triangles must hold the same numbers"


@pytest.mark.parametrize("m,C,dtype", [(1, 128, torch.float32), (37, 256, torch.bfloat16), (513, 384, torch.float16),
                                       (1000, 1024, torch.bfloat16), (300, 2048, torch.float32), (0, 128, torch.bfloat16)])
def test_hessian_accum_ragged(cuda, precision, m, C, dtype):
    x = synthetic.activations(max(m, 1), C, 3, dtype)[:m]
    H0 = synthetic.layer_weight(C, C, 9)
    H0 = (H0 + H0.t()).contiguous()
    H = H0.clone().to(cuda)
    ops.hessian_accum(H, x.to(cuda), 0.25, 0.5, precision)
    want = 0.25 * H0.double() + 0.5 * (x.double().t() @ x.double())
    err = (H.cpu().double() - want).abs().max() / want.abs().max()
    assert float(err) < 5e-6   # tensor-core fp32 accumulation truncates; fp32 FMA path reaches ~3e-7


@pytest.mark.parametrize("pad,offset", [(8, 0), (3, 0), (8, 1), (10, 2)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_hessian_accum_activation_views(cuda, dtype, pad, offset):
    """16-bit activations are read in place through a tensor map when their rows are 16-byte
    aligned (pad 8, offset 0); a row stride that is not a multiple of 8 elements or a start that is
    not 16-byte aligned goes through the transposed copy.  Both must give the same Hessian, with
    ragged token and channel counts."""
    m, C = 333, 1000
    g = torch.Generator().manual_seed(17)
    big = torch.randn(m, C + pad + offset, generator=g).to(dtype)
    xd = big.to(cuda)[:, offset:offset + C]
    assert xd.stride(0) == C + pad + offset and xd.stride(1) == 1
    H0 = synthetic.layer_weight(C, C, 5)
    H0 = (H0 + H0.t()).contiguous()
    H = H0.clone().to(cuda)
    ops.hessian_accum(H, xd, 0.75, 2.0 / m, ops.Precision(math=MATH_TENSOR))
    x = big[:, offset:offset + C].double()
    want = 0.75 * H0.double() + (2.0 / m) * (x.t() @ x)
    Hc = H.cpu()
    assert float((Hc.double() - want).abs().max() / want.abs().max()) < 5e-6
    assert torch.equal(Hc, Hc.t())


# ------------------------------------------------------------------ prepare
def test_prepare_golden(cuda, golden):
    H = golden.t("H_final").clone().to(cuda)
    W = golden.W.float().to(cuda)
    flags = ops.hessian_prepare(H, W, 1e-2).cpu().tolist()
    torch.testing.assert_close(H.cpu(), golden.t("H_damped"), rtol=1e-6, atol=1e-7)
    dead = len(golden.meta.get("dead", ()))
    zero_w = len(golden.meta.get("zero_w", ()))
    assert flags == [0, dead, dead + zero_w, 0]
    for j in golden.meta.get("dead", ()):
        assert float(W[:, j].abs().max()) == 0.0


def test_prepare_nan_hessian_becomes_identity(cuda):
    H = torch.eye(64, device=cuda) * 3
    H[5, 7] = float("nan")
    flags = ops.hessian_prepare(H, None, 0.5).cpu().tolist()
    assert flags[0] == 1
    torch.testing.assert_close(H.cpu(), torch.eye(64) * 1.5)


# ------------------------------------------------------------------ scales
def test_scales_golden(cuda, golden):
    _, Wf, _, _ = O.pre_step(golden.t("H_final").clone(), golden.W)
    got = ops.absmax_scales(Wf.to(cuda), golden.group, 4, golden.dtype).cpu()
    assert torch.equal(got, golden.t("scale", typed=True).float())


@pytest.mark.parametrize("g", [4, 8, 32, 64, 128, 256, 1024])
def test_scales_group_sizes(cuda, g):
    W = synthetic.layer_weight(19, 1024, 4)
    for dt in (torch.float32, torch.bfloat16, torch.float16):
        want, _, _ = O.symmetric_grid(W, g, 4, dt)
        got = ops.absmax_scales(W.to(cuda), g, 4, dt).cpu()
        assert torch.equal(got, want)


# ------------------------------------------------------------------ Hessian inverse factor
def test_hinv_golden(cuda, golden, precision):
    U, flags, _ = ops.hinv_upper(golden.t("H_damped").clone().to(cuda), precision)
    assert flags.cpu().tolist()[3] == 0
    Uc = U.cpu()
    assert float(Uc.tril(-1).abs().max()) == 0.0
    assert torch.equal(Uc.diag(), torch.ones(Uc.shape[0]))
    torch.testing.assert_close(Uc, golden.t("Uhat"), rtol=2e-3, atol=2e-5)


@pytest.mark.parametrize("C", [128, 136, 640, 1000, 1536])
def test_hinv_sizes(cuda, precision, C):
    x = synthetic.activations(C // 2 + 11, C, 21)
    H, _ = O.hessian_update(None, 0, x)
    W = synthetic.layer_weight(8, C, 2)
    want, failed = O.hessian_inverse(H, W, 1e-2)  # damps H in place
    assert not failed
    U, flags, _ = ops.hinv_upper(H.clone().to(cuda), precision)
    assert flags.cpu().tolist()[3] == 0
    rel = (U.cpu() - want).norm() / want.norm()
    assert float(rel) < 2e-4


def test_hinv_not_positive_definite_gives_identity(cuda, precision):
    H = torch.eye(256)
    H[200, 200] = -1.0
    U, flags, _ = ops.hinv_upper(H.to(cuda), precision)
    assert flags.cpu().tolist()[3] == 201
    assert torch.equal(U.cpu(), torch.eye(256))


def test_inv_sym_seam(cuda, precision):
    from moe_quant_b200 import linalg_utils
    x = synthetic.activations(400, 256, 8)
    H, _ = O.hessian_update(None, 0, x)
    H += 0.1 * torch.eye(256)
    got = linalg_utils.inv_sym(H.to(cuda), precision).cpu().double()
    eye = got @ H.double()
    assert float((eye - torch.eye(256, dtype=torch.float64)).abs().max()) < 5e-3


# ------------------------------------------------------------------ sweep
def _grid(golden):
    _, Wf, _, _ = O.pre_step(golden.t("H_final").clone(), golden.W)
    scale, _, _ = O.symmetric_grid(Wf, golden.group, 4, golden.dtype)
    return Wf, scale


def test_sweep_with_reference_factor(cuda, golden, precision):
    Wf, scale = _grid(golden)
    R, C = Wf.shape
    codes, deq = ops.gptq_sweep(Wf.to(cuda), golden.t("Uhat").to(cuda), scale.to(cuda), None, golden.group,
                                C // golden.group, 1, 4, golden.dtype, True, precision)
    assert O.code_agreement(codes.cpu(), golden.t("qweight")) >= 0.999
    want = O.dequantize_linear_weight(codes.cpu(), golden.t("scale", typed=True), golden.t("zero", typed=True))
    assert torch.equal(deq.cpu().float(), want.float())


def test_gptq_loop_seam(cuda, golden, precision):
    """The reference's inner seam: transposed weight, per-element scale and zero."""
    from moe_quant_b200 import gptq_loop
    ops.set_default_precision(precision)
    try:
        Wf, scale = _grid(golden)
        g = golden.group
        sf = scale.repeat_interleave(g, -1)
        zf = torch.full_like(sf, 8.0)
        wt = Wf.t().contiguous().to(cuda)
        q = gptq_loop.gptq_loop(wt, golden.t("Uhat").to(cuda), sf.t().contiguous().to(cuda), zf.t().contiguous().to(cuda),
                                torch.tensor(15.0, device=cuda), golden.dtype, 128)
    finally:
        ops.set_default_precision(ops.Precision())
    assert q.shape == wt.shape and q.dtype == torch.float32
    codes = q.t().contiguous().to(torch.uint8).cpu()
    assert O.code_agreement(codes, golden.t("qweight")) >= 0.999
    deq = O.dequantize_linear_weight(codes, golden.t("scale", typed=True), golden.t("zero", typed=True))
    assert torch.equal(wt.t().cpu().to(golden.dtype).float(), deq.float())


# ------------------------------------------------------------------ argument errors (no fallback, loud failures)
def test_cpu_tensor_is_rejected():
    with pytest.raises(MoeQuantError):
        ops.pack_int4(torch.zeros(4, 8, dtype=torch.uint8))


def test_bad_group_is_rejected(cuda):
    with pytest.raises(MoeQuantError):
        ops.absmax_scales(torch.zeros(4, 96, device=cuda), 64, 4, torch.float32)


# ------------------------------------------------------------------ the GEMM engine alone, against torch fp32
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (128, 128, 64), (130, 257, 128), (300, 1000, 100), (2048, 640, 128),
                                   (257, 129, 1000), (512, 512, 4096)])
@pytest.mark.parametrize("layout", ["nn", "tn", "nt"])
def test_gemm_engine_against_torch(cuda, precision, M, N, K, layout):
    g = torch.Generator().manual_seed(M * 7 + N * 3 + K)
    A = torch.randn(M, K, generator=g)
    B = torch.randn(K, N, generator=g)
    C0 = torch.randn(M, N, generator=g)
    Ad = A.to(cuda) if layout != "tn" else A.t().contiguous().to(cuda).t()     # column-major A
    Bd = B.to(cuda) if layout != "nt" else B.t().contiguous().to(cuda).t()     # column-major B
    Cd = C0.clone().to(cuda)
    ops.gemm(Ad, Bd, Cd, alpha=-0.5, beta=1.0, precision=precision)
    want = C0.double() - 0.5 * (A.double() @ B.double())
    err = float((Cd.cpu().double() - want).abs().max() / want.abs().max())
    # the tensor pipe truncates when it aligns addends, so its error grows ~linearly with K;
    # fp32 FMAs round to nearest and stay near sqrt(K) * 6e-8
    tol = 5e-6 * max(1.0, K / 256.0) if precision.math == MATH_TENSOR else 5e-6
    assert err < tol, f"relative error {err:.3e} (tolerance {tol:.1e})"


def test_gemm_engine_two_plane_split_is_coarser_but_close(cuda):
    g = torch.Generator().manual_seed(9)
    A, B = torch.randn(256, 128, generator=g), torch.randn(128, 384, generator=g)
    want = A.double() @ B.double()
    errs = {}
    for split in (1, 2, 3):
        C = torch.zeros(256, 384, device=cuda)
        ops.gemm(A.to(cuda), B.to(cuda), C, precision=ops.Precision(math=MATH_TENSOR), split=split)
        errs[split] = float((C.cpu().double() - want).abs().max() / want.abs().max())
    assert errs[1] < 2e-2 and errs[2] < 1e-4 and errs[3] < 5e-6
    assert errs[3] < errs[2] < errs[1]


def test_gemm_engine_upper_tiles_only(cuda, precision):
    g = torch.Generator().manual_seed(4)
    P = torch.randn(640, 128, generator=g)
    C0 = torch.randn(640, 640, generator=g)
    Cd = C0.clone().to(cuda)
    Pd = P.to(cuda)
    ops.gemm(Pd, Pd.t(), Cd, alpha=-1.0, beta=1.0, upper_tiles_only=True, precision=precision)
    want = C0.double() - P.double() @ P.double().t()
    got = Cd.cpu().double()
    blocks = torch.arange(640) // 128
    upper = blocks[:, None] <= blocks[None, :]
    assert float((got - want)[upper].abs().max() / want.abs().max()) < 5e-6
    assert torch.equal(got[~upper], C0.double()[~upper]), "tiles below the diagonal must not be touched"


@pytest.mark.parametrize("beta", [0.0, 1.0, 0.5])
@pytest.mark.parametrize("upper,N", [(False, 2780), (False, 2777), (True, 3304)])
@pytest.mark.parametrize("deep", [False, True])
def test_gemm_engine_rank128_update_many_tiles(cuda, beta, upper, N, deep):
    """Rank-128 updates with at least two tiles per SM leave through the TMA unit (store for
    beta 0, add at the L2 for beta 1); any other beta, or fewer tiles, goes through the warps'
    own loads and stores, and so does an N that is not a multiple of 4.  Ragged edges (M, N not
    multiples of the 32-wide boxes) and a C that is a window of a wider matrix must not touch
    anything outside the window.  `deep`: the same with 512 (and a ragged 300) contraction
    columns, the persistent streaming kernel that the two-level updates of the factorisation
    and of the sweep use."""
    M, K = (N, 128) if upper else (2500, 100)
    if deep:
        K = 512 if upper else 300
    g = torch.Generator().manual_seed(11)
    A, B = torch.randn(M, K, generator=g), torch.randn(K, N, generator=g)
    if upper:
        B = A.t().clone()
    big = torch.randn(M + 3, (N + 43) // 4 * 4, generator=g)   # row stride is a multiple of 4 floats
    big_d = big.clone().to(cuda)
    Cd = big_d[2:2 + M, 8:8 + N]                      # 16-byte aligned window of a wider matrix
    ops.gemm(A.to(cuda), B.to(cuda), Cd, alpha=-1.0, beta=beta, upper_tiles_only=upper,
             precision=ops.Precision(math=MATH_TENSOR))
    want = beta * big[2:2 + M, 8:8 + N].double() - A.double() @ B.double()
    got = big_d.cpu()
    win = got[2:2 + M, 8:8 + N].double()
    mask = torch.ones(M, N, dtype=torch.bool)
    if upper:
        blocks_m, blocks_n = torch.arange(M) // 128, torch.arange(N) // 128
        mask = blocks_m[:, None] <= blocks_n[None, :]
        assert torch.equal(win[~mask], big[2:2 + M, 8:8 + N].double()[~mask])
    assert float((win - want)[mask].abs().max() / want.abs().max()) < 5e-6
    outside = torch.ones_like(big, dtype=torch.bool)
    outside[2:2 + M, 8:8 + N] = False
    assert torch.equal(got[outside], big[outside]), "elements outside the C window were modified"


@pytest.mark.parametrize("M,N,K,upper", [(300, 1000, 200, False), (2048, 256, 96, True), (2048, 256, 300, True), (1000, 1000, 64, True),
                                         (129, 257, 1000, False), (4000, 4000, 130, True), (1500, 1500, 4096, True)])
def test_gemm_engine_one_plane_persistent(cuda, M, N, K, upper):
    """One bf16 plane and N >= 256: the persistent kernel (one CTA per SM walking 128 x 256 tiles).
    Inputs are bf16-representable, so one plane is exact and the result must agree with float64 to
    accumulation error; tiles below the diagonal stay untouched with upper_tiles_only, also when the
    matrix has more rows than columns."""
    g = torch.Generator().manual_seed(M + N + K)
    A = torch.randn(M, K, generator=g).to(torch.bfloat16).float()
    B = torch.randn(K, N, generator=g).to(torch.bfloat16).float()
    C0 = torch.randn(M, N, generator=g)
    Cd = C0.clone().to(cuda)
    ops.gemm(A.to(cuda), B.to(cuda), Cd, alpha=0.5, beta=-1.0, upper_tiles_only=upper,
             precision=ops.Precision(math=MATH_TENSOR), split=1)
    want = 0.5 * (A.double() @ B.double()) - C0.double()
    got = Cd.cpu().double()
    must = torch.ones(M, N, dtype=torch.bool)
    if upper:
        # guaranteed: every 128-block on or above the diagonal is computed; nothing below the
        # diagonal's 256-wide tile is touched (K <= 128 runs in the 128 x 128 panel kernel, larger
        # K in 128 x 256 tiles, and what lies between the two tilings may be either)
        must = (torch.arange(N)[None, :] // 128) >= (torch.arange(M)[:, None] // 128)
        never = ((torch.arange(N)[None, :] // 256) * 256 + 256) <= ((torch.arange(M)[:, None] // 128) * 128)
        assert torch.equal(got[never], C0.double()[never])
    assert float((got - want)[must].abs().max() / want.abs().max()) < 5e-6 * max(1.0, K / 256.0)


# ------------------------------------------------------------------ inverse-free form of the sweep
def test_unit_factor_is_inverse_of_reference_factor(cuda, golden, precision):
    H = golden.t("H_damped").clone().to(cuda)
    flags, diag = ops.chol_unit_factor(H, precision)
    assert flags.cpu().tolist()[3] == 0
    Ut = H.cpu().double()
    assert float(Ut.tril(-1).abs().max()) == 0.0 and torch.equal(Ut.diag(), torch.ones(Ut.shape[0], dtype=torch.float64))
    eye = Ut @ golden.t("Uhat").double()
    assert float((eye - torch.eye(Ut.shape[0], dtype=torch.float64)).abs().max()) < 2e-3
    # diag(T)^2 reproduces the pivots: H = Utilde diag(T)^2 Utilde^T
    back = (Ut * diag.cpu().double()[None, :] ** 2) @ Ut.t()
    Hd = golden.t("H_damped").double()
    assert float((back - Hd).abs().max() / Hd.abs().max()) < 1e-5


def test_sweep_inverse_free_form_matches_reference_codes(cuda, golden, precision):
    Wf, scale = _grid(golden)
    R, C = Wf.shape
    Ut = torch.linalg.inv(golden.t("Uhat").double()).float().contiguous()
    codes, deq = ops.gptq_sweep(Wf.clone().to(cuda), Ut.to(cuda), scale.to(cuda), None, golden.group, C // golden.group, 1,
                                4, golden.dtype, True, precision, W_original=Wf.to(cuda))
    assert O.code_agreement(codes.cpu(), golden.t("qweight")) >= 0.999
    want = O.dequantize_linear_weight(codes.cpu(), golden.t("scale", typed=True), golden.t("zero", typed=True))
    assert torch.equal(deq.cpu().float(), want.float())


# ------------------------------------------------------------------ MSE scale search
@pytest.mark.parametrize("R,C,g,dtype", [(64, 512, 128, torch.bfloat16), (40, 256, 32, torch.float16),
                                         (24, 384, 64, torch.float32), (8, 2048, 2048, torch.bfloat16)])
def test_mse_scales_match_oracle(cuda, R, C, g, dtype):
    """The shrink-factor search of src/quant_utils.py:104-139.  The loss sums |.|^2.4 over the
    group in an order the reference leaves open, so a candidate next to the minimum may win on
    one side and not the other: nearly all scales must be identical, every scale must be one of
    the candidates, and its loss must equal the oracle's minimum to rounding."""
    W = synthetic.layer_weight(R, C, 91, dtype).float()
    s0, zero, maxq = O.symmetric_grid(W, g, 4, dtype)
    want = O.mse_scale(W.unflatten(-1, (-1, g)), s0, zero, maxq, dtype)
    got = ops.mse_scales(W.to(cuda), ops.absmax_scales(W.to(cuda), g, 4, dtype), g, 4, dtype).cpu()
    assert float((got == want).float().mean()) >= 0.97
    p = torch.linspace(1, 0.2, 100)
    cands = O.round_fp(s0[..., None] * p, dtype)
    assert bool((cands == got[..., None]).any(-1).all())

    def loss(s):
        Wg = W.unflatten(-1, (-1, g))
        q = torch.clamp(torch.floor((Wg / s[..., None] + 8.0) + 0.5), 0.0, 15.0)
        y = O.round_fp((q - 8.0) * s[..., None], dtype)
        return ((y - Wg).abs().log() * 2.4).exp().sum(-1)

    torch.testing.assert_close(loss(got), loss(want), rtol=1e-3, atol=0)


# ------------------------------------------------------------------ compact launches
@pytest.mark.parametrize("R,C,g,dtype,math", [(200, 512, 128, torch.bfloat16, MATH_TENSOR), (64, 384, 64, torch.float16, MATH_TENSOR),
                                              (333, 640, 32, torch.float32, MATH_TENSOR), (130, 512, 512, torch.bfloat16, MATH_FP32),
                                              (96, 392, 56, torch.float16, MATH_TENSOR), (2500, 256, 64, torch.bfloat16, MATH_TENSOR)])
def test_compact_sweep_is_bit_identical(cuda, R, C, g, dtype, math):
    """MQ_MATH_COMPACT only changes the launch shape of the sweep's full tiles (one weight row per
    thread instead of eight lanes per row): codes, dequantized values, packed words and scales
    must be the same bits, through the whole-layer call and through the sweep alone with zero
    points and the factor of the inverse (the reference's form of the recurrence).  The last case
    (group 56, C = 3 tiles + 8) has no tile the row kernel takes and a narrow last tile.  2500 rows
    are more than the grid of the sixteen-lane shape holds at once: such layers take eight lanes
    per row, and that case is also held to the CPU oracle."""
    W = synthetic.layer_weight(R, C, 3, dtype).to(cuda)
    X = synthetic.activations(2 * C, C, 4, dtype).to(cuda)
    H = torch.zeros(C, C, device=cuda)
    ops.hessian_accum(H, X, 0.0, 2.0 / X.shape[0])
    outs = []
    for compact in (False, True):
        p = ops.Precision(math=math, compact=compact)
        outs.append(ops.quantize_layer([W], H.clone(), g, 4, 1e-2, want_dequantized=True, precision=p, want_packed=True))
    (c0, s0, d0, f0, p0), (c1, s1, d1, f1, p1) = outs
    assert torch.equal(c0[0], c1[0]) and torch.equal(s0[0], s1[0]) and torch.equal(p0[0], p1[0])
    assert torch.equal(d0[0].float(), d1[0].float()) and torch.equal(f0, f1)
    if R > 2368:
        want = O.quantize_layer(W.cpu(), H.cpu().clone(), bits=4, group_size=g, rel_damp=1e-2, block_size=128)
        assert torch.equal(s0[0].cpu(), want["scale"].float())
        assert O.code_agreement(c0[0].cpu(), want["qweight"]) >= CODE_AGREEMENT

    # the sweep alone: factor of the inverse, per-group zero points
    Hd = H.clone()
    ops.hessian_prepare(Hd, W.float(), 1e-2)
    U, _, _ = ops.hinv_upper(Hd, ops.Precision(math=math))
    scale = ops.absmax_scales(W.float(), g, 4, dtype)
    gen = torch.Generator().manual_seed(1)
    zero = torch.randint(6, 11, scale.shape, generator=gen).float().to(cuda)
    res = []
    for compact in (False, True):
        p = ops.Precision(math=math, compact=compact)
        res.append(ops.gptq_sweep(W.float().clone(), U, scale, zero, g, C // g, 1, 4, dtype, True, p))
    assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1].float(), res[1][1].float())
