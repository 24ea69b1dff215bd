"""Generates the golden fixtures in this directory from the reference itself.

Run where the MoE-Quant checkout is available:

    python tests/golden/make_golden.py /path/to/MoE-Quant

The reference's ``src.gptq.GPTQ`` class, ``src.quant_utils`` helpers and
``pack_quantized_model.pack_weight`` are imported UNCHANGED and driven on CPU
tensors.  The one piece that cannot execute without a GPU is the Triton column
sweep (``src/gptq_loop.py``); ``src.gptq_loop.gptq_loop`` is therefore replaced
by the restatement in ``oracle/gptq_oracle.py`` for the duration of the run.
Everything else in the fixtures (Hessians, damped Hessians, the row-normalised
factor, scales, zeros, the transposes and casts at the end of ``_quantize``,
the packed words) is the reference's own arithmetic.  The sweep itself is pinned
separately by ``make_golden_sweep_gpu.py``, which runs the reference's Triton loop
on a GPU over these same fixtures (``sweep_triton.npz``).

The fixtures store inputs as well as outputs, so no random-number generator
has to agree between the machine that wrote them and the one that reads them.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from moe_quant_b200 import synthetic  # noqa: E402
from oracle import gptq_oracle  # noqa: E402

CASES = [
    # name, R, C, tokens (two batches), dtype, group, block, dead cols, zero weight cols
    dict(name="fp32_g128", R=48, C=256, n=(96, 64), dtype="float32", g=128, b=128),
    dict(name="bf16_rankdef", R=64, C=384, n=(100, 60), dtype="bfloat16", g=128, b=128),
    dict(name="fp16_g32_dead", R=33, C=256, n=(200, 120), dtype="float16", g=32, b=128, dead=(5, 130), zero_w=(17,)),
    dict(name="bf16_perchannel", R=40, C=256, n=(300,), dtype="bfloat16", g=256, b=128),
    dict(name="fp16_ragged_block", R=24, C=320, n=(500,), dtype="float16", g=64, b=128),
    dict(name="bf16_g64_fullblock", R=16, C=128, n=(64, 64, 64), dtype="bfloat16", g=64, b=None),
]


def _np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    import transformers  # noqa: F401  (must be imported before accelerate is stubbed)

    if "accelerate" not in sys.modules:
        stub = types.ModuleType("accelerate")
        stub.init_empty_weights = lambda *a, **k: None
        sys.modules["accelerate"] = stub
    import src.gptq as ref_gptq
    import src.gptq_loop as ref_loop
    import src.quant_utils as ref_qu
    import pack_quantized_model as ref_pack

    def sweep_adapter(weight, hessian_inv, scale, qzero, maxq, dtype, gptq_block_size=128):
        return gptq_oracle.gptq_sweep(
            weight.contiguous(), hessian_inv.contiguous(), scale.contiguous(), qzero.contiguous(),
            float(maxq), dtype, gptq_block_size,
        )

    ref_loop.gptq_loop = sweep_adapter

    for case_id, c in enumerate(CASES):
        dtype = getattr(torch, c["dtype"])
        seed = 1000 + case_id
        W = synthetic.layer_weight(c["R"], c["C"], seed, dtype)
        for j in c.get("zero_w", ()):
            W[:, j] = 0
        batches = []
        for k, n in enumerate(c["n"]):
            x = synthetic.activations(n, c["C"], seed + 31 * k, dtype)
            for j in c.get("dead", ()):
                x[:, j] = 0
            batches.append(x)

        layer = nn.Linear(c["C"], c["R"], bias=False, dtype=dtype)
        layer.weight.data = W.clone()
        handle = ref_gptq.GPTQ(layer, c["g"], True, 1e-2, c["b"], "default", "absmax")
        h_steps = []
        for x in batches:
            handle.update(x)
            h_steps.append(handle.H.clone())
        captured = {}
        orig_inv = handle._get_hessian_inverse

        def spy():
            u = orig_inv()
            captured["Uhat"] = u.clone().contiguous()
            return u

        handle._get_hessian_inverse = spy
        qweight, scale, zero = handle.quantize(4)
        deq = ref_qu.dequantize_linear_weight(qweight, scale, zero)
        rel = ref_qu.get_relative_mse_error(deq.float(), W.float(), handle.H)
        packed = ref_pack.pack_weight({"qweight": qweight, "scale": scale, "zero": zero}, 4, True, c["g"])

        out = {
            "W": _np(W),
            "H_final": _np(h_steps[-1]),
            "H_damped": _np(handle.H),
            "Uhat": _np(captured["Uhat"]),
            "qweight": _np(qweight),
            "scale": _np(scale),
            "zero": _np(zero),
            "dequantized": _np(deq),
            "rel_error": np.float64(rel.item()),
            "weight_packed": _np(packed["weight_packed"]),
            "weight_shape": _np(packed["weight_shape"]),
            "tokens": np.int64(handle.tokens_collected),
        }
        for k, x in enumerate(batches):
            out[f"X{k}"] = _np(x)
        if len(batches) > 1:
            out["H_after0"] = _np(h_steps[0])
        meta = dict(c)
        meta["n"] = list(c["n"])
        out["meta"] = np.array(repr(meta))
        np.savez_compressed(os.path.join(HERE, f"{c['name']}.npz"), **out)
        print(f"{c['name']}: rel_error {rel.item():.3e}, codes {tuple(qweight.shape)}")

    # packer-only vectors: odd widths, every nibble value, straight from the installed library
    from compressed_tensors.compressors import pack_to_int32

    g = torch.Generator().manual_seed(77)
    pk = {}
    for R, C in [(3, 8), (5, 13), (2, 1), (7, 64), (4, 100)]:
        v = torch.randint(-8, 8, (R, C), generator=g, dtype=torch.int8)
        pk[f"v_{R}x{C}"] = v.numpy()
        pk[f"p_{R}x{C}"] = pack_to_int32(v, 4).numpy()
    np.savez_compressed(os.path.join(HERE, "pack_int4.npz"), **pk)
    print("pack_int4: done")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python make_golden.py <path to a checkout of IST-DASLab/MoE-Quant>")
    main(sys.argv[1])
