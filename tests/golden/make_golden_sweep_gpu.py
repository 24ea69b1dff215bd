"""Pins the column sweep: runs the reference's own Triton ``gptq_loop`` on a CUDA device.

    python tests/golden/make_golden_sweep_gpu.py /path/to/MoE-Quant [output directory]

Needs a GPU, triton and a checkout of IST-DASLab/MoE-Quant; writes ``sweep_triton.npz``.
``make_golden.py`` (CPU only) has to replace ``src.gptq_loop.gptq_loop`` by the oracle's
restatement, so the codes in its fixtures are the oracle's.  This script closes that gap: every
number it stores comes out of the reference's modules imported UNCHANGED and run on the device,

  * ``<case>.sweep_codes``: ``src.gptq_loop.gptq_loop`` (the captured Triton loop plus
    ``addmm_``) on the inputs of the CPU fixture ``<case>.npz`` (its weight after the pre-step,
    its ``Uhat``, its scales), so the sweep is checked in isolation;
  * ``<case>.qweight`` / ``<case>.scale``: the whole ``src.gptq.GPTQ`` handle on the device
    (cuBLAS Hessian, cuSOLVER factorisations, Triton sweep) fed with the fixture's batches;
  * ``mid_*``: two larger layers (several GPTQ blocks, hundreds of tokens) whose inputs are
    stored here as well, with the handle's ``Uhat`` so that the sweep can be replayed alone;
  * ``mse_*``: ``src.quant_utils.get_quantization_grid`` with ``QuantizationScale.MSE`` (the
    Triton shrink-factor search, which the reference's own handle never reaches because it
    compares a string with the Enum) on three small weight matrices stored alongside.

The reference passes ``torch.empty(0, dtype=...)`` to its kernel for the rounding dtype
(``src/gptq_loop.py:62``); nothing is changed about that.
"""
from __future__ import annotations

import ast
import os
import sys

import numpy as np
import torch
import torch.nn as nn

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from moe_quant_b200 import synthetic  # noqa: E402

CPU_CASES = ["fp32_g128", "bf16_rankdef", "fp16_g32_dead", "bf16_perchannel", "fp16_ragged_block",
             "bf16_g64_fullblock"]
MID_CASES = [
    dict(name="mid_bf16_g128", R=96, C=512, n=700, dtype="bfloat16", g=128, b=128, seed=2101),
    dict(name="mid_fp16_g64", R=64, C=384, n=300, dtype="float16", g=64, b=128, seed=2102),
]


def _np(t: torch.Tensor) -> np.ndarray:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


def _load(name):
    z = np.load(os.path.join(HERE, name + ".npz"))
    meta = ast.literal_eval(str(z["meta"]))
    dtype = getattr(torch, meta["dtype"])

    def t(key, typed=False):
        a = torch.from_numpy(np.array(z[key]))
        return a.view(torch.bfloat16) if typed and dtype == torch.bfloat16 else a

    return meta, dtype, t


def main(ref_root: str, out_dir: str) -> None:
    if not torch.cuda.is_available():
        raise SystemExit("this generator needs a CUDA device (the reference's sweep is Triton-only)")
    sys.path.insert(0, ref_root)
    import src.gptq as ref_gptq
    import src.gptq_loop as ref_loop

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    out = {}

    def sweep_alone(Wf, Uhat, scale_rg, group, dtype, block):
        """codes (R, C) uint8 from the reference's gptq_loop on transposed inputs (src/gptq.py:191-199)."""
        R, C = Wf.shape
        scale = scale_rg.float().repeat_interleave(group, dim=-1)
        zero = torch.full_like(scale, 8.0)
        q = ref_loop.gptq_loop(
            weight=Wf.t().contiguous().to(dev), hessian_inv=Uhat.contiguous().to(dev),
            scale=scale.t().contiguous().to(dev), qzero=zero.t().contiguous().to(dev),
            maxq=torch.tensor(15.0, device=dev), dtype=dtype, gptq_block_size=block or C)
        return q.t().contiguous().to(torch.uint8).cpu()

    def handle_on_device(W, batches, group, block):
        layer = nn.Linear(W.shape[1], W.shape[0], bias=False, dtype=W.dtype, device=dev)
        layer.weight.data = W.clone().to(dev)
        handle = ref_gptq.GPTQ(layer, group, True, 1e-2, block, "default", "absmax")
        for x in batches:
            handle.update(x.to(dev))
        captured = {}
        orig = handle._get_hessian_inverse

        def spy():
            u = orig()
            captured["Uhat"] = u.clone().contiguous()
            return u

        handle._get_hessian_inverse = spy
        q, s, z = handle.quantize(4)
        return q.cpu(), s.cpu(), z.cpu(), captured["Uhat"].cpu()

    for name in CPU_CASES:
        meta, dtype, t = _load(name)
        W = t("W", typed=True)
        Wf = W.float()
        dead = torch.diag(t("H_final")) == 0
        Wf[:, dead] = 0
        out[f"{name}.sweep_codes"] = _np(sweep_alone(Wf, t("Uhat"), t("scale", typed=True), meta["g"], dtype, meta["b"]))
        batches = [t(f"X{k}", typed=True) for k in range(len(meta["n"]))]
        q, s, _z, _u = handle_on_device(W, batches, meta["g"], meta["b"])
        out[f"{name}.qweight"] = _np(q)
        out[f"{name}.scale"] = _np(s)
        agree = float((q == t("qweight")).float().mean())
        print(f"{name}: device handle vs CPU fixture codes {agree:.5f}; sweep alone vs CPU fixture "
              f"{float((torch.from_numpy(out[f'{name}.sweep_codes']) == t('qweight')).float().mean()):.5f}")

    for c in MID_CASES:
        dtype = getattr(torch, c["dtype"])
        W = synthetic.layer_weight(c["R"], c["C"], c["seed"], dtype)
        X = synthetic.activations(c["n"], c["C"], c["seed"], dtype)
        q, s, _z, U = handle_on_device(W, [X], c["g"], c["b"])
        codes = sweep_alone(W.float(), U, s, c["g"], dtype, c["b"])
        n = c["name"]
        out[f"{n}.W"], out[f"{n}.X"], out[f"{n}.Uhat"] = _np(W), _np(X), _np(U)
        out[f"{n}.qweight"], out[f"{n}.scale"], out[f"{n}.sweep_codes"] = _np(q), _np(s), _np(codes)
        out[f"{n}.meta"] = np.array(repr(c))
        print(f"{n}: handle vs its own sweep replayed alone {float((q == codes).float().mean()):.5f}")

    import src.quant_utils as ref_qu
    for k, (R, C, g, dname) in enumerate([(24, 256, 128, "bfloat16"), (16, 256, 32, "float16"), (12, 192, 64, "float32")]):
        dtype = getattr(torch, dname)
        W = synthetic.layer_weight(R, C, 2300 + k, dtype)
        scale, zero, maxq = ref_qu.get_quantization_grid(W.float().to(dev), g, 4, True, dtype, ref_qu.QuantizationScale.MSE)
        base, _, _ = ref_qu.get_quantization_grid(W.float().to(dev), g, 4, True, dtype, ref_qu.QuantizationScale.ABSMAX)
        n = f"mse_{dname}_g{g}"
        out[f"{n}.W"] = _np(W)
        out[f"{n}.scale"] = _np(scale[:, ::g].contiguous())
        out[f"{n}.scale_absmax"] = _np(base[:, ::g].contiguous())
        out[f"{n}.meta"] = np.array(repr(dict(R=R, C=C, g=g, dtype=dname)))
        print(f"{n}: mean shrink {float((scale / base).mean()):.4f}")

    out["environment"] = np.array(repr({"torch": torch.__version__, "device": torch.cuda.get_device_name(0),
                                        "triton": __import__("triton").__version__}))
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "sweep_triton.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        raise SystemExit("usage: python make_golden_sweep_gpu.py <path to a checkout of IST-DASLab/MoE-Quant> [out dir]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) == 3 else HERE)
