"""The per-block loop of quant.py (quant.py:243-424) on top of the B200 GPTQ handles:
hook every nn.Linear, run the calibration inputs through the block to collect Hessians,
quantize the shared layers first and the routed experts second, save the integer results in
the reference's `quantized_weight.pt` format, put the dequantized weights back into the block
and recompute the block's outputs as the next block's inputs.

Differences from the reference loop, all on the throughput side: routed experts are quantized
several at a time on CUDA streams (`quantize_many`), and with `tie_gptq_handles` a gate/up pair
shares one factorisation (`quantize_many` groups tied handles).  The saved tensors are what the reference saves.
"""
from __future__ import annotations

import os
import re
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn
from torch import Tensor

from . import dist_utils, model_utils, quant_utils
from .gptq import GPTQ, quantize_many, quantize_shared

ROUTED_EXPERTS_REGEX = r".*mlp\.experts\.\d+\.(down|gate|up)_proj$"   # quant.py:24


def _save(save_dir: Optional[str], name: str, q: Tensor, s: Tensor, z: Tensor) -> None:
    if not save_dir:
        return
    d = os.path.join(save_dir, name)
    os.makedirs(d, exist_ok=True)
    torch.save({"qweight": q, "scale": s, "zero": z}, os.path.join(d, "quantized_weight.pt"))   # quant.py:321-326


@torch.no_grad()
def quantize_block(
    block: nn.Module,
    inputs: Sequence[Tensor],
    *,
    prefix: str = "",
    bits: int = 4,
    group_size: Optional[int] = 128,
    sym: bool = True,
    rel_damp: float = 1e-2,
    block_size: int = 128,
    quantization_order: str = "default",
    quantization_scale: str = "absmax",
    quantize_only_experts: bool = False,
    tie_gptq_handles: bool = False,
    save_dir: Optional[str] = None,
    log_error: bool = False,
    streams: int = 8,
    forward_kwargs: Optional[dict] = None,
) -> Dict[str, object]:
    """Returns {'outputs': block outputs after quantization (the next block's inputs),
    'layers': names in quantization order, 'issues': {'zero_samples','nan_hessian','non_invertible'},
    'relative_error': {name: float} when log_error}."""
    forward_kwargs = forward_kwargs or {}
    layers = model_utils.select_layers(block, "", ".*", model_utils.LINEAR_LAYERS)
    handles: Dict[str, GPTQ] = {}
    hooks = []

    def make_hook(name):
        def _hook(_module, inp, _out):
            handles[name].update(inp[0])
        return _hook

    for name, layer in layers.items():
        full = f"{prefix}{name}"
        routed = re.search(ROUTED_EXPERTS_REGEX, full) is not None
        if quantize_only_experts and not routed:
            continue
        tied = None
        if tie_gptq_handles and name.endswith("up_proj"):
            tied = handles.get(name.rsplit(".", 1)[0] + ".gate_proj")
        handles[name] = GPTQ(layer, group_size, sym, rel_damp, block_size, quantization_order, quantization_scale,
                             is_distributed=not routed, tied_gptq_handle=tied)
        if tied is None:
            hooks.append(layer.register_forward_hook(make_hook(name)))

    for x in inputs:                                   # Hessian pass, one sequence at a time (quant.py:280-281)
        block(x, **forward_kwargs)
    for h in hooks:
        h.remove()
    dist_utils.barrier()

    shared = [n for n in handles if re.search(ROUTED_EXPERTS_REGEX, f"{prefix}{n}") is None]
    experts = [n for n in handles if n not in shared]
    issues = {"zero_samples": 0, "nan_hessian": 0, "non_invertible": 0}
    rel_err: Dict[str, float] = {}
    order: List[str] = []

    def finish(name: str, result, main_only: bool, error: Optional[float] = None) -> None:
        h = handles[name]
        q, s, z = result
        deq = quant_utils.dequantize_linear_weight(q, s, z)
        if not bool(torch.isfinite(deq).all()):
            raise RuntimeError(f"{prefix}{name} weight is broken after quantization.")      # quant.py:300-302
        issues["zero_samples"] += int(h.issue_zero_samples)
        issues["nan_hessian"] += int(h.issue_nan_hessian)
        issues["non_invertible"] += int(h.issue_non_invertible)
        if log_error and error is not None:
            rel_err[name] = error
        elif log_error and main_only is False and not h.has_hessian_issues() and h.H is not None:
            rel_err[name] = float(quant_utils.get_relative_mse_error(deq.float(), h.layer.weight.float(), h.H))
        # shared layers hold the same result on every rank and are written once (quant.py:321);
        # a routed expert exists on its owner rank only, which writes it itself (quant.py:375-380)
        if dist_utils.is_main() or not main_only:
            _save(save_dir, f"{prefix}{name}", q, s, z)
        h.layer.weight.data = deq.to(h.layer.weight.dtype).reshape(h.layer.weight.shape)     # quant.py:328
        order.append(name)

    # shared layers first (quant.py:295-330).  With several ranks each layer's Hessian is reduced
    # to an owner rank, owners quantize side by side and broadcast (gptq.quantize_shared); the
    # reference lets rank 0 do them one after the other.
    shared_out = quantize_shared([handles[n] for n in shared], bits, streams=streams, want_error=log_error)
    shared_results, shared_errors = shared_out if log_error else (shared_out, [None] * len(shared))
    for name, res, err in zip(shared, shared_results, shared_errors):
        finish(name, res, main_only=True, error=err)
    for name in shared:
        handles[name].reset()

    # routed experts: independent of each other and of other ranks (quant.py:351-387)
    # (with tie_gptq_handles an up_proj handle is tied to its gate_proj: quantize_many gives each
    # such pair one factorisation)
    pending = list(experts)
    results = quantize_many([handles[n] for n in pending], bits, streams=streams)
    for name, res in zip(pending, results):
        finish(name, res, main_only=False)
    for name in experts:
        handles[name].reset()

    outputs = [block(x, **forward_kwargs) for x in inputs]                                   # quant.py:414-416
    for o in outputs:
        if not bool(torch.isfinite(o).all()):
            raise RuntimeError("block outputs are not finite after quantization")
    return {"outputs": outputs, "layers": order, "issues": issues, "relative_error": rel_err}
