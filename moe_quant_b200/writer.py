"""compressed-tensors writer: the part of pack_quantized_model.py that touches the quantized
layers (pack_quantized_model.py:57-109, 185-203).  Reads the `quantized_weight.pt` files the
quantization loop saved, packs the codes on the GPU and writes one safetensors shard with the
reference's key names, plus the `quantization_config` block that goes into config.json.
"""
from __future__ import annotations

import os
from typing import Dict, Iterable, Optional

import torch
from safetensors.torch import save_file

from .packing import pack_weight


def quantization_config(bits: int, group_size: int, quantize_only_experts: bool = False) -> dict:
    """pack_quantized_model.py:78-109."""
    ignored = ["lm_head"]
    if quantize_only_experts:
        ignored += ["re:.*self_attn.*", "re:.*shared_experts.*", r"re:.*mlp\.(gate|up|gate_up|down)_proj.*"]
    return {
        "config_groups": {
            "group_0": {
                "input_activations": None,
                "output_activations": None,
                "targets": ["Linear"],
                "weights": {
                    "actorder": None, "block_structure": None, "dynamic": False, "group_size": group_size,
                    "num_bits": bits, "observer": "minmax", "observer_kwargs": {}, "strategy": "group",
                    "symmetric": True, "type": "int",
                },
            }
        },
        "format": "pack-quantized",
        "ignore": ignored,
        "kv_cache_scheme": None,
        "quant_method": "compressed-tensors",
        "quantization_status": "compressed",
    }


def pack_saved_layers(quantized_model_path: str, layer_names: Iterable[str], out_file: str, bits: int = 4,
                      group_size: Optional[int] = 128, sym: bool = True,
                      other_tensors: Optional[Dict[str, torch.Tensor]] = None) -> Dict[str, torch.Tensor]:
    """For every layer: <path>/<layer>/quantized_weight.pt -> `<layer>.weight_packed` (int32),
    `<layer>.weight_shape` (int64 [R, C]), `<layer>.weight_scale` (layer dtype)
    [+ `<layer>.weight_zero_point`], written with `other_tensors` (unquantized parameters of the
    block) into one safetensors file.  Returns the state dict that was written."""
    state: Dict[str, torch.Tensor] = dict(other_tensors or {})
    for name in layer_names:
        saved = torch.load(os.path.join(quantized_model_path, name, "quantized_weight.pt"), weights_only=True,
                           map_location="cpu")
        packed = pack_weight(saved, bits, sym, group_size)
        state.pop(f"{name}.weight", None)
        for k, v in packed.items():
            state[f"{name}.{k}"] = v.cpu().contiguous()
    os.makedirs(os.path.dirname(os.path.abspath(out_file)), exist_ok=True)
    save_file(state, out_file)
    return state
