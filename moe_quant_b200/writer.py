"""compressed-tensors writer: the part of pack_quantized_model.py that touches the quantized
layers (pack_quantized_model.py:57-109, 185-203).  Reads the `quantized_weight.pt` files the
quantization loop saved, packs the codes on the GPU and writes one safetensors shard with the
reference's key names, plus the `quantization_config` block that goes into config.json.
"""
from __future__ import annotations

import json
import os
from collections import defaultdict
from typing import Dict, Iterable, Mapping, Optional

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


def pack_model(quantized_model_path: str, packed_model_path: str, num_blocks: int,
               block_tensors: Optional[Mapping[int, Dict[str, torch.Tensor]]] = None,
               head_tensors: Optional[Dict[str, torch.Tensor]] = None,
               tail_tensors: Optional[Dict[str, torch.Tensor]] = None,
               config: Optional[dict] = None, sym: bool = True) -> Dict[str, str]:
    """The output side of pack_quantized_model.py:136-235 for a model whose layers were saved as
    `<quantized_model_path>/model.layers.<i>.<...>/quantized_weight.pt` together with
    `metadata.pt` ({'bits', 'group_size', 'quantize_only_experts'}, quant.py:430-440).

    One shard per transformer block, numbered like the reference (`model-00001` holds the
    embeddings = head_tensors, blocks follow, the last shard holds lm_head and the final norm =
    tail_tensors; `num_blocks + 2` shards in all), `model.safetensors.index.json` with the weight
    map, and `config.json` carrying the `quantization_config` block.  block_tensors[i] are the
    unquantized parameters of block i (norms, router, ...), already in their final dtype; the
    original checkpoint's FP8 ingest is not part of this path.  Returns the weight map."""
    meta = torch.load(os.path.join(quantized_model_path, "metadata.pt"), weights_only=True)
    bits, group_size = int(meta["bits"]), meta["group_size"]
    names = defaultdict(list)
    for layer_name in sorted(os.listdir(quantized_model_path)):
        if os.path.isdir(os.path.join(quantized_model_path, layer_name)):
            names[int(layer_name.split(".")[2])].append(layer_name)          # pack_quantized_model.py:143-146
    os.makedirs(packed_model_path, exist_ok=True)
    n_shards = num_blocks + 2
    index: Dict[str, str] = {}

    def shard(i: int) -> str:
        return f"model-{i:05}-of-{n_shards:05}.safetensors"

    if head_tensors:
        save_file({k: v.contiguous() for k, v in head_tensors.items()}, os.path.join(packed_model_path, shard(1)))
        index.update({k: shard(1) for k in head_tensors})
    for b in range(num_blocks):
        state = pack_saved_layers(quantized_model_path, names.get(b, []), os.path.join(packed_model_path, shard(b + 2)),
                                  bits, group_size, sym, (block_tensors or {}).get(b))
        index.update({k: shard(b + 2) for k in state})
    if tail_tensors:
        save_file({k: v.contiguous() for k, v in tail_tensors.items()}, os.path.join(packed_model_path, shard(n_shards)))
        index.update({k: shard(n_shards) for k in tail_tensors})
    with open(os.path.join(packed_model_path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": index}, f)                  # pack_quantized_model.py:229-230
    cfg = dict(config or {})
    cfg.pop("quantization_config", None)
    cfg["quantization_config"] = quantization_config(bits, group_size, bool(meta.get("quantize_only_experts", False)))
    with open(os.path.join(packed_model_path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    return index
