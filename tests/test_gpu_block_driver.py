"""The per-block loop (hooks -> Hessians -> shared layers -> routed experts -> save -> write back ->
refresh activations) on a small DeepSeek-shaped MoE block, each layer checked against the oracle
fed with the very activations the hooks saw, then the compressed-tensors shard written from
the saved results."""
import copy
import re
import os

import pytest
import torch
import torch.nn as nn
from safetensors.torch import load_file

from moe_quant_b200 import model_utils
from moe_quant_b200.block_driver import ROUTED_EXPERTS_REGEX, quantize_block
from moe_quant_b200.synthetic_block import SyntheticMoEBlock
from moe_quant_b200.writer import pack_saved_layers, quantization_config
from oracle import gptq_oracle as O

pytestmark = pytest.mark.gpu

CODE_AGREEMENT = 0.995


def _inputs(cuda, n_seq=3, tokens=160, hidden=256):
    g = torch.Generator().manual_seed(11)
    chan = torch.exp(0.5 * torch.randn(hidden, generator=g))
    return [(torch.randn(1, tokens, hidden, generator=g) * chan).to(torch.bfloat16).to(cuda) for _ in range(n_seq)]


def _capture(block, inputs):
    """Inputs of every nn.Linear during the Hessian pass of the unquantized block."""
    seen = {}
    hooks = []
    for name, layer in model_utils.select_layers(block, "", ".*", nn.Linear).items():
        hooks.append(layer.register_forward_hook(
            lambda _m, inp, _o, name=name: seen.setdefault(name, []).append(inp[0].reshape(-1, inp[0].shape[-1]).cpu())))
    with torch.no_grad():
        for x in inputs:
            block(x)
    for h in hooks:
        h.remove()
    return seen


@pytest.mark.parametrize("tie", [False, True])
def test_block_loop_matches_oracle_layer_by_layer(cuda, tmp_path, tie):
    torch.manual_seed(0)
    block = SyntheticMoEBlock(hidden=256, inter=128, n_experts=8, top_k=2, seed=3).to(torch.bfloat16).to(cuda)
    block.mlp.gate.disabled_experts = [5]   # starve one expert
    inputs = _inputs(cuda)
    original = copy.deepcopy(block)
    seen = _capture(original, inputs)
    with torch.no_grad():
        before = [original(x) for x in inputs]
    save_dir = str(tmp_path / "quantized")
    res = quantize_block(block, inputs, prefix="model.layers.3.", bits=4, group_size=128, sym=True, rel_damp=1e-2,
                         block_size=128, tie_gptq_handles=tie, save_dir=save_dir, log_error=True, streams=3)
    layers = model_utils.select_layers(original, "", ".*", nn.Linear)
    assert sorted(res["layers"]) == sorted(layers)
    # shared layers are quantized before any routed expert (quant.py:295, 351)
    first_expert = min(i for i, n in enumerate(res["layers"]) if "experts." in n and "shared" not in n)
    assert all("mlp.experts." not in n for n in res["layers"][:first_expert])
    # the starved expert saw no token: three handles with identity Hessians (untied) or two (tied up_proj reuses gate's)
    assert "mlp.experts.5.gate_proj" not in seen
    assert res["issues"]["zero_samples"] == (2 if tie else 3) and res["issues"]["nan_hessian"] == 0 and res["issues"]["non_invertible"] == 0

    for name, layer in layers.items():
        saved = torch.load(os.path.join(save_dir, "model.layers.3." + name, "quantized_weight.pt"), weights_only=True,
                           map_location="cpu")
        assert set(saved) == {"qweight", "scale", "zero"}
        W = layer.weight.detach().cpu()
        R, C = W.shape
        g = 128 if C % 128 == 0 else C
        assert saved["qweight"].dtype == torch.uint8 and saved["qweight"].shape == (R, C)
        assert saved["scale"].dtype == torch.bfloat16 and saved["scale"].shape == (R, C // 128)
        H = None
        if name in seen:
            n = 0
            for x in seen[name]:
                H, n = O.hessian_update(H, n, x)
        want = O.quantize_layer(W, H, bits=4, group_size=128, rel_damp=1e-2, block_size=128)
        assert torch.equal(saved["scale"].float(), want["scale"].float()), name
        assert O.code_agreement(saved["qweight"], want["qweight"]) >= CODE_AGREEMENT, name
        # the block now carries the dequantized weights
        deq = O.dequantize_linear_weight(saved["qweight"], saved["scale"], saved["zero"])
        live = dict(block.named_modules())[name].weight.detach().cpu()
        assert torch.equal(live.float(), deq.float()), name
    # refreshed activations come from the quantized block and stay close to the original ones
    for o_new, o_old in zip(res["outputs"], before):
        rel = float((o_new.float() - o_old.float()).norm() / o_old.float().norm())
        assert 0.0 < rel < 0.2
    assert all(0.0 < v < 0.1 for v in res["relative_error"].values())

    # ---- writer
    names = ["model.layers.3." + n for n in res["layers"]]
    other = {"model.layers.3.input_layernorm.weight": original.input_layernorm.weight.detach().cpu().contiguous()}
    out = str(tmp_path / "packed" / "model-00001-of-00001.safetensors")
    pack_saved_layers(save_dir, names, out, bits=4, group_size=128, other_tensors=other)
    state = load_file(out)
    for name in names:
        saved = torch.load(os.path.join(save_dir, name, "quantized_weight.pt"), weights_only=True, map_location="cpu")
        ref = O.pack_weight(saved, 4, True, 128)
        assert torch.equal(state[name + ".weight_packed"], ref["weight_packed"])
        assert state[name + ".weight_packed"].dtype == torch.int32
        assert state[name + ".weight_shape"].tolist() == list(saved["qweight"].shape)
        assert torch.equal(state[name + ".weight_scale"].float(), saved["scale"].float())
        assert name + ".weight" not in state
    assert "model.layers.3.input_layernorm.weight" in state
    cfg = quantization_config(4, 128)
    assert cfg["format"] == "pack-quantized" and cfg["config_groups"]["group_0"]["weights"]["num_bits"] == 4

    # ---- whole-model writer: shards per block, index and config (pack_quantized_model.py:136-235)
    import json
    from moe_quant_b200.writer import pack_model
    torch.save({"bits": 4, "group_size": 128, "quantize_only_experts": False}, os.path.join(save_dir, "metadata.pt"))
    packed_dir = str(tmp_path / "packed_model")
    emb = {"model.embed_tokens.weight": torch.randn(32, 256).to(torch.bfloat16)}
    tail = {"lm_head.weight": torch.randn(32, 256).to(torch.bfloat16), "model.norm.weight": torch.ones(256).to(torch.bfloat16)}
    weight_map = pack_model(save_dir, packed_dir, num_blocks=4, block_tensors={3: other}, head_tensors=emb, tail_tensors=tail,
                            config={"model_type": "deepseek_v3", "hidden_size": 256, "quantization_config": {"stale": True}})
    with open(os.path.join(packed_dir, "model.safetensors.index.json")) as f:
        idx = json.load(f)
    assert idx["metadata"] == {} and idx["weight_map"] == weight_map
    assert weight_map["model.embed_tokens.weight"] == "model-00001-of-00006.safetensors"
    assert weight_map["lm_head.weight"] == weight_map["model.norm.weight"] == "model-00006-of-00006.safetensors"
    assert weight_map[names[0] + ".weight_packed"] == "model-00005-of-00006.safetensors"      # block 3 -> shard 3 + 2
    shard = load_file(os.path.join(packed_dir, "model-00005-of-00006.safetensors"))
    assert torch.equal(shard[names[0] + ".weight_packed"], state[names[0] + ".weight_packed"])
    assert set(os.listdir(packed_dir)) >= {f"model-{i:05}-of-00006.safetensors" for i in range(1, 7)}
    with open(os.path.join(packed_dir, "config.json")) as f:
        cfg_file = json.load(f)
    assert cfg_file["model_type"] == "deepseek_v3" and cfg_file["quantization_config"] == quantization_config(4, 128)


def test_routed_expert_regex_matches_reference_names():
    import re
    assert re.search(ROUTED_EXPERTS_REGEX, "model.layers.3.mlp.experts.17.up_proj")
    assert not re.search(ROUTED_EXPERTS_REGEX, "model.layers.3.mlp.shared_experts.up_proj")
    assert not re.search(ROUTED_EXPERTS_REGEX, "model.layers.3.self_attn.o_proj")


def test_non_main_rank_writes_its_experts_but_not_the_shared_layers(cuda, tmp_path, monkeypatch):
    """Shared layers hold the same result on every rank and are written by rank 0 only
    (quant.py:321); a routed expert is written by the rank that quantized it (quant.py:375-380)."""
    from moe_quant_b200 import dist_utils
    block = SyntheticMoEBlock(hidden=256, inter=128, n_experts=4, top_k=2, seed=9).to(torch.bfloat16).to(cuda)
    monkeypatch.setattr(dist_utils, "is_main", lambda: False)
    save_dir = str(tmp_path / "rank1")
    res = quantize_block(block, _inputs(cuda, n_seq=2), prefix="model.layers.0.", save_dir=save_dir, streams=2)
    written = set(os.listdir(save_dir))
    experts = {"model.layers.0." + n for n in res["layers"] if re.search(ROUTED_EXPERTS_REGEX, "model.layers.0." + n)}
    assert experts and written == experts
