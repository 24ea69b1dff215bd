"""World-size-2 run of the distributed handle on CPU ranks (gloo): Hessian reduction and the
rank-0-computes-then-broadcast protocol of src/gptq.py:138-139, 167-212.  The layer itself is
quantized by the oracle here (there is no device); what is under test is the host protocol."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn as nn

from moe_quant_b200 import GPTQ, synthetic
from oracle import gptq_oracle as O


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, counts, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        R, C = 16, 128
        W = synthetic.layer_weight(R, C, 3, torch.bfloat16)
        X = synthetic.activations(sum(counts), C, 3, torch.bfloat16)
        lo = sum(counts[:rank])
        mine = X[lo: lo + counts[rank]]
        layer = nn.Linear(C, R, bias=False, dtype=torch.bfloat16)
        layer.weight.data = W
        h = GPTQ(layer, 64, True, 1e-2, 128, is_distributed=True)
        h.H, h.num_samples = O.hessian_update(None, 0, mine)

        def oracle_quantize(bits, g):
            res = O.quantize_layer(W, h.H, bits=bits, group_size=g, rel_damp=h.rel_damp, block_size=128)
            return res["qweight"], res["scale"].float()

        h._quantize_default = oracle_quantize          # only rank 0 must ever call this
        if rank != 0:
            def boom(*a):
                raise AssertionError("a non-main rank tried to quantize")
            h._quantize_default = boom
        H_full, _ = O.hessian_update(None, 0, X)
        h.quantization_pre_step()                      # token-weighted all-reduce of H
        ok = torch.tensor([float(torch.allclose(h.H, H_full, rtol=1e-4, atol=1e-5))])
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        ok_h = bool(ok.item())
        q, s, z = h._quantize(4)
        gathered = [torch.empty_like(q) for _ in range(world)]
        dist.all_gather(gathered, q)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        if rank == 0:
            want = O.quantize_layer(W, H_full.clone(), bits=4, group_size=64, block_size=128)
            agree = O.code_agreement(q, want["qweight"])
            torch.save({"same": same, "agree": agree, "ok_h": ok_h, "zero8": bool((z.float() == 8).all()),
                        "dtype": str(s.dtype)}, out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("counts", [(96, 96), (150, 42)])
def test_two_rank_distributed_handle(tmp_path, counts):
    out = str(tmp_path / "r0.pt")
    mp.spawn(_worker, args=(2, _free_port(), counts, out), nprocs=2, join=True)
    res = torch.load(out)
    assert res["ok_h"], "the reduced Hessian differs from the Hessian of all tokens"
    assert res["same"], "ranks ended with different codes"
    assert res["zero8"] and res["dtype"] == "torch.bfloat16"
    # equal shards reproduce the reference's AVG; ragged shards are exact only with token weights
    assert res["agree"] >= 0.995


# ---------------------------------------------------------------------------- owner-rank scheme
def _shared_worker(rank, world, port, counts, out):
    """Five shared layers of different shapes, ragged token counts per rank (one rank holds no
    token at all for the run with a zero count), owner-rank scheme of gptq.quantize_shared."""
    from moe_quant_b200.gptq import quantize_shared, shared_layer_owners
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        shapes = [(16, 128), (24, 64), (8, 192), (32, 64), (12, 256)]
        handles, full_H, weights, calls = [], [], [], []
        for k, (R, C) in enumerate(shapes):
            W = synthetic.layer_weight(R, C, 50 + k, torch.bfloat16)
            X = synthetic.activations(sum(counts), C, 60 + k, torch.bfloat16)
            lo = sum(counts[:rank])
            mine = X[lo: lo + counts[rank]]
            layer = nn.Linear(C, R, bias=False, dtype=torch.bfloat16)
            layer.weight.data = W
            h = GPTQ(layer, 64, True, 1e-2, 128, is_distributed=True)
            if counts[rank] > 0:
                h.H, h.num_samples = O.hessian_update(None, 0, mine)

            def oracle_quantize(bits, g, h=h, W=W, k=k):
                calls.append(k)
                res = O.quantize_layer(W, h.H, bits=bits, group_size=g, rel_damp=h.rel_damp, block_size=128)
                return res["qweight"], res["scale"].float()

            h._quantize_default = oracle_quantize
            handles.append(h)
            weights.append(W)
            full_H.append(O.hessian_update(None, 0, X)[0])
        owners = shared_layer_owners(handles, world)
        results = quantize_shared(handles, 4)
        # only the owner of a layer quantized it, and every rank owns something
        assert sorted(calls) == [k for k in range(len(shapes)) if owners[k] == rank], (rank, calls, owners)
        ok = True
        for k, (q, s, z) in enumerate(results):
            gathered = [torch.empty_like(q) for _ in range(world)]
            dist.all_gather(gathered, q)
            ok &= all(torch.equal(gathered[0], t) for t in gathered)
            gs = [torch.empty_like(s) for _ in range(world)]
            dist.all_gather(gs, s)
            ok &= all(torch.equal(gs[0], t) for t in gs)
            ok &= bool((z.float() == 8).all()) and s.dtype == torch.bfloat16
        agree = []
        for k, (q, s, z) in enumerate(results):
            want = O.quantize_layer(weights[k], full_H[k].clone(), bits=4, group_size=64, block_size=128)
            agree.append(O.code_agreement(q, want["qweight"]))
        flags = [h.has_hessian_issues() for h in handles]
        if rank == 0:
            torch.save({"ok": ok, "agree": agree, "owners": owners, "flags": flags}, out)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("counts", [(96, 96), (150, 42), (0, 200)])
def test_shared_layers_are_quantized_by_owner_ranks(tmp_path, counts):
    out = str(tmp_path / "shared.pt")
    mp.spawn(_shared_worker, args=(2, _free_port(), counts, out), nprocs=2, join=True)
    res = torch.load(out)
    assert res["ok"], "ranks ended with different results"
    assert set(res["owners"]) == {0, 1}
    assert min(res["agree"]) >= 0.995, res["agree"]
    assert not any(res["flags"])


def test_owner_table_balances_cost_and_keeps_tied_handles_together():
    from moe_quant_b200.gptq import shared_layer_owners

    def handle(R, C, tied=None):
        return GPTQ(nn.Linear(C, R, bias=False, device="meta"), 128, True, is_distributed=True, tied_gptq_handle=tied)

    mla = [handle(1536, 7168), handle(24576, 1536), handle(576, 7168), handle(32768, 512), handle(7168, 16384)]
    gate = handle(2048, 7168)
    up = handle(2048, 7168, tied=gate)
    hs = mla + [gate, up, handle(7168, 2048)]
    assert shared_layer_owners(hs, 1) == [0] * 8
    for world in (2, 4, 8):
        owners = shared_layer_owners(hs, world)
        assert owners[5] == owners[6], "a tied handle must live with the owner of its Hessian"
        assert all(0 <= r < world for r in owners)
        assert [r for r in owners].count(owners[4]) == 1 or world == 2, "o_proj dominates: it gets a rank to itself"
    assert len(set(shared_layer_owners(hs, 8))) == 7


# ---------------------------------------------------------------------------- expert-parallel block
def _ep_worker(rank, world, port, out):
    from moe_quant_b200.synthetic_block import SyntheticMoEBlock
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ep = SyntheticMoEBlock(hidden=64, inter=32, n_experts=8, top_k=2, q_rank=32, kv_rank=32, n_heads=2, nope_dim=16,
                               rope_dim=16, v_dim=16, seed=5, expert_parallel=True)
        full = SyntheticMoEBlock(hidden=64, inter=32, n_experts=8, top_k=2, q_rank=32, kv_rank=32, n_heads=2, nope_dim=16,
                                 rope_dim=16, v_dim=16, seed=5)
        xs = [torch.randn(2, 24 + 8 * r, 64, generator=torch.Generator().manual_seed(100 + r)) for r in range(world)]
        local = [i for i, e in enumerate(ep.mlp.experts) if e is not None]
        assert local == list(range(rank * 4, rank * 4 + 4))
        seen = {i: 0 for i in local}
        for i in local:
            ep.mlp.experts[i].gate_proj.register_forward_hook(
                lambda _m, inp, _o, i=i: seen.__setitem__(i, seen[i] + inp[0].shape[0]))
        with torch.no_grad():
            y_ep = ep(xs[rank])
            y_full = full(xs[rank])
            # tokens every rank routes to each expert, from the (identical) router of the full block
            want = torch.zeros(8, dtype=torch.long)
            for x in xs:
                h = x + full.self_attn(full.input_layernorm(x))
                idx, _ = full.mlp.gate(full.post_attention_layernorm(h).reshape(-1, 64))
                want += torch.bincount(idx.reshape(-1), minlength=8)
        ok = torch.allclose(y_ep, y_full, rtol=1e-5, atol=1e-5) and all(seen[i] == int(want[i]) for i in local)
        flag = torch.tensor([float(ok)])
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        if rank == 0:
            torch.save({"ok": bool(flag.item()), "seen": seen, "want": want.tolist()}, out)
    finally:
        dist.destroy_process_group()


def test_expert_parallel_block_routes_tokens_to_the_owning_rank(tmp_path):
    out = str(tmp_path / "ep.pt")
    mp.spawn(_ep_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    res = torch.load(out)
    assert res["ok"], res
