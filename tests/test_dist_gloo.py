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
