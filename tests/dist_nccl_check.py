"""Two or more GPUs, one process each (torchrun): a distributed (shared-layer) handle over NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29511 tests/dist_nccl_check.py

Every rank accumulates the Hessian of its own slice of the calibration tokens (slices of
different length), `quantize` all-reduces it, rank 0 quantizes, results are broadcast.  Checks:
the reduced Hessian equals the Hessian of all tokens, every rank ends with identical tensors,
and the codes agree with a single-GPU run on all tokens.  Not collected by pytest (it needs
more than one device); the CPU twin of this protocol test is tests/test_dist_gloo.py.
"""
import os
import sys

import torch
import torch.distributed as dist
import torch.nn as nn

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from moe_quant_b200 import GPTQ, synthetic  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("nccl", device_id=dev)
    R, C, N = 512, 1536, 6000
    W = synthetic.layer_weight(R, C, 3, torch.bfloat16).to(dev)
    X = synthetic.activations(N, C, 3, torch.bfloat16).to(dev)
    cuts = [0] + [int(N * (i + 1) ** 1.3 / world ** 1.3) for i in range(world)]   # ragged slices
    mine = X[cuts[rank]: cuts[rank + 1]]

    def handle(distributed):
        layer = nn.Linear(C, R, bias=False, dtype=torch.bfloat16, device=dev)
        layer.weight.data = W.clone()
        return GPTQ(layer, 128, True, 1e-2, 128, is_distributed=distributed)

    h = handle(True)
    h.update(mine)
    full = handle(False)
    full.update(X)
    H_full = full.H.clone()
    h.quantization_pre_step()
    rel = float((h.H - H_full).norm() / H_full.norm())
    q, s, z = h._quantize(4)
    q1, s1, z1 = full.quantize(4)
    gathered = [torch.empty_like(q) for _ in range(world)]
    dist.all_gather(gathered, q)
    same = all(torch.equal(gathered[0], t) for t in gathered)
    agree = float((q == q1).double().mean())
    ok = rel < 1e-4 and same and agree >= 0.995 and torch.equal(s, s1)
    flag = torch.tensor([float(ok)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"world {world}: reduced-H rel err {rel:.2e}, identical on all ranks {same}, "
              f"agreement with single-GPU run {agree:.5f} -> {'OK' if flag.item() else 'FAIL'}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() else 1)


if __name__ == "__main__":
    main()
