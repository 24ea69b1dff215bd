"""Two or more GPUs, one process each (torchrun): a distributed (shared-layer) handle over NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        --master-port 29511 tests/dist_nccl_check.py

Every rank accumulates the Hessian of its own slice of the calibration tokens (slices of
different length).  Part 1, the reference's scheme: `quantize` all-reduces it, rank 0 quantizes,
results are broadcast.  Part 2, the owner-rank scheme (`gptq.quantize_shared`): five layers of
different shapes, each Hessian reduced to its owner, owners quantize side by side, results
broadcast from their owners.  Checks: the reduced Hessian equals the Hessian of all tokens,
every rank ends with identical tensors, and the codes agree with a single-GPU run on all
tokens.  Not collected by pytest (it needs more than one device); the CPU twin of this protocol
test is tests/test_dist_gloo.py.
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

    # ---- part 2: owner-rank scheme on five layers
    from moe_quant_b200.gptq import quantize_shared, shared_layer_owners
    shapes = [(384, 1024), (1024, 512), (192, 1024), (2048, 256), (512, 2048)]
    Ws = [synthetic.layer_weight(r, c, 30 + i, torch.bfloat16).to(dev) for i, (r, c) in enumerate(shapes)]
    Xs = [synthetic.activations(N, c, 40 + i, torch.bfloat16).to(dev) for i, (_, c) in enumerate(shapes)]

    def handles(distributed):
        out = []
        for w in Ws:
            layer = nn.Linear(w.shape[1], w.shape[0], bias=False, dtype=torch.bfloat16, device=dev)
            layer.weight.data = w.clone()
            out.append(GPTQ(layer, 128, True, 1e-2, 128, is_distributed=distributed))
        return out

    hs, ref = handles(True), handles(False)
    for h, r, x in zip(hs, ref, Xs):
        h.update(x[cuts[rank]: cuts[rank + 1]])
        r.update(x)
    owners = shared_layer_owners(hs, world)
    results = quantize_shared(hs, 4)
    ok2 = len(set(owners)) == min(world, len(shapes))
    worst = 1.0
    for (q, s, z), r in zip(results, ref):
        q1, s1, _ = r.quantize(4)
        gathered = [torch.empty_like(q) for _ in range(world)]
        dist.all_gather(gathered, q)
        ok2 &= all(torch.equal(gathered[0], t) for t in gathered) and torch.equal(s, s1)
        worst = min(worst, float((q == q1).double().mean()))
    ok2 &= worst >= 0.995 and not any(h.has_hessian_issues() for h in hs)
    flag2 = torch.tensor([float(ok2)], device=dev)
    dist.all_reduce(flag2, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"world {world}: owner-rank scheme, owners {owners}, worst agreement with single-GPU runs {worst:.5f} "
              f"-> {'OK' if flag2.item() else 'FAIL'}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() and flag2.item() else 1)


if __name__ == "__main__":
    main()
