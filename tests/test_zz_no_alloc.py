"""The workspace-free variant of the Hessian preparation step.

Hosts that cannot hand the library scratch memory (a bare C caller, a plug-in inside a process
whose allocator is off limits) use mq_hessian_prepare_noalloc, whose channel lists live in a
static device array.  It must give exactly what mq_hessian_prepare gives, also on a second
call that finds the array dirty from the first.  Collected last on purpose: a run that stops
at the first failure has then already run every other test.
"""
import pytest
import torch

from moe_quant_b200 import _lib, ops, synthetic

pytestmark = pytest.mark.gpu


def _case(C, R, seed, dead, zero_w, dev):
    x = synthetic.activations(C // 2 + 5, C, seed)
    x[:, list(dead)] = 0
    H = (2.0 / x.shape[0]) * (x.t() @ x)
    W = synthetic.layer_weight(R, C, seed)
    W[:, list(zero_w)] = 0
    return H.to(dev), W.to(dev)


def _both(H, W, rel_damp):
    H1, W1 = H.clone(), W.clone()
    f1 = ops.hessian_prepare(H1, W1, rel_damp)                 # existing entry point, caller workspace
    H2, W2 = H.clone(), W.clone()
    f2 = torch.full((4,), -1, dtype=torch.int32, device=H.device)
    ops.hessian_prepare_noalloc(H2, W2, rel_damp, f2)          # new entry point, built-in scratch
    torch.testing.assert_close(H2, H1, rtol=1e-6, atol=1e-7)   # tolerance of test_prepare_golden
    assert torch.equal(W2, W1)
    assert f2.tolist() == f1.tolist()
    return f2.tolist()


def test_noalloc_matches_workspace_variant_twice_in_a_row(cuda):
    # first call: many masked channels, so the built-in lists are left well filled
    H, W = _case(512, 24, 1, dead=(3, 77, 300, 301, 511), zero_w=(10, 11, 12, 200), dev=cuda)
    flags = _both(H, W, 1e-2)
    assert flags == [0, 5, 9, 0]
    # second call straight after it: smaller problem, other channels, must not see stale entries
    H, W = _case(256, 9, 2, dead=(5,), zero_w=(), dev=cuda)
    flags = _both(H, W, 5e-2)
    assert flags == [0, 1, 1, 0]
    # and a clean Hessian: nothing masked although the lists still hold old indices
    H, W = _case(256, 9, 3, dead=(), zero_w=(), dev=cuda)
    assert _both(H, W, 1e-2) == [0, 0, 0, 0]


def test_noalloc_rejects_sizes_beyond_its_scratch(cuda):
    L = _lib.lib()
    flags = torch.zeros(4, dtype=torch.int32, device=cuda)
    H = torch.eye(8, device=cuda)
    before = H.clone()
    # the size check comes first, so a small real buffer is enough to probe it
    rc = L.mq_hessian_prepare_noalloc(H.data_ptr(), 32768 + 8, 32768 + 8, None, 0, 0, 0.01, flags.data_ptr(), None)
    assert rc == 3 and b"32768" in L.mq_last_error()
    torch.cuda.synchronize()
    assert torch.equal(H, before)
