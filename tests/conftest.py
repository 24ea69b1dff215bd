import ast
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")
GOLDEN_CASES = ["fp32_g128", "bf16_rankdef", "fp16_g32_dead", "bf16_perchannel", "fp16_ragged_block",
                "bf16_g64_fullblock"]


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


class Golden:
    """One fixture file written by tests/golden/make_golden.py."""

    def __init__(self, name):
        z = np.load(os.path.join(GOLDEN, name + ".npz"))
        self.meta = ast.literal_eval(str(z["meta"]))
        self.dtype = getattr(torch, self.meta["dtype"])
        self.name = name
        self._z = z

    def t(self, key, typed=False):
        a = torch.from_numpy(np.array(self._z[key]))
        if typed and self.dtype == torch.bfloat16:
            a = a.view(torch.bfloat16)
        return a

    @property
    def W(self):
        return self.t("W", typed=True)

    @property
    def batches(self):
        return [self.t(f"X{k}", typed=True) for k in range(len(self.meta["n"]))]

    @property
    def group(self):
        return self.meta["g"]

    @property
    def block(self):
        return self.meta["b"]


@pytest.fixture(params=GOLDEN_CASES)
def golden(request):
    return Golden(request.param)


@pytest.fixture
def cuda():
    """Fails (never skips) when there is no device: a GPU test that did not run is not a pass."""
    if not torch.cuda.is_available():
        pytest.fail("this test needs a CUDA device")
    return torch.device("cuda", 0)


@pytest.fixture(autouse=True)
def _engine_health(request):
    """After every GPU test: no bounded device-side wait may have expired."""
    yield
    if request.node.get_closest_marker("gpu") and torch.cuda.is_available():
        from moe_quant_b200 import _lib
        assert _lib.engine_fault() == 0, "a tensor-core kernel gave up on a wait"
