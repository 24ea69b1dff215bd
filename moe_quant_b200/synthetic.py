"""Seeded synthetic layers and calibration activations.

Stand-ins for the DeepSeek-V3 weights and the calibration corpora that the
reference streams from disk (quant.py:144-236, src/data_utils.py): weights are
0.02*N(0,1) and activations N(0,1) with one LogNormal(0,1) factor per input
channel, which gives the outlier channels that make GPTQ differ from plain
rounding.  All values come from a CPU ``torch.Generator`` so that a test on any
machine sees the same numbers.
"""
from __future__ import annotations

import torch


def channel_scales(d_col: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed + 7919)
    return torch.exp(torch.randn(d_col, generator=g))


def layer_weight(d_row: int, d_col: int, seed: int, dtype=torch.float32) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return (0.02 * torch.randn(d_row, d_col, generator=g)).to(dtype)


def activations(tokens: int, d_col: int, seed: int, dtype=torch.float32) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed + 104729)
    x = torch.randn(tokens, d_col, generator=g) * channel_scales(d_col, seed)
    return x.to(dtype)


def ragged_expert_counts(tokens: int, experts: int, top_k: int, seed: int) -> torch.Tensor:
    """Token count per routed expert for ``tokens`` tokens sent to their top-k
    experts by a random sigmoid router: the ragged m_e of an expert-parallel
    Hessian pass.  Only the counts are needed to size each expert's batch."""
    g = torch.Generator().manual_seed(seed + 15485863)
    hidden = 64
    x = torch.randn(tokens, hidden, generator=g)
    router = torch.randn(hidden, experts, generator=g) / hidden ** 0.5
    scores = torch.sigmoid(x @ router)
    idx = scores.topk(top_k, dim=-1).indices.reshape(-1)
    return torch.bincount(idx, minlength=experts)
