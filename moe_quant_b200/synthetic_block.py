"""A small DeepSeek-V3-shaped transformer block with random weights, for driving the GPTQ path
the way quant.py drives the real model (quant.py:243-424).

The real block comes from DeepSeek's remote modelling code, which is not part of the reference
repository.  What matters to the quantization path is reproduced: the module NAMES that
quant.py's regexes select (`self_attn.*_proj`, `mlp.experts.<i>.{gate,up,down}_proj`,
`mlp.shared_experts.*`), one nn.Linear per expert projection, a sigmoid top-k router that sends
each expert a ragged, possibly empty set of tokens, and gate/up projections that see the same
input (so their Hessians can be tied).  Attention itself is replaced by a per-token stand-in
with the MLA projection chain (q_a -> q_b, kv_a -> kv_b, o): no token mixing, no RoPE.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class _RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        v = x.float()
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.eps)
        return (v * self.weight.float()).to(x.dtype)


class _MLP(nn.Module):
    def __init__(self, hidden: int, inter: int):
        super().__init__()
        self.gate_proj = nn.Linear(hidden, inter, bias=False)
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class _Router(nn.Module):
    """Sigmoid scores, top-k; deliberately not an nn.Linear (the reference never quantizes it)."""

    def __init__(self, hidden: int, n_experts: int, top_k: int):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(n_experts, hidden) / hidden ** 0.5)
        self.top_k = top_k
        self.disabled_experts: list = []   # experts that never receive a token (tests of the zero-sample path)

    def forward(self, x):
        scores = torch.sigmoid(x.float() @ self.weight.float().t())
        if self.disabled_experts:
            scores[:, self.disabled_experts] = -1.0
        w, idx = scores.topk(self.top_k, dim=-1)
        return idx, (w / w.sum(-1, keepdim=True)).to(x.dtype)


class _MoE(nn.Module):
    def __init__(self, hidden: int, inter: int, n_experts: int, top_k: int):
        super().__init__()
        self.gate = _Router(hidden, n_experts, top_k)
        self.experts = nn.ModuleList([_MLP(hidden, inter) for _ in range(n_experts)])
        self.shared_experts = _MLP(hidden, inter)

    def forward(self, x):
        flat = x.reshape(-1, x.shape[-1])
        idx, w = self.gate(flat)
        out = torch.zeros_like(flat)
        for e, expert in enumerate(self.experts):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue          # an expert that sees no token never fires its hooks
            out.index_add_(0, tok, expert(flat[tok]) * w[tok, slot].unsqueeze(-1))
        return (out + self.shared_experts(flat)).reshape(x.shape)


class _AttentionStandIn(nn.Module):
    def __init__(self, hidden: int, q_rank: int, kv_rank: int, heads_dim: int):
        super().__init__()
        self.q_a_proj = nn.Linear(hidden, q_rank, bias=False)
        self.q_b_proj = nn.Linear(q_rank, heads_dim, bias=False)
        self.kv_a_proj_with_mqa = nn.Linear(hidden, kv_rank, bias=False)
        self.kv_b_proj = nn.Linear(kv_rank, heads_dim, bias=False)
        self.o_proj = nn.Linear(heads_dim, hidden, bias=False)

    def forward(self, x):
        q = self.q_b_proj(self.q_a_proj(x))
        kv = self.kv_b_proj(self.kv_a_proj_with_mqa(x))
        return self.o_proj(torch.sigmoid(q.float()).to(x.dtype) * kv)


class SyntheticMoEBlock(nn.Module):
    def __init__(self, hidden: int = 256, inter: int = 128, n_experts: int = 8, top_k: int = 2, q_rank: int = 128,
                 kv_rank: int = 128, heads_dim: int = 256, seed: int = 0):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        self.input_layernorm = _RMSNorm(hidden)
        self.self_attn = _AttentionStandIn(hidden, q_rank, kv_rank, heads_dim)
        self.post_attention_layernorm = _RMSNorm(hidden)
        self.mlp = _MoE(hidden, inter, n_experts, top_k)
        for prm in self.parameters():
            if prm.dim() > 1:
                prm.data = torch.randn(prm.shape, generator=gen) * (0.5 / prm.shape[-1] ** 0.5)

    def forward(self, x, **_unused):
        x = x + self.self_attn(self.input_layernorm(x))
        return x + self.mlp(self.post_attention_layernorm(x))
