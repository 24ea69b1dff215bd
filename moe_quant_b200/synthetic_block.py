"""A small DeepSeek-V3-shaped transformer block with random weights, for driving the GPTQ path
the way quant.py drives the real model (quant.py:243-424).

The real block comes from DeepSeek's remote modelling code, which is not part of the reference
repository.  What matters to the quantization path is reproduced: the module NAMES that
quant.py's regexes select (`self_attn.*_proj`, `mlp.experts.<i>.{gate,up,down}_proj`,
`mlp.shared_experts.*`), one nn.Linear per expert projection, a sigmoid top-k router that sends
each expert a ragged, possibly empty set of tokens, gate/up projections that see the same
input (so their Hessians can be tied), multi-head latent attention with its low-rank
projection chain (q_a -> norm -> q_b, kv_a -> norm -> kv_b, a rotary part shared by all heads,
causal softmax attention, o_proj), and expert parallelism: with `expert_parallel=True` under an
initialised process group each rank keeps only its slice of the routed experts (the others are
None, as with `ep_size` in quant.py:124) and tokens travel to the rank of their expert and back
through two all-to-all exchanges, so a local expert's Hessian sees the tokens of every rank.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
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
    def __init__(self, hidden: int, inter: int, n_experts: int, top_k: int, expert_parallel: bool = False):
        super().__init__()
        self.gate = _Router(hidden, n_experts, top_k)
        self.n_experts = n_experts
        self.ep = bool(expert_parallel) and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
        if self.ep:
            world, rank = dist.get_world_size(), dist.get_rank()
            assert n_experts % world == 0, "experts must divide evenly over the ranks"
            self.per_rank = n_experts // world
            lo = rank * self.per_rank
            local = range(lo, lo + self.per_rank)
        else:
            self.per_rank = n_experts
            local = range(n_experts)
        # every rank builds every expert and drops the ones it does not own, so that expert i has
        # the same weights whatever the number of ranks
        self.experts = nn.ModuleList([_MLP(hidden, inter) for _ in range(n_experts)])
        self._local = set(local)
        self.shared_experts = _MLP(hidden, inter)

    def drop_remote_experts(self) -> None:
        for i in range(self.n_experts):
            if i not in self._local:
                self.experts[i] = None

    def _run_experts(self, tokens, expert_ids):
        out = torch.zeros_like(tokens)
        for e in sorted(self._local):
            rows = (expert_ids == e).nonzero(as_tuple=True)[0]
            if rows.numel() == 0:
                continue          # an expert that sees no token never fires its hooks
            out[rows] = self.experts[e](tokens[rows])
        return out

    def forward(self, x):
        flat = x.reshape(-1, x.shape[-1])
        idx, w = self.gate(flat)
        n, k = idx.shape
        pair_token = torch.arange(n, device=flat.device).repeat_interleave(k)
        pair_expert = idx.reshape(-1)
        pair_weight = w.reshape(-1, 1)
        if not self.ep:
            y = self._run_experts(flat[pair_token], pair_expert)
        else:
            # dispatch: pairs sorted by expert are contiguous per destination rank
            world = dist.get_world_size()
            order = torch.argsort(pair_expert, stable=True)
            send_counts = torch.bincount(pair_expert[order] // self.per_rank, minlength=world)
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts)
            s_in, s_out = send_counts.tolist(), recv_counts.tolist()
            tok_out = flat.new_empty(sum(s_out), flat.shape[1])
            ids_out = pair_expert.new_empty(sum(s_out))
            dist.all_to_all_single(tok_out, flat[pair_token[order]].contiguous(), output_split_sizes=s_out, input_split_sizes=s_in)
            dist.all_to_all_single(ids_out, pair_expert[order].contiguous(), output_split_sizes=s_out, input_split_sizes=s_in)
            y_remote = self._run_experts(tok_out, ids_out)
            # combine: results travel back along the same splits
            y_sorted = flat.new_empty(order.numel(), flat.shape[1])
            dist.all_to_all_single(y_sorted, y_remote, output_split_sizes=s_in, input_split_sizes=s_out)
            y = torch.empty_like(y_sorted)
            y[order] = y_sorted
        out = torch.zeros_like(flat)
        out.index_add_(0, pair_token, y * pair_weight)
        return (out + self.shared_experts(flat)).reshape(x.shape)


def _rotate(x, cos, sin):
    x1, x2 = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


class _MLAttention(nn.Module):
    """Multi-head latent attention with DeepSeek-V3's projection chain: queries through a low-rank
    pair (q_a, q_b), keys and values through a shared latent (kv_a, kv_b) plus one rotary key part
    common to all heads; rotary embedding on the rope slices; causal softmax attention."""

    def __init__(self, hidden: int, q_rank: int, kv_rank: int, n_heads: int, nope_dim: int, rope_dim: int, v_dim: int):
        super().__init__()
        self.n_heads, self.nope, self.rope, self.v_dim, self.kv_rank = n_heads, nope_dim, rope_dim, v_dim, kv_rank
        self.q_a_proj = nn.Linear(hidden, q_rank, bias=False)
        self.q_a_layernorm = _RMSNorm(q_rank)
        self.q_b_proj = nn.Linear(q_rank, n_heads * (nope_dim + rope_dim), bias=False)
        self.kv_a_proj_with_mqa = nn.Linear(hidden, kv_rank + rope_dim, bias=False)
        self.kv_a_layernorm = _RMSNorm(kv_rank)
        self.kv_b_proj = nn.Linear(kv_rank, n_heads * (nope_dim + v_dim), bias=False)
        self.o_proj = nn.Linear(n_heads * v_dim, hidden, bias=False)

    def forward(self, x, position_ids=None):
        B, T, _ = x.shape
        H = self.n_heads
        q = self.q_b_proj(self.q_a_layernorm(self.q_a_proj(x))).view(B, T, H, self.nope + self.rope).transpose(1, 2)
        q_nope, q_pe = q.split([self.nope, self.rope], dim=-1)
        ckv = self.kv_a_proj_with_mqa(x)
        latent, k_pe = ckv.split([self.kv_rank, self.rope], dim=-1)
        kv = self.kv_b_proj(self.kv_a_layernorm(latent)).view(B, T, H, self.nope + self.v_dim).transpose(1, 2)
        k_nope, v = kv.split([self.nope, self.v_dim], dim=-1)
        pos = (torch.arange(T, device=x.device)[None, :] if position_ids is None else position_ids).float()
        inv_freq = 1.0 / (10000.0 ** (torch.arange(0, self.rope, 2, device=x.device).float() / self.rope))
        ang = pos[:, None, :, None] * inv_freq                      # (B or 1, 1, T, rope/2)
        cos, sin = ang.cos().to(x.dtype), ang.sin().to(x.dtype)
        q_pe = _rotate(q_pe, cos, sin)
        k_pe = _rotate(k_pe.view(B, 1, T, self.rope), cos, sin).expand(B, H, T, self.rope)
        attn = F.scaled_dot_product_attention(torch.cat([q_nope, q_pe], -1), torch.cat([k_nope, k_pe], -1), v, is_causal=True)
        return self.o_proj(attn.transpose(1, 2).reshape(B, T, H * self.v_dim))


class SyntheticMoEBlock(nn.Module):
    def __init__(self, hidden: int = 256, inter: int = 128, n_experts: int = 8, top_k: int = 2, q_rank: int = 128,
                 kv_rank: int = 128, n_heads: int = 4, nope_dim: int = 32, rope_dim: int = 32, v_dim: int = 64,
                 seed: int = 0, expert_parallel: bool = False):
        super().__init__()
        gen = torch.Generator().manual_seed(seed)
        self.input_layernorm = _RMSNorm(hidden)
        self.self_attn = _MLAttention(hidden, q_rank, kv_rank, n_heads, nope_dim, rope_dim, v_dim)
        self.post_attention_layernorm = _RMSNorm(hidden)
        self.mlp = _MoE(hidden, inter, n_experts, top_k, expert_parallel)
        for prm in self.parameters():
            if prm.dim() > 1:
                prm.data = torch.randn(prm.shape, generator=gen) * (0.5 / prm.shape[-1] ** 0.5)
        self.mlp.drop_remote_experts()

    def forward(self, x, position_ids=None, **_unused):
        x = x + self.self_attn(self.input_layernorm(x), position_ids)
        return x + self.mlp(self.post_attention_layernorm(x))
