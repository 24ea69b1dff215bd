"""GPTQ handle with the constructor, attributes and methods of src.gptq.GPTQ
(src/gptq.py:22-243), driving the sm_100a engine.

What differs from the reference, by design:
  * `update` feeds the activation batch to the Hessian kernel in its own dtype;
    no fp32 copy of X is made (src/gptq.py:97).
  * `quantize` is one C-ABI call: the NaN / dead-channel / zero-column checks run
    on the device and are read back once, together, after the layer is done.
  * `quantize_tied` quantizes handles that share a Hessian with ONE factorisation;
    the reference refactors the same matrix per tied handle (src/gptq.py:189).
  * distributed handles: the Hessian is summed with token-count weights, so ranks
    may hold different numbers of tokens (the reference's plain AVG, src/gptq.py:139,
    is exact only for equal counts).
"""
from __future__ import annotations

from enum import Enum
import dataclasses
from typing import List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
from torch import Tensor
from torch.nn.modules.conv import _ConvNd

from . import _lib, dist_utils, model_utils, ops
from ._lib import MoeQuantError


class QuantizationOrder(Enum):
    DEFAULT = "default"
    ACTIVATION = "activation"


class GPTQ:
    def __init__(
        self,
        layer: nn.Module,
        group_size: Optional[int] = None,
        sym: bool = False,
        rel_damp: float = 1e-2,
        block_size: Optional[int] = None,
        quantization_order: str = "default",
        quantization_scale: str = "absmax",
        is_distributed: bool = False,
        tied_gptq_handle: Optional["GPTQ"] = None,
        precision: Optional[ops.Precision] = None,
    ):
        self._validate_layer(layer)
        self.layer = layer
        self.W = layer.weight
        self.d_row, self.d_col = model_utils.get_number_of_rows_and_cols(layer)
        self.sym = sym
        self.group_size = group_size
        self.rel_damp = rel_damp
        self.block_size = block_size or self.d_col
        self.quantization_order = QuantizationOrder(quantization_order)
        self.quantization_scale = quantization_scale
        self.W_device = self.W.device
        self.W_dtype = self.W.dtype
        self.W_shape = self.W.shape
        self.H: Optional[Tensor] = None
        self.num_samples = 0
        self.is_distributed = is_distributed
        self.tied_gptq_handle = tied_gptq_handle
        self.num_tied_handles = 0
        if tied_gptq_handle is not None:
            tied_gptq_handle.num_tied_handles += 1
        self.issue_zero_samples = False
        self._nan_hessian = False
        self._non_invertible = False
        self._pending_flags: List[Tensor] = []   # device-side status words not yet read back
        self.precision = precision
        self.pre_step_completed = False
        self._hessian_ready = False   # True once H has been masked and damped
        self._uhat: Optional[Tensor] = None
        self._was_reset = False

    @staticmethod
    def _validate_layer(layer) -> None:
        assert isinstance(layer, (nn.Linear, _ConvNd)), "OBC supports only linear and convolutional layers."

    # The NaN / non-invertible checks run on the device.  Their status words are read back
    # only when one of these attributes is looked at, so quantize() itself never blocks the host.
    def _resolve_flags(self) -> None:
        if not self._pending_flags:
            return
        for flags in self._pending_flags:
            nan, _dead, _zero, not_pd = flags.tolist()
            self._nan_hessian = self._nan_hessian or bool(nan)
            self._non_invertible = self._non_invertible or bool(not_pd)
        device = self._pending_flags[0].device
        self._pending_flags = []
        # The read-back above synchronised with the layer's kernels, so this is the place where an
        # expired device-side wait of the tensor-core kernels shows: the layer's codes are garbage
        # then and must not be saved as if they were a result.
        if device.type == "cuda":
            with torch.cuda.device(device):
                code = _lib.engine_fault()
        else:
            code = _lib.engine_fault()
        if code != 0:
            raise MoeQuantError(
                f"a tensor-core kernel gave up on a bounded wait (code {code}) on {device}: results computed since "
                "are invalid; call moe_quant_b200._lib.engine_fault_clear() before reusing the device")

    @property
    def issue_nan_hessian(self) -> bool:
        self._resolve_flags()
        return self._nan_hessian

    @issue_nan_hessian.setter
    def issue_nan_hessian(self, value: bool) -> None:
        self._nan_hessian = bool(value)

    @property
    def issue_non_invertible(self) -> bool:
        self._resolve_flags()
        return self._non_invertible

    @issue_non_invertible.setter
    def issue_non_invertible(self, value: bool) -> None:
        self._non_invertible = bool(value)

    def has_hessian_issues(self) -> bool:
        return any([self.issue_zero_samples, self.issue_nan_hessian, self.issue_non_invertible])

    # ------------------------------------------------------------------ Hessian
    @torch.no_grad()
    def update(self, input: Tensor) -> None:
        """H <- n/(n+m) H + 2/(n+m) X^T X (src/gptq.py:74-105)."""
        if self.H is None:
            self.H = torch.zeros((self.d_col, self.d_col), device=input.device, dtype=torch.float32)
            self._was_reset = False
        if isinstance(self.layer, nn.Linear):
            x = input.reshape(-1, input.shape[-1])
        else:
            unfold = nn.Unfold(self.layer.kernel_size, dilation=self.layer.dilation, padding=self.layer.padding,
                               stride=self.layer.stride)
            x = unfold(input).transpose(1, 2).flatten(0, 1)
        if x.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            x = x.float()
        m = x.shape[0]
        if m == 0:
            return
        beta = self.num_samples / (self.num_samples + m)
        alpha = 2.0 / (self.num_samples + m)
        ops.hessian_accum(self.H, x, beta, alpha, self.precision)
        self.num_samples += m

    @property
    def tokens_collected(self) -> int:
        return self.num_samples

    def reset(self) -> None:
        """src/gptq.py:111-120.  A Hessian shared with tied handles (and its cached factor) is
        released when the owner and every tied handle have been reset; the reference keeps it
        until the owner object itself is dropped."""
        self.W = self.layer.weight
        owner = self.tied_gptq_handle
        if owner is not None:
            self.H = None
            if not self._was_reset:
                owner.num_tied_handles -= 1
            if owner.num_tied_handles == 0 and owner._was_reset:
                owner._drop_hessian()
        elif self.num_tied_handles == 0:
            self._drop_hessian()
        self._was_reset = True
        self.num_samples = 0
        self.pre_step_completed = False

    def _drop_hessian(self) -> None:
        self.H = None
        self._uhat = None
        self._hessian_ready = False

    # ------------------------------------------------------------------ pre-step
    @torch.no_grad()
    def quantization_pre_step(self) -> None:
        """Host part of src/gptq.py:123-154: Hessian fallback and cross-rank reduction.
        The NaN / dead-channel fixes and the fp32 clone of W happen inside the kernels."""
        reduce_if_needed = True
        if self.H is None:
            if self.tied_gptq_handle is not None:
                self.H = self.tied_gptq_handle.H
            if self.H is None:
                self.H = torch.eye(self.d_col, device=self.W_device, dtype=torch.float32)
                self.issue_zero_samples = True
            reduce_if_needed = False
        if self.is_distributed and reduce_if_needed and dist_utils.is_dist_available_and_initialized():
            self._reduce_hessian()
        self.pre_step_completed = True

    def _reduce_hessian(self) -> None:
        """Token-weighted mean of the per-rank running means.  With equal token counts this
        is the reference's all_reduce(AVG) (src/gptq.py:139)."""
        n = torch.tensor([float(self.num_samples)], device=self.H.device, dtype=torch.float64)
        dist.all_reduce(n, op=dist.ReduceOp.SUM)
        total = float(n.item())
        if total > 0:
            self.H.mul_(self.num_samples / total)
            dist.all_reduce(self.H, op=dist.ReduceOp.SUM)

    # ------------------------------------------------------------------ quantize
    def _group(self) -> int:
        g = self.group_size or self.d_col
        if self.d_col % g != 0:
            raise MoeQuantError(f"group_size {g} does not divide d_col {self.d_col}")
        return g

    def _weight_2d(self) -> Tensor:
        w = self.layer.weight.detach()
        return w.flatten(1, -1) if w.dim() > 2 else w

    def _absorb_flags(self, flags: Tensor) -> None:
        self._pending_flags.append(flags)

    @torch.no_grad()
    def _quantize(self, bits: int) -> Tuple[Tensor, Tensor, Tensor]:
        if not self.sym:
            raise MoeQuantError("only symmetric quantization is implemented (the reference's asymmetric grid is broken)")
        d_row, d_col, device, dtype = self.d_row, self.d_col, self.W_device, self.W_dtype
        g = self._group()
        n_groups = d_col // g
        main = dist_utils.is_main() or not self.is_distributed
        if main:
            if self.quantization_order == QuantizationOrder.ACTIVATION:
                qweight, scale = self._quantize_act_order(bits, g)
            else:
                qweight, scale = self._quantize_default(bits, g)
            scale = scale.to(dtype)
            zero = torch.full_like(scale, (2 ** bits) / 2)
        else:
            qweight = torch.empty(d_row, d_col, device=device, dtype=torch.uint8)
            scale = torch.empty(d_row, n_groups, device=device, dtype=dtype)
            zero = torch.empty(d_row, n_groups, device=device, dtype=dtype)
        if self.is_distributed and dist_utils.is_dist_available_and_initialized():
            dist.barrier()
            dist.broadcast(qweight, src=0)
            dist.broadcast(scale, src=0)
            dist.broadcast(zero, src=0)
        return qweight, scale, zero

    def _mse_search(self) -> bool:
        """True when the scales are refined by the shrink-factor search.  The reference compares
        the stored value with the Enum member (src/quant_utils.py:218), and its driver stores the
        command-line STRING (quant.py:270): "mse" as a string therefore means absmax there, and
        means absmax here.  Passing QuantizationScale.MSE itself switches the search on."""
        from .quant_utils import QuantizationScale
        return self.quantization_scale == QuantizationScale.MSE

    def _quantize_mse(self, bits: int, g: int) -> Tuple[Tensor, Tensor]:
        """Default column order with MSE-refined scales: the stages of the fused entry point one
        by one, with the search between the absmax grid and the sweep."""
        W = self._weight_2d()
        Wf = W.float().contiguous() if W.dtype != torch.float32 else W.clone().contiguous()
        self._prepare_shared_hessian(Wf)
        scale = ops.absmax_scales(Wf, g, bits, self.W_dtype)
        ops.mse_scales(Wf, scale, g, bits, self.W_dtype)
        U = self.H.clone()
        flags, _ = ops.chol_unit_factor(U, self.precision)
        self._absorb_flags(flags)
        codes, _ = ops.gptq_sweep(Wf.clone(), U, scale, None, g, self.d_col // g, 1, bits, self.W_dtype,
                                  precision=self.precision, W_original=Wf)
        return codes, scale

    def _quantize_default(self, bits: int, g: int) -> Tuple[Tensor, Tensor]:
        if self._mse_search():
            return self._quantize_mse(bits, g)
        W = self._weight_2d()
        shares_hessian = self.num_tied_handles > 0 or self.tied_gptq_handle is not None
        if not shares_hessian:
            codes, scales, _, flags = ops.quantize_layer([W], self.H, g, bits, self.rel_damp, precision=self.precision)
            self._hessian_ready = True
            self._absorb_flags(flags)
            return codes[0], scales[0]
        # Handles that share a Hessian and are quantized one call at a time (the reference
        # driver's loop, quant.py:351-387): regularise H once, factor it once, keep the factor
        # until the last of them is reset.
        Wf = W.float().contiguous() if W.dtype != torch.float32 else W.clone().contiguous()
        owner = self.tied_gptq_handle if self.tied_gptq_handle is not None else self
        self._prepare_shared_hessian(Wf)
        if owner._uhat is None:
            owner._uhat, flags, _ = ops.hinv_upper(self.H.clone(), self.precision)
            self._absorb_flags(flags)
        scale = ops.absmax_scales(Wf, g, bits, self.W_dtype)
        codes, _ = ops.gptq_sweep(Wf, owner._uhat, scale, None, g, self.d_col // g, 1, bits, self.W_dtype,
                                  precision=self.precision)
        return codes, scale

    def _prepare_shared_hessian(self, Wf: Tensor) -> None:
        """Masks and damps H exactly once per Hessian: the handle that owns it keeps the flag, and a
        tied handle finds the work done (the reference skips the regularisation for tied handles,
        src/gptq.py:227)."""
        owner = self.tied_gptq_handle if self.tied_gptq_handle is not None else self
        if not owner._hessian_ready:
            flags = ops.hessian_prepare(self.H, Wf, self.rel_damp)
            owner._hessian_ready = True
            self._absorb_flags(flags)
        self._hessian_ready = True

    def _quantize_act_order(self, bits: int, g: int) -> Tuple[Tensor, Tensor]:
        """Activation ordering (src/gptq.py:180-187): columns sorted by decreasing diag(H); each
        column keeps the scale of its original group."""
        W = self._weight_2d()
        Wf = W.float().contiguous() if W.dtype != torch.float32 else W.clone().contiguous()
        self._prepare_shared_hessian(Wf)
        scale = ops.absmax_scales(Wf, g, bits, self.W_dtype)
        if self._mse_search():
            ops.mse_scales(Wf, scale, g, bits, self.W_dtype)
        perm = torch.argsort(self.H.diag(), descending=True)
        Hp = self.H[perm][:, perm].contiguous()
        U, flags, _ = ops.hinv_upper(Hp, self.precision)
        self._absorb_flags(flags)
        Wp = Wf[:, perm].contiguous()
        sp = scale.repeat_interleave(g, dim=-1)[:, perm].contiguous()
        codes_p, _ = ops.gptq_sweep(Wp, U, sp, None, 1, self.d_col, 1, bits, self.W_dtype, precision=self.precision)
        codes = torch.empty_like(codes_p)
        codes[:, perm] = codes_p
        return codes, scale

    def quantize(self, bits: int | float) -> Tuple[Tensor, Tensor, Tensor]:
        self.quantization_pre_step()
        return self._quantize(int(bits))

    @torch.no_grad()
    def quantize_packed(self, bits: int | float) -> dict:
        """quantize(bits) and pack_weight (pack_quantized_model.py:57-75) in one pass: the column
        sweep writes the int32 words of the compressed-tensors layout next to the uint8 codes, so
        the codes are never read back by a packing kernel.  Returns the three tensors of
        quantize() and the three of pack_weight():
            qweight, scale, zero, weight_packed (R, C/8) int32, weight_shape int64 [R, C], weight_scale.
        Handles on another route (tied, distributed, activation order, MSE scales) pack in a
        second pass; the result is the same."""
        bits = int(bits)
        fused = (bits == 4 and self.sym and not self.is_distributed and self.tied_gptq_handle is None
                 and self.num_tied_handles == 0 and self.quantization_order == QuantizationOrder.DEFAULT
                 and not self._mse_search() and self.d_col % 8 == 0)
        self.quantization_pre_step()
        if fused:
            codes, scales, _, flags, packed = ops.quantize_layer([self._weight_2d()], self.H, self._group(), bits,
                                                                 self.rel_damp, precision=self.precision, want_packed=True)
            self._hessian_ready = True
            self._absorb_flags(flags)
            qweight, scale, words = codes[0], scales[0].to(self.W_dtype), packed[0]
            zero = torch.full_like(scale, (2 ** bits) / 2)
        else:
            qweight, scale, zero = self._quantize(bits)
            words = ops.pack_int4(qweight)
        return {"qweight": qweight, "scale": scale, "zero": zero, "weight_packed": words,
                "weight_shape": torch.tensor([self.d_row, self.d_col]), "weight_scale": scale}

    @torch.no_grad()
    def _get_hessian_inverse(self) -> Tensor:
        """Seam of src/gptq.py:220-243: mask, damp (once per Hessian) and factor."""
        Wf = self._weight_2d().float().contiguous()
        self._prepare_shared_hessian(Wf)
        U, flags, _ = ops.hinv_upper(self.H.clone(), self.precision)
        self._absorb_flags(flags)
        return U


_stream_pools: dict = {}


def _side_streams(device: torch.device, n: int):
    key = (device.index if device.index is not None else torch.cuda.current_device())
    pool = _stream_pools.setdefault(key, [])
    while len(pool) < n:
        pool.append(torch.cuda.Stream(device=device))
    return pool[:n]


class compact_launches:
    """While several layers are in flight on different streams, a handle asks the engine for launch
    shapes that occupy few SMs (ops.Precision.compact); the results are the same bits.
    `quantize_many` wraps its calls in this; a caller that spreads `quantize` / `quantize_tied`
    calls over streams of its own uses it the same way (for tied handles, on the owner)."""

    def __init__(self, handle: GPTQ, on: bool = True):
        self.handle, self.on, self.saved = handle, on, None

    def __enter__(self):
        if self.on:
            self.saved = self.handle.precision
            base = ops.DEFAULT_PRECISION if self.saved is None else self.saved
            self.handle.precision = dataclasses.replace(base, compact=True)
        return self

    def __exit__(self, *exc):
        if self.on:
            self.handle.precision = self.saved
        return False


def _tied_groups(handles: Sequence[GPTQ]) -> List[List[int]]:
    """Indices of `handles` grouped by shared Hessian: a handle that owns its Hessian leads the
    handles of the list that are tied to it; a tied handle whose owner is not in the list stands
    alone."""
    groups: List[List[int]] = []
    for i, h in enumerate(handles):
        if h.tied_gptq_handle is None:
            groups.append([i] + [j for j, t in enumerate(handles) if t.tied_gptq_handle is h])
        elif not any(h.tied_gptq_handle is t for t in handles):
            groups.append([i])
    return groups


@torch.no_grad()
def quantize_many(handles: Sequence[GPTQ], bits: int, streams: int = 8) -> List[Tuple[Tensor, Tensor, Tensor]]:
    """Quantizes independent, non-distributed handles (the routed experts of a rank,
    quant.py:351-387) round-robin on `streams` CUDA streams.  One layer's GPTQ is a long chain of
    dependent kernels, many of them too small to fill 148 SMs; chains of different layers have no
    dependency on each other, so running a few side by side fills the machine.  Handles of the
    list that are tied to another handle of the list (gate_proj / up_proj of an expert with
    --tie_gptq_handles) are quantized with it, one factorisation per group (`quantize_tied`).
    Results are the same tensors handle.quantize(bits) returns, in the order of `handles`, ready
    for use on the stream that was current at the call."""
    if not handles:
        return []
    if any(h.is_distributed for h in handles):
        raise MoeQuantError("quantize_many is for non-distributed handles; distributed ones broadcast their results")
    device = handles[0].W_device
    current = torch.cuda.current_stream(device)
    groups = _tied_groups(handles)
    pool = _side_streams(device, max(1, min(streams, len(groups))))
    for s in pool:
        s.wait_stream(current)
    out: List[Optional[Tuple[Tensor, Tensor, Tensor]]] = [None] * len(handles)
    for k, grp in enumerate(groups):
        hs = [handles[i] for i in grp]
        with torch.cuda.stream(pool[k % len(pool)]), compact_launches(hs[0], len(pool) > 1):
            res = quantize_tied(hs, bits) if len(hs) > 1 else [hs[0].quantize(bits)]
        for i, r in zip(grp, res):
            out[i] = r
    for s in pool:
        current.wait_stream(s)
    for res in out:
        for t in res:
            t.record_stream(current)
    return out


@torch.no_grad()
def quantize_tied(handles: Sequence[GPTQ], bits: int) -> List[Tuple[Tensor, Tensor, Tensor]]:
    """Quantizes handles that share one Hessian (gate_proj/up_proj of an expert,
    quant.py:258-262) with a single factorisation.  handles[0] owns H; the others were
    built with tied_gptq_handle=handles[0].  Returns one (qweight, scale, zero) per handle,
    identical to calling handle.quantize(bits) on each in turn."""
    owner = handles[0]
    for h in handles[1:]:
        if h.tied_gptq_handle is not owner:
            raise MoeQuantError("quantize_tied: every handle after the first must be tied to the first")
    if owner.quantization_order != QuantizationOrder.DEFAULT or not owner.sym or any(h._mse_search() for h in handles):
        return [h.quantize(bits) for h in handles]
    owner.quantization_pre_step()
    for h in handles[1:]:
        h.quantization_pre_step()
    if owner.is_distributed and not dist_utils.is_main():
        return [h._quantize(bits) for h in handles]
    g = owner._group()
    codes, scales, _, flags = ops.quantize_layer([h._weight_2d() for h in handles], owner.H, g, int(bits),
                                                 owner.rel_damp, precision=owner.precision)
    owner._hessian_ready = True
    owner._absorb_flags(flags)
    out = []
    for h, q, s in zip(handles, codes, scales):
        h._hessian_ready = True
        if h is not owner:
            h._absorb_flags(flags)
        s = s.to(h.W_dtype)
        z = torch.full_like(s, (2 ** int(bits)) / 2)
        if h.is_distributed and dist_utils.is_dist_available_and_initialized():
            dist.barrier()
            for t in (q, s, z):
                dist.broadcast(t, src=0)
        out.append((q, s, z))
    return out


def shared_layer_owners(handles: Sequence[GPTQ], world: int) -> List[int]:
    """Rank that quantizes each distributed handle.  Handles are dealt out by estimated cost
    (factorisation 2/3 C^3 plus sweep R C^2 flop), largest first, each to the rank with the least
    work so far; a tied handle goes where the handle that owns its Hessian goes.  Depends only on
    shapes and order, so every rank computes the same table."""
    n = len(handles)
    index = {id(h): i for i, h in enumerate(handles)}
    cost = [0.0] * n
    for i, h in enumerate(handles):
        root = index.get(id(h.tied_gptq_handle), i) if h.tied_gptq_handle is not None else i
        c = float(h.d_col)
        cost[root] += (0.0 if root != i else 2.0 / 3.0 * c ** 3) + float(h.d_row) * c * c
    owner = [-1] * n
    load = [0.0] * world
    for i in sorted((i for i in range(n) if cost[i] > 0.0 or handles[i].tied_gptq_handle is None), key=lambda i: (-cost[i], i)):
        if handles[i].tied_gptq_handle is not None and id(handles[i].tied_gptq_handle) in index:
            continue
        r = min(range(world), key=lambda k: (load[k], k))
        owner[i] = r
        load[r] += cost[i]
    for i, h in enumerate(handles):
        if owner[i] < 0:
            owner[i] = owner[index[id(h.tied_gptq_handle)]] if id(h.tied_gptq_handle) in index else 0
    return owner


@torch.no_grad()
def quantize_shared(handles: Sequence[GPTQ], bits: int, streams: int = 4, want_error: bool = False):
    """Quantizes the distributed handles of a block (attention projections, shared experts, dense
    MLPs: the layers every rank sees tokens for) with every rank working.

    The reference all-reduces each Hessian, lets rank 0 quantize one layer after the other while
    the other ranks wait, and broadcasts each result (src/gptq.py:138-139, 167-212).  Here each
    layer has an owner rank (`shared_layer_owners`): its Hessian is REDUCED to the owner with
    token-count weights, owners quantize their layers side by side, and every result is broadcast
    from its owner, so all ranks end with identical (qweight, scale, zero) as the reference
    requires.  The five MLA projections of a DeepSeek block then cost about as much as the
    largest of them instead of their sum.

    Returns [(qweight, scale, zero)] in the order of `handles`; with want_error also the list of
    get_relative_mse_error values (computed by the owner against the reduced, damped Hessian, as
    rank 0 does in quant.py:314-316; None where the Hessian had an issue).
    The issue flags of every handle are set on every rank.
    """
    handles = list(handles)
    bits = int(bits)
    if not handles:
        return ([], []) if want_error else []
    distributed = dist_utils.is_dist_available_and_initialized() and dist_utils.get_world_size() > 1
    world, rank = (dist_utils.get_world_size(), dist_utils.get_rank()) if distributed else (1, 0)
    owners = shared_layer_owners(handles, world)
    device = handles[0].W_device
    roots = [i for i, h in enumerate(handles) if h.tied_gptq_handle is None]

    # ---- Hessians to their owners, weighted by token counts (ranks may hold different numbers)
    if distributed:
        counts = torch.tensor([float(handles[i].num_samples if handles[i].H is not None else 0) for i in roots],
                              dtype=torch.float64, device=device)
        totals = counts.clone()
        dist.all_reduce(totals, op=dist.ReduceOp.SUM)
        totals = totals.tolist()
        for k, i in enumerate(roots):
            h = handles[i]
            total = float(totals[k])
            if total == 0.0:                       # nobody saw a token: identity Hessian (src/gptq.py:129-136)
                h.H = None
                continue
            if h.H is None:
                h.H = torch.zeros(h.d_col, h.d_col, device=device, dtype=torch.float32)
            else:
                h.H.mul_(h.num_samples / total)
            dist.reduce(h.H, dst=owners[i], op=dist.ReduceOp.SUM)
            h.num_samples = int(total)
    for h in handles:
        was_distributed, h.is_distributed = h.is_distributed, False     # the collectives are done here
        try:
            h.quantization_pre_step()
        finally:
            h.is_distributed = was_distributed

    # ---- owners quantize what they own, groups that share a Hessian with one factorisation
    mine = [i for i in range(len(handles)) if owners[i] == rank]
    results: List[Optional[Tuple[Tensor, Tensor, Tensor]]] = [None] * len(handles)
    groups: List[List[int]] = []
    for i in mine:
        h = handles[i]
        if h.tied_gptq_handle is None:
            groups.append([i] + [j for j in mine if handles[j].tied_gptq_handle is h])
        elif not any(h.tied_gptq_handle is handles[j] for j in mine):
            groups.append([i])
    if groups:
        current = torch.cuda.current_stream(device) if device.type == "cuda" else None
        pool = _side_streams(device, max(1, min(streams, len(groups)))) if current is not None else [None]
        for s in pool:
            if s is not None:
                s.wait_stream(current)
        for k, grp in enumerate(groups):
            s = pool[k % len(pool)]
            ctx = torch.cuda.stream(s) if s is not None else _NullContext()
            with ctx:
                hs = [handles[i] for i in grp]
                flags = [h.is_distributed for h in hs]
                for h in hs:
                    h.is_distributed = False
                try:
                    res = quantize_tied(hs, bits) if len(hs) > 1 else [hs[0]._quantize(bits)]
                finally:
                    for h, f in zip(hs, flags):
                        h.is_distributed = f
                for i, r in zip(grp, res):
                    results[i] = r
        if current is not None:
            for s in pool:
                current.wait_stream(s)
            for i in mine:
                for t in results[i]:
                    t.record_stream(current)

    # ---- status and error metric of every layer, then the results, from their owners
    errors: List[Optional[float]] = [None] * len(handles)
    status = torch.zeros(len(handles), 4, dtype=torch.float64, device=device)
    for i in mine:
        h = handles[i]
        status[i, 0], status[i, 1], status[i, 2] = float(h.issue_zero_samples), float(h.issue_nan_hessian), float(h.issue_non_invertible)
        if want_error:
            e = _relative_error(h, results[i])
            status[i, 3] = float("nan") if e is None else e
    if distributed:
        dist.all_reduce(status, op=dist.ReduceOp.SUM)      # every row has exactly one writer
    status = status.cpu()
    pending = []
    for i, h in enumerate(handles):
        h.issue_zero_samples = bool(status[i, 0])
        h._nan_hessian, h._non_invertible = bool(status[i, 1]), bool(status[i, 2])
        e = float(status[i, 3])
        errors[i] = None if (e != e or not want_error) else e
        if results[i] is None:
            g = h._group()
            results[i] = (torch.empty(h.d_row, h.d_col, device=device, dtype=torch.uint8),
                          torch.empty(h.d_row, h.d_col // g, device=device, dtype=h.W_dtype),
                          torch.empty(h.d_row, h.d_col // g, device=device, dtype=h.W_dtype))
        if distributed:
            for t in results[i]:
                pending.append(dist.broadcast(t, src=owners[i], async_op=True))
    for work in pending:
        work.wait()
    return (results, errors) if want_error else results


def _relative_error(h: GPTQ, result) -> Optional[float]:
    from . import quant_utils
    if h.has_hessian_issues() or h.H is None:
        return None
    q, s, z = result
    deq = quant_utils.dequantize_linear_weight(q, s, z)
    return float(quant_utils.get_relative_mse_error(deq.float(), h._weight_2d().float(), h.H))


class _NullContext:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False
