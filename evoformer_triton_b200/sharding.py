"""Sharding of the MSA-row axis (N_seq) across the GPUs of one node.

Every (b, h, s) slab is an independent attention problem; only the pair-bias gradient
couples the N_seq rows (it is their sum, dsevoformer-triton/evoformer.py:458).  So each rank
runs the unchanged local op on its rows and the job needs exactly one collective: a sum
all-reduce of d(pair_bias) over NCCL.

The reference views ``[B, N_seq, N_res, H, D]`` buffers as ``[B, H, N_seq, N_res, D]``
(evoformer.py:648-650), so "row s" means row s of that *attention view*; slicing axis 1 of
the label shape would hand out something else.  The helpers below slice in the view.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def row_range(n_rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous block of rows owned by ``rank`` (sizes differ by at most one)."""
    base, extra = divmod(n_rows, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_rows(x: torch.Tensor, rank: int, world: int, layout: str = "reinterpret") -> torch.Tensor:
    """Local shard of a ``[B, N_seq, N_res, H, D]`` tensor, again in label shape
    ``[B, rows, N_res, H, D]``, such that the local op sees rows ``row_range(...)`` of
    the global attention view."""
    B, S, R, H, D = x.shape
    s0, s1 = row_range(S, rank, world)
    if layout == "reinterpret":
        return x.reshape(B, H, S, R, D)[:, :, s0:s1].contiguous().reshape(B, s1 - s0, R, H, D)
    return x[:, s0:s1].contiguous()


def unshard_rows(parts: List[torch.Tensor], layout: str = "reinterpret") -> torch.Tensor:
    """Inverse of :func:`shard_rows` over all ranks' results."""
    B, _, R, H, D = parts[0].shape
    if layout == "reinterpret":
        views = [p.reshape(B, H, p.shape[1], R, D) for p in parts]
        full = torch.cat(views, dim=2)
        return full.reshape(B, full.shape[2], R, H, D)
    return torch.cat(parts, dim=1)


def shard_mask(res_mask: Optional[torch.Tensor], rank: int, world: int) -> Optional[torch.Tensor]:
    """Rows of a ``[B, N_seq, 1, 1, N_res]`` mask that belong to ``rank``."""
    if res_mask is None:
        return None
    s0, s1 = row_range(res_mask.shape[1], rank, world)
    return res_mask[:, s0:s1].contiguous()


class _SumGradAcrossRanks(torch.autograd.Function):
    """Identity in forward; sum all-reduce of the gradient in backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        if g.dtype in (torch.bfloat16, torch.float16):  # sum in fp32, never in a 16-bit type
            g32 = g.float()
            dist.all_reduce(g32, op=dist.ReduceOp.SUM, group=ctx.group)
            return g32.to(g.dtype), None
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


def replicate_pair_bias(pair_bias: torch.Tensor, group=None) -> torch.Tensor:
    """Mark a pair bias that every rank holds in full: its gradient is summed over ranks."""
    return _SumGradAcrossRanks.apply(pair_bias, group)


def sharded_evoformer_attention(attn_fn, Q, K, V, res_mask, pair_bias, group=None):
    """Run ``attn_fn`` (``EvoformerAttention.apply`` or a stand-in) on this rank's rows.

    Q, K, V, res_mask are already local shards; pair_bias is the full bias.  Forward needs
    no communication; backward all-reduces d(pair_bias).
    """
    if pair_bias is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        owner = getattr(attn_fn, "__self__", None)
        from . import attention
        if isinstance(owner, type) and issubclass(owner, attention._EvoformerAttentionBase):
            # this package's op: its backward all-reduces the fp32 d(pair_bias) as it leaves the
            # kernel, before the cast to the bias dtype (one collective, no extra conversions, and
            # the local partial sums are never rounded to 16 bits)
            with attention.pair_bias_grad_summed_over(group):
                return attn_fn(Q, K, V, res_mask, pair_bias)
        pair_bias = replicate_pair_bias(pair_bias, group)
    return attn_fn(Q, K, V, res_mask, pair_bias)
