"""Causal ring attention for MLA heads (q/k dim 192, v dim 128) on the sm_100a kernels.

Same public surface as ``pithtrain/operators/ring_attention/mla.py``: ``ring_mla_attention_func`` (:152),
``RingMLAAttentionFunc`` (:43), ``_online_softmax_combine_log2`` (:27), plus the optional ``sharding``
argument. LSE is kept in the log2 domain as the reference's MLA kernels do.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import _ring
from .sharding import check_sharding


def _online_softmax_combine_log2(out1, lse1, out2, lse2):
    """Merge two partial attention results, log2-domain LSE (reference: mla.py:27-40).

    out: [B, S, H, D] (bf16 or fp32), lse: [B, H, S] fp32. Returns (contiguous fp32 out, fp32 lse).
    """
    from ... import kernels
    return kernels.combine(out1, lse1, out2, lse2, natural=False)


class RingMLAAttentionFunc(torch.autograd.Function):
    """Causal ring MLA attention; ``apply(q, k, v, softmax_scale, cp_rank, cp_size, global_ranks[, sharding])``."""

    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, cp_rank, cp_size, global_ranks, *extra):
        sharding = extra[0] if extra else "contiguous"
        ctx.n_extra = len(extra)
        assert k.is_contiguous() and v.is_contiguous(), "ring MLA attention k or v is not contiguous"
        check_sharding(sharding)
        out, lse = _ring.ring_forward_auto(q, k, v, softmax_scale, cp_rank, cp_size, global_ranks, sharding)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.softmax_scale = softmax_scale
        ctx.cp_rank, ctx.cp_size, ctx.global_ranks, ctx.sharding = cp_rank, cp_size, global_ranks, sharding
        return out

    @staticmethod
    def backward(ctx, dout):
        dout = dout.contiguous()
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = _ring.ring_backward_auto(q, k, v, out, lse, dout, ctx.softmax_scale, ctx.cp_rank, ctx.cp_size,
                                              ctx.global_ranks, ctx.sharding)
        return (dq, dk, dv, None, None, None, None) + (None,) * ctx.n_extra


def ring_mla_attention_func(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float,
                            cp_group: dist.ProcessGroup, sharding: str = "contiguous"):
    """Causal ring MLA attention across context-parallel ranks (reference: mla.py:152-163).

    q/k [B, S_local, H, 192], v [B, S_local, H, 128] bf16 -> out [B, S_local, H, 128] bf16.
    """
    cp_rank = cp_group.rank()
    cp_size = cp_group.size()
    global_ranks = [dist.distributed_c10d.get_global_rank(cp_group, r) for r in range(cp_size)]
    _ring.register_group(global_ranks, cp_group)
    return RingMLAAttentionFunc.apply(q, k, v, softmax_scale, cp_rank, cp_size, global_ranks, sharding)
