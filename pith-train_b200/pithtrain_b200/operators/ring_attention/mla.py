"""Causal ring attention for MLA heads (q/k dim 192, v dim 128) on the sm_100a kernels.

Same public surface as ``pithtrain/operators/ring_attention/mla.py``: ``ring_mla_attention_func`` (:152),
``RingMLAAttentionFunc`` (:43), ``_online_softmax_combine_log2`` (:27), plus the optional ``sharding``
argument. LSE is kept in the log2 domain as the reference's MLA kernels do.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import _ring


def _online_softmax_combine_log2(out1, lse1, out2, lse2):
    """Merge two partial attention results, log2-domain LSE (reference: mla.py:27-40).

    out: [B, S, H, D] (bf16 or fp32), lse: [B, H, S] fp32. Returns (contiguous fp32 out, fp32 lse).
    """
    from ... import kernels
    return kernels.combine(out1, lse1, out2, lse2, natural=False)


class RingMLAAttentionFunc(_ring.RingFunction):
    """Causal ring MLA attention; ``apply(q, k, v, softmax_scale, cp_rank, cp_size, global_ranks[, sharding])``
    (reference: mla.py:43). Only the wording of the contiguity check differs from the GQA operator."""

    @staticmethod
    def forward(ctx, q, k, v, *args):
        assert k.is_contiguous() and v.is_contiguous(), "ring MLA attention k or v is not contiguous"
        return _ring.RingFunction.forward(ctx, q, k, v, *args)


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
