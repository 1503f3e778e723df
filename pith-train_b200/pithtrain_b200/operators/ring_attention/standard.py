"""Causal ring attention for GQA/MHA heads (head_dim 128) on the sm_100a kernels.

Same public surface as ``pithtrain/operators/ring_attention/standard.py``:
``ring_attention_func`` (:192), ``RingAttentionFunc`` (:69), ``_online_softmax_combine`` (:53),
``_ring_send_recv_kv`` (:29). The one addition is the optional ``sharding`` argument
(``"contiguous"``, the reference's layout, by default; ``"zigzag"`` for the load-balanced layout).
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from . import _ring


def _ring_send_recv_kv(send_k: torch.Tensor, send_v: torch.Tensor, next_global: int, prev_global: int):
    """Blocking K/V exchange with the ring neighbours (reference: standard.py:29-50).

    Kept for callers that use it directly; the attention operators overlap their exchanges instead.
    """
    assert send_k.is_contiguous() and send_v.is_contiguous(), (
        "ring attention send_k or send_v is not contiguous"
    )
    recv_k = torch.empty_like(send_k)
    recv_v = torch.empty_like(send_v)
    reqs = dist.batch_isend_irecv([
        dist.P2POp(dist.isend, send_k, next_global),
        dist.P2POp(dist.isend, send_v, next_global),
        dist.P2POp(dist.irecv, recv_k, prev_global),
        dist.P2POp(dist.irecv, recv_v, prev_global),
    ])
    for req in reqs:
        req.wait()
    return recv_k, recv_v


def _online_softmax_combine(out1, lse1, out2, lse2):
    """Merge two partial attention results, natural-log LSE (reference: standard.py:53-66).

    out: [B, S, H, D] (bf16 or fp32), lse: [B, H, S] fp32. Returns (fp32 out, fp32 lse).
    One fused HBM pass on the GPU.
    """
    from ... import kernels
    return kernels.combine(out1, lse1, out2, lse2, natural=True)


class RingAttentionFunc(_ring.RingFunction):
    """Causal ring attention; ``apply(q, k, v, softmax_scale, cp_rank, cp_size, global_ranks[, sharding])``
    (reference: standard.py:69)."""


def ring_attention_func(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float,
                        cp_group: dist.ProcessGroup, sharding: str = "contiguous"):
    """Causal ring attention across context-parallel ranks (reference: standard.py:192-203).

    q [B, S_local, Hq, 128], k/v [B, S_local, Hkv, 128] bf16 -> out [B, S_local, Hq, 128] bf16.
    """
    cp_rank = cp_group.rank()
    cp_size = cp_group.size()
    global_ranks = [dist.distributed_c10d.get_global_rank(cp_group, r) for r in range(cp_size)]
    _ring.register_group(global_ranks, cp_group)
    return RingAttentionFunc.apply(q, k, v, softmax_scale, cp_rank, cp_size, global_ranks, sharding)
