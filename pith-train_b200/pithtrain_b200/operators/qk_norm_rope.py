"""Per-head q/k RMSNorm + rotary position embedding in one kernel (and one for the backward).

Stands in for the three calls the reference's attention layer makes between the projections and the attention
operator (``pithtrain/models/qwen3_30b_a3b.py:417-421``):

    query_states = self.q_norm(query_states)            # nn.RMSNorm(head_dim), :381
    key_states = self.k_norm(key_states)                # nn.RMSNorm(head_dim), :382
    query_states, key_states = apply_rotary_pos_emb(query_states, key_states, cos, sin)   # :107-136

which run as two normalisation kernels and eight elementwise kernels, each rounding to bf16. Here q and k are read
once and written once; the arithmetic is fp32 with a single rounding. head_dim 128, bf16 activations, CUDA only.
"""

from __future__ import annotations

import torch


class QKNormRopeFunc(torch.autograd.Function):
    """``apply(q, k, q_weight, k_weight, cos, sin, eps) -> (q_embed, k_embed)``."""

    @staticmethod
    def forward(ctx, q, k, q_weight, k_weight, cos, sin, eps):
        from .. import kernels
        q_embed, k_embed = kernels.qk_norm_rope_fwd(q, k, q_weight, k_weight, cos, sin, eps)
        ctx.save_for_backward(q, k, q_weight, k_weight, cos, sin)
        ctx.eps = eps
        return q_embed, k_embed

    @staticmethod
    def backward(ctx, dq_embed, dk_embed):
        from .. import kernels
        q, k, q_weight, k_weight, cos, sin = ctx.saved_tensors
        if dq_embed.stride(-1) != 1:
            dq_embed = dq_embed.contiguous()
        if dk_embed.stride(-1) != 1:
            dk_embed = dk_embed.contiguous()
        dq, dk, dwq, dwk = kernels.qk_norm_rope_bwd(q, k, q_weight, k_weight, cos, sin, ctx.eps, dq_embed, dk_embed)
        return dq, dk, dwq.to(q_weight.dtype), dwk.to(k_weight.dtype), None, None, None


def qk_norm_rope(q: torch.Tensor, k: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor,
                 cos: torch.Tensor, sin: torch.Tensor, eps: float):
    """q [B,S,Hq,128], k [B,S,Hkv,128] bf16 (last dimension contiguous; views of the projections are fine),
    weights [128], cos/sin [B or 1, S, 128] as ``Qwen3MoeRotaryEmbedding.forward`` returns them
    (``qwen3_30b_a3b.py:73-97``) -> (q_embed, k_embed) bf16, contiguous."""
    return QKNormRopeFunc.apply(q, k, q_weight, k_weight, cos, sin, float(eps))


def apply_qk_norm_rope(query_states, key_states, q_norm: torch.nn.RMSNorm, k_norm: torch.nn.RMSNorm,
                       position_embeddings):
    """The reference's three calls with its own modules: ``q_norm`` / ``k_norm`` are the layer's ``nn.RMSNorm``
    instances, ``position_embeddings`` the ``(cos, sin)`` pair the layer receives."""
    cos, sin = position_embeddings
    eps = q_norm.eps if q_norm.eps is not None else torch.finfo(query_states.dtype).eps
    if k_norm.eps != q_norm.eps:
        raise ValueError("q_norm and k_norm must share eps")
    return qk_norm_rope(query_states, key_states, q_norm.weight, k_norm.weight, cos, sin, eps)
