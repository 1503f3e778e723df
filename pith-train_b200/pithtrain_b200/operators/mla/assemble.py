"""Rotary embedding of q_pe / k_pe and assembly of the MLA operator's inputs in one kernel (and one for the backward).

Stands in for the statements between the projections and the attention operator in the reference's MLA layer
(``pithtrain/models/deepseek_v2_lite.py:446-454`` and the ``value_states.contiguous()`` at ``:463`` / ``:468``):

    q_pe, k_pe = apply_rotary_pos_emb(q_pe, k_pe, cos, sin, position_ids, unsqueeze_dim=2)      # :173-187
    query_states = k_pe.new_empty(bsz, q_len, self.num_heads, self.q_head_dim)
    query_states[:, :, :, : self.qk_nope_head_dim] = q_nope
    query_states[:, :, :, self.qk_nope_head_dim :] = q_pe
    key_states = k_pe.new_empty(bsz, q_len, self.num_heads, self.q_head_dim)
    key_states[:, :, :, : self.qk_nope_head_dim] = k_nope
    key_states[:, :, :, self.qk_nope_head_dim :] = k_pe

which run as about ten elementwise kernels and five copies. Sizes are DeepSeek-V2-Lite's (nope 128, rope 64, v 128);
bf16, CUDA only.
"""

from __future__ import annotations

import torch


class MLAAssembleFunc(torch.autograd.Function):
    """``apply(q, kv, k_pe, cos, sin) -> (query_states, key_states, value_states)`` with cos/sin gathered by position."""

    @staticmethod
    def forward(ctx, q, kv, k_pe, cos, sin):
        from ... import kernels
        query, key, value = kernels.mla_assemble_fwd(q, kv, k_pe, cos, sin)
        ctx.save_for_backward(cos, sin)
        ctx.k_pe_shape = k_pe.shape  # the backward reads no forward data
        return query, key, value

    @staticmethod
    def backward(ctx, dquery, dkey, dvalue):
        from ... import kernels
        cos, sin = ctx.saved_tensors
        dquery, dkey, dvalue = (t if t.stride(-1) == 1 else t.contiguous() for t in (dquery, dkey, dvalue))
        dq, dkv, dk_pe = kernels.mla_assemble_bwd(cos, sin, dquery, dkey, dvalue)
        return dq, dkv, dk_pe.view(ctx.k_pe_shape), None, None


def mla_assemble(q: torch.Tensor, kv: torch.Tensor, k_pe: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                 position_ids: torch.Tensor | None = None):
    """q ``[B,S,H,192]`` = ``[q_nope | q_pe]`` (the projection output, viewed per head), kv ``[B,S,H,256]`` =
    ``[k_nope | v]``, k_pe ``[B,S,1,64]`` or ``[B,S,64]`` (views with a contiguous last dimension are fine).

    cos/sin: either the rotary module's tables ``[max_seq, 64]`` together with ``position_ids`` ``[B,S]`` — exactly
    what the reference hands to ``apply_rotary_pos_emb`` — or tensors already gathered to ``[B or 1, S, 64]``.
    Returns ``(query_states, key_states, value_states)`` ready for ``ring_mla_attention_func`` / ``MLA``.
    """
    if position_ids is not None:
        cos, sin = cos[position_ids], sin[position_ids]
    elif cos.dim() == 2:
        cos, sin = cos[None, : q.shape[1]], sin[None, : q.shape[1]]
    if cos.dtype not in (torch.bfloat16, torch.float32):
        cos, sin = cos.float(), sin.float()
    return MLAAssembleFunc.apply(q, kv, k_pe, cos.contiguous(), sin.contiguous())
