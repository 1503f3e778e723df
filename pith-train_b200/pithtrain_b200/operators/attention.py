"""Single-GPU (CP = 1) causal attention on the sm_100a kernels, registered as ``torch.library`` custom ops
so that it can sit inside a ``torch.compile(fullgraph=True)`` region the way the reference's attention does
(``flash_attn_func`` at pithtrain/models/qwen3_30b_a3b.py:424-430 inside the region compiled at :518; the
Triton MLA op registered at pithtrain/operators/mla/triton.py:445-508).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch


def _kernels():
    from .. import kernels
    return kernels


@torch.library.custom_op("pithtrain_b200::attn_fwd", mutates_args=())
def attn_fwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float,
                causal: bool) -> Tuple[torch.Tensor, torch.Tensor]:
    """(O bf16 [B,Sq,Hq,Dv], LSE fp32 log2-domain [B,Hq,Sq])."""
    K = _kernels()
    if q.is_cuda:  # an anomaly an earlier step reported surfaces here, without a synchronisation
        K.poll_device_status(q.device)
    return K.attn_fwd(q, k, v, softmax_scale, causal, 0)


@attn_fwd_op.register_fake
def _(q, k, v, softmax_scale, causal):
    b, sq, hq, _ = q.shape
    o = torch.empty((b, sq, hq, v.shape[-1]), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((b, hq, sq), dtype=torch.float32, device=q.device)
    return o, lse


@torch.library.custom_op("pithtrain_b200::attn_bwd", mutates_args=())
def attn_bwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, o: torch.Tensor, lse: torch.Tensor,
                do: torch.Tensor, softmax_scale: float, causal: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(dQ, dK, dV) in bf16; fp32 accumulation inside, one rounding at the end."""
    K = _kernels()
    if do.stride(-1) != 1:
        do = do.contiguous()
    delta = K.bwd_preprocess(o, do)
    dk = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
    dv = torch.zeros(v.shape, dtype=torch.float32, device=q.device)
    if q.shape[-1] == 128:  # the dQ pass stores its bf16 result directly
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        K.attn_bwd(q, k, v, do, lse, delta, softmax_scale, causal, 0, None, dk, dv, dq_out=dq)
        K.post_status_copy(q.device)
        return dq, K.cast_to_bf16(dk), K.cast_to_bf16(dv)
    dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    K.attn_bwd(q, k, v, do, lse, delta, softmax_scale, causal, 0, dq, dk, dv)
    K.post_status_copy(q.device)
    return K.cast_to_bf16(dq), K.cast_to_bf16(dk), K.cast_to_bf16(dv)


@attn_bwd_op.register_fake
def _(q, k, v, o, lse, do, softmax_scale, causal):
    return (torch.empty(q.shape, dtype=torch.bfloat16, device=q.device),
            torch.empty(k.shape, dtype=torch.bfloat16, device=q.device),
            torch.empty(v.shape, dtype=torch.bfloat16, device=q.device))


def _setup_context(ctx, inputs, output):
    q, k, v, softmax_scale, causal = inputs
    o, lse = output
    ctx.save_for_backward(q, k, v, o, lse)
    ctx.softmax_scale = softmax_scale
    ctx.causal = causal


def _backward(ctx, grad_o, grad_lse):
    q, k, v, o, lse = ctx.saved_tensors
    dq, dk, dv = attn_bwd_op(q, k, v, o, lse, grad_o, ctx.softmax_scale, ctx.causal)
    return dq, dk, dv, None, None


attn_fwd_op.register_autograd(_backward, setup_context=_setup_context)


def flash_attn_func(q, k, v, dropout_p: float = 0.0, softmax_scale: Optional[float] = None, causal: bool = False,
                    window_size=(-1, -1), softcap: float = 0.0, alibi_slopes=None, deterministic: bool = False,
                    return_attn_probs: bool = False):
    """Stand-in for ``flash_attn.flash_attn_func`` with the arguments PithTrain uses
    (pithtrain/models/qwen3_30b_a3b.py:424-430: ``softmax_scale=..., causal=True``). GQA by head grouping.
    Features the kernels do not have raise instead of being ignored; that includes ``deterministic=True``: dK and
    dV of a GQA group are summed with fp32 atomics, so their last bits depend on the order of arrival.
    The LSE the forward op also returns is an internal by-product: no gradient flows through it.
    """
    if dropout_p != 0.0 or tuple(window_size) != (-1, -1) or softcap != 0.0 or alibi_slopes is not None \
            or return_attn_probs or deterministic:
        raise NotImplementedError("pithtrain_b200.flash_attn_func supports softmax_scale and causal only "
                                  "(no dropout, window, softcap, alibi, attention probabilities or deterministic mode)")
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** -0.5
    o, _ = attn_fwd_op(q, k, v, float(softmax_scale), bool(causal))
    return o
