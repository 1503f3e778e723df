"""CPU oracle for the q/k RMSNorm + rotary-embedding step in front of attention. TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` leg of ``bench.py`` may import this module; the
shipped operators never do.

What it follows in the reference (paths inside the PithTrain repository):

* ``rms_norm``            — ``nn.RMSNorm(head_dim, eps=rms_norm_eps)`` as constructed at
  ``pithtrain/models/qwen3_30b_a3b.py:381-382`` and applied to ``[B, S, H, head_dim]`` at ``:417-418``:
  ``x * rsqrt(mean(x^2, -1) + eps) * weight``.
* ``rotate_half``         — ``pithtrain/models/qwen3_30b_a3b.py:100-104``.
* ``apply_rotary``        — ``apply_rotary_pos_emb`` (``:107-136``): cos/sin ``[B, S, head_dim]`` broadcast over heads,
  ``x * cos + rotate_half(x) * sin``.
* ``qk_norm_rope``        — the two together, as the attention layer runs them (``:417-421``).
* ``qk_norm_rope_bwd``    — autograd of the above (the reference has no hand-written backward for this step).

Everything is computed in the dtype of the inputs given (tests pass fp32 or fp64), i.e. without the bf16 rounding
the reference takes after each of its elementwise kernels.

Pinning: ``tests/golden/golden_qk_norm_rope.npz`` holds outputs and gradients of the reference's own
``apply_rotary_pos_emb`` and ``torch.nn.RMSNorm`` modules run on CPU in fp32 (``tests/golden/make_golden.py``);
``tests/test_oracle.py`` checks this module against them.
"""

from __future__ import annotations

import torch


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    cos, sin = cos.unsqueeze(2), sin.unsqueeze(2)
    return x * cos + rotate_half(x) * sin


def qk_norm_rope(q, k, q_weight, k_weight, cos, sin, eps: float):
    """(q_embed, k_embed) for q [B,S,Hq,D], k [B,S,Hkv,D], weights [D], cos/sin [B or 1, S, D]."""
    return (apply_rotary(rms_norm(q, q_weight, eps), cos, sin),
            apply_rotary(rms_norm(k, k_weight, eps), cos, sin))


def qk_norm_rope_bwd(q, k, q_weight, k_weight, cos, sin, eps: float, dq_embed, dk_embed):
    """(dq, dk, dq_weight, dk_weight) by autograd through ``qk_norm_rope``."""
    leaves = [t.detach().clone().requires_grad_() for t in (q, k, q_weight, k_weight)]
    qe, ke = qk_norm_rope(leaves[0], leaves[1], leaves[2], leaves[3], cos, sin, eps)
    torch.autograd.backward([qe, ke], [dq_embed, dk_embed])
    return tuple(t.grad for t in leaves)


def rope_tables(positions: torch.Tensor, dim: int, base: float = 1000000.0, dtype=torch.float32):
    """cos/sin ``[1, S, dim]`` for integer positions, as ``Qwen3MoeRotaryEmbedding`` builds them
    (``pithtrain/models/qwen3_30b_a3b.py:54-71``): inv_freq = base^(-2i/dim), emb = cat(freqs, freqs)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    freqs = torch.outer(positions.to(torch.float32), inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype)[None], emb.sin().to(dtype)[None]
