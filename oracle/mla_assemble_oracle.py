"""CPU oracle for the rotary embedding + input assembly in front of the MLA attention operator. TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` leg of ``bench.py`` may import this module; the
shipped operators never do.

What it follows in the reference (paths inside the PithTrain repository):

* ``rotate_half``          — ``pithtrain/models/deepseek_v2_lite.py:165-169``.
* ``apply_rotary_deepseek``— ``apply_rotary_pos_emb`` (``:173-187``) as called with ``unsqueeze_dim=2`` at ``:446``: the
  last dimension is de-interleaved (``view(..., d//2, 2).transpose(-1, -2).reshape(..., d)``), then
  ``x * cos + rotate_half(x) * sin`` with cos/sin gathered by position and broadcast over heads.
* ``mla_assemble``         — the attention layer's assembly (``:426-454``, ``:463``): split q into nope/rope parts, split
  kv into k_nope / v, rotate q_pe and k_pe, concatenate ``[q_nope | q_pe]`` and ``[k_nope | k_pe (broadcast over
  heads)]``, value made contiguous.
* ``mla_assemble_bwd``     — autograd of the above (the reference has no hand-written backward for this step).

Pinning: ``tests/golden/golden_mla_assemble.npz`` holds outputs and gradients produced with the reference's own
``apply_rotary_pos_emb`` and ``DeepseekV2LiteYarnRotaryEmbedding`` on CPU in fp32 (``tests/golden/make_golden.py``);
``tests/test_oracle.py`` checks this module against them.
"""

from __future__ import annotations

import torch


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    half = x.shape[-1] // 2
    return torch.cat((-x[..., half:], x[..., :half]), dim=-1)


def apply_rotary_deepseek(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B,S,H,d] with interleaved pairs, cos/sin [B or 1, S, d] already gathered by position."""
    d = x.shape[-1]
    x = x.reshape(*x.shape[:-1], d // 2, 2).transpose(-1, -2).reshape(*x.shape[:-1], d)
    cos, sin = cos.unsqueeze(2), sin.unsqueeze(2)
    return x * cos + rotate_half(x) * sin


def mla_assemble(q, kv, k_pe, cos, sin):
    """q [B,S,H,192], kv [B,S,H,256], k_pe [B,S,64] -> (query [B,S,H,192], key [B,S,H,192], value [B,S,H,128])."""
    q_nope, q_pe = q[..., :128], q[..., 128:]
    k_nope, value = kv[..., :128], kv[..., 128:]
    q_rot = apply_rotary_deepseek(q_pe, cos, sin)
    k_rot = apply_rotary_deepseek(k_pe.unsqueeze(2), cos, sin)
    query = torch.cat((q_nope, q_rot), dim=-1)
    key = torch.cat((k_nope, k_rot.expand(-1, -1, q.shape[2], -1)), dim=-1)
    return query, key, value.contiguous()


def mla_assemble_bwd(q, kv, k_pe, cos, sin, dquery, dkey, dvalue):
    leaves = [t.detach().clone().requires_grad_() for t in (q, kv, k_pe)]
    outs = mla_assemble(leaves[0], leaves[1], leaves[2], cos, sin)
    torch.autograd.backward(list(outs), [dquery, dkey, dvalue])
    return tuple(t.grad for t in leaves)
