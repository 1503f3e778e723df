"""CPU oracle for the context-parallel attention path. TEST INFRASTRUCTURE ONLY.

This module restates, in plain PyTorch on CPU tensors (fp32 or fp64), the arithmetic the
reference performs on the GPU for ring attention. Only ``tests/``, ``__graft_entry__.smoke()``
and the ``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may import it; the shipped
operators never do.

What each function follows in the reference (paths inside the PithTrain repository):

* ``attention_fwd``      — the manual attention the reference tests use as ground truth,
  ``tests/operators/mla/test_triton_non_causal.py:48-60`` (same text at
  ``tests/test_online_softmax_combine_log2.py:21-33``): fp32 ``QK^T * scale``, ``triu(diagonal=1)``
  mask with -inf, softmax, ``@ V``.  GQA broadcasts each kv head over ``Hq / Hkv`` query heads
  (flash-attn semantics used at ``pithtrain/operators/ring_attention/standard.py:91-93``).
  The log2 LSE equals ``log2(l) + m * scale * log2(e)`` of ``pithtrain/operators/mla/triton.py:92``.
* ``attention_bwd``      — the block backward with EXTERNAL (global) LSE and delta, as
  ``bwd_phase_2_kernel`` / ``bwd_phase_3_kernel`` compute it (``pithtrain/operators/mla/triton.py:128-266``):
  ``P = exp2(S * scale * log2e - lse)``, ``dV = P^T dO``, ``dS = P * (dO V^T - delta) * scale``,
  ``dK = dS^T Q``, ``dQ = dS K``.
* ``delta``              — ``bwd_phase_1_kernel`` (``triton.py:99-122``).
* ``combine``            — ``_online_softmax_combine`` (``ring_attention/standard.py:53-66``) and
  ``_online_softmax_combine_log2`` (``ring_attention/mla.py:27-40``).
* ``ring_contiguous_*``  — the schedule of ``RingAttentionFunc.forward/backward``
  (``ring_attention/standard.py:72-189``): rank r attends to kv ranks <= r, causal only on its own.
* ``zigzag_*``           — load-balanced sharding (rank r owns chunks r and 2C-1-r of 2C); the reference
  names it as future work (``standard.py:16-18``); its ground truth is full attention re-sliced.

Pinning: ``tests/golden/`` holds vectors produced by the reference's own ``_online_softmax_combine``,
``_online_softmax_combine_log2`` and ``_reference_attention`` (+ autograd) run on CPU
(``tests/golden/make_golden.py``); ``tests/test_oracle.py`` checks this module against them.
The GPU kernels of flash-attn / Triton themselves cannot run in a GPU-less container, so the
attention arithmetic is pinned to the reference's test oracle, not to its GPU output.
"""

from __future__ import annotations


import torch

LOG2E = 1.4426950408889634
LN2 = 0.6931471805599453


def _expand_kv(x: torch.Tensor, hq: int) -> torch.Tensor:
    """[B,S,Hkv,D] -> [B,S,Hq,D] by repeating each kv head over its query-head group."""
    hkv = x.shape[2]
    assert hq % hkv == 0
    return x if hq == hkv else x.repeat_interleave(hq // hkv, dim=2)


def visibility_mask(sq: int, sk: int, causal: bool, causal_offset: int = 0) -> torch.Tensor:
    """Boolean [Sq,Sk]: True where key n is visible to query m (n <= m + causal_offset)."""
    if not causal:
        return torch.ones(sq, sk, dtype=torch.bool)
    m = torch.arange(sq).unsqueeze(1)
    n = torch.arange(sk).unsqueeze(0)
    return n <= m + causal_offset


def attention_fwd(q, k, v, scale: float, causal: bool, causal_offset: int = 0, dtype=torch.float32):
    """Returns (O [B,Sq,Hq,Dv], LSE_log2 [B,Hq,Sq]) in ``dtype``. Rows with no visible key give O=0, LSE=-inf."""
    hq = q.shape[2]
    qt = q.to(dtype).permute(0, 2, 1, 3)
    kt = _expand_kv(k, hq).to(dtype).permute(0, 2, 1, 3)
    vt = _expand_kv(v, hq).to(dtype).permute(0, 2, 1, 3)
    scores = torch.matmul(qt, kt.transpose(-2, -1)) * scale
    vis = visibility_mask(q.shape[1], k.shape[1], causal, causal_offset)
    scores = scores.masked_fill(~vis, float("-inf"))
    lse_nat = torch.logsumexp(scores, dim=-1)
    probs = torch.exp(scores - torch.where(torch.isinf(lse_nat), torch.zeros_like(lse_nat), lse_nat).unsqueeze(-1))
    probs = torch.where(vis, probs, torch.zeros_like(probs))
    out = torch.matmul(probs, vt).permute(0, 2, 1, 3).contiguous()
    return out, lse_nat * LOG2E


def delta(o, do, dtype=torch.float32):
    """[B,H,S] rowsum(O * dO)."""
    return (o.to(dtype) * do.to(dtype)).sum(-1).permute(0, 2, 1).contiguous()


def attention_bwd(q, k, v, do, lse_log2, delta_, scale: float, causal: bool, causal_offset: int = 0,
                  dtype=torch.float32):
    """Gradient contributions of one (Q block, KV block) pair given the complete row's LSE and delta.

    Returns (dQ [B,Sq,Hq,Dqk], dK [B,Sk,Hkv,Dqk], dV [B,Sk,Hkv,Dv]) in ``dtype``; dK/dV are summed
    over the query heads of each kv-head group.
    """
    b, sq, hq, _ = q.shape
    hkv = k.shape[2]
    g = hq // hkv
    qt = q.to(dtype).permute(0, 2, 1, 3)
    kt = _expand_kv(k, hq).to(dtype).permute(0, 2, 1, 3)
    vt = _expand_kv(v, hq).to(dtype).permute(0, 2, 1, 3)
    dot = do.to(dtype).permute(0, 2, 1, 3)
    s2 = torch.matmul(qt, kt.transpose(-2, -1)) * (scale * LOG2E)
    vis = visibility_mask(sq, k.shape[1], causal, causal_offset)
    lse = lse_log2.to(dtype).unsqueeze(-1)
    p = torch.exp2(s2 - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse))
    p = torch.where(vis & ~torch.isinf(lse), p, torch.zeros_like(p))
    dv = torch.matmul(p.transpose(-2, -1), dot)
    dp = torch.matmul(dot, vt.transpose(-2, -1))
    ds = p * (dp - delta_.to(dtype).unsqueeze(-1)) * scale
    dq = torch.matmul(ds, kt)
    dk = torch.matmul(ds.transpose(-2, -1), qt)
    dq = dq.permute(0, 2, 1, 3).contiguous()
    dk = dk.permute(0, 2, 1, 3).reshape(b, k.shape[1], hkv, g, -1).sum(3)
    dv = dv.permute(0, 2, 1, 3).reshape(b, k.shape[1], hkv, g, -1).sum(3)
    return dq, dk.contiguous(), dv.contiguous()


def combine(out1, lse1, out2, lse2, log2: bool):
    """Merge two partial (O [B,S,H,D], LSE [B,H,S]); formula and operation order of the reference."""
    mx = torch.maximum(lse1, lse2)
    if log2:
        x1, x2 = torch.exp2(lse1 - mx), torch.exp2(lse2 - mx)
    else:
        x1, x2 = torch.exp(lse1 - mx), torch.exp(lse2 - mx)
    e1 = x1.transpose(1, 2).unsqueeze(-1)
    e2 = x2.transpose(1, 2).unsqueeze(-1)
    out = (e1 * out1 + e2 * out2) / (e1 + e2)
    lse = mx + (torch.log2(x1 + x2) if log2 else torch.log(x1 + x2))
    return out.contiguous(), lse


def full_attention_fwd_bwd(q, k, v, do, scale: float, dtype=torch.float32):
    """Full-sequence causal attention forward + backward. Returns dict(o, lse_log2, dq, dk, dv)."""
    o, lse = attention_fwd(q, k, v, scale, True, 0, dtype)
    dl = delta(o, do, dtype)
    dq, dk, dv = attention_bwd(q, k, v, do, lse, dl, scale, True, 0, dtype)
    return {"o": o, "lse_log2": lse, "dq": dq, "dk": dk, "dv": dv}


# ----------------------------------------------------------------------------- sharding
def zigzag_indices(seq_len: int, cp_size: int, rank: int) -> torch.Tensor:
    """Global positions held by ``rank``: chunk ``rank`` then chunk ``2*cp_size-1-rank`` of ``2*cp_size``."""
    assert seq_len % (2 * cp_size) == 0
    c = seq_len // (2 * cp_size)
    lo = torch.arange(rank * c, (rank + 1) * c)
    hi = torch.arange((2 * cp_size - 1 - rank) * c, (2 * cp_size - rank) * c)
    return torch.cat([lo, hi])


def contiguous_indices(seq_len: int, cp_size: int, rank: int) -> torch.Tensor:
    assert seq_len % cp_size == 0
    c = seq_len // cp_size
    return torch.arange(rank * c, (rank + 1) * c)


# ----------------------------------------------------------------------------- ring schedules
def ring_contiguous_fwd(q_shards, k_shards, v_shards, scale: float, log2: bool = True, dtype=torch.float32):
    """Reference schedule on contiguous shards: rank r merges blocks from kv ranks r, r-1, ..., 0."""
    cp = len(q_shards)
    outs, lses = [], []
    for r in range(cp):
        b, s, h, _ = q_shards[r].shape
        acc_o = torch.zeros(b, s, h, v_shards[r].shape[-1], dtype=dtype)
        acc_l = torch.full((b, h, s), torch.finfo(torch.float32).min, dtype=dtype)
        for step in range(cp):
            kv = (r - step) % cp
            if kv <= r:
                o, l2 = attention_fwd(q_shards[r], k_shards[kv], v_shards[kv], scale, kv == r, 0, dtype)
                l = l2 if log2 else l2 * LN2
                acc_o, acc_l = combine(acc_o, acc_l, o, l, log2)
        outs.append(acc_o)
        lses.append(acc_l if log2 else acc_l * LOG2E)
    return outs, lses  # lses always returned in the log2 domain


def zigzag_step_kind(rank: int, src: int) -> str:
    """Which part of the (local Q, received KV) pair carries work when the KV comes from ``src``."""
    if src == rank:
        return "causal"        # all local Q x all local KV, causal in local order
    return "kv_first_half" if src < rank else "q_second_half"


def ring_zigzag_fwd(q_shards, k_shards, v_shards, scale: float, dtype=torch.float32):
    """Zigzag schedule: every rank computes at every step; returns per-rank (O, LSE_log2)."""
    cp = len(q_shards)
    outs, lses = [], []
    for r in range(cp):
        b, s, h, _ = q_shards[r].shape
        c = s // 2
        acc_o = torch.zeros(b, s, h, v_shards[r].shape[-1], dtype=dtype)
        acc_l = torch.full((b, h, s), float("-inf"), dtype=dtype)
        for step in range(cp):
            src = (r - step) % cp
            kind = zigzag_step_kind(r, src)
            if kind == "causal":
                o, l = attention_fwd(q_shards[r], k_shards[src], v_shards[src], scale, True, 0, dtype)
                acc_o, acc_l = o, l
            elif kind == "kv_first_half":
                o, l = attention_fwd(q_shards[r], k_shards[src][:, :c], v_shards[src][:, :c], scale, False, 0, dtype)
                acc_o, acc_l = combine(acc_o, acc_l, o, l, True)
            else:
                o, l = attention_fwd(q_shards[r][:, c:], k_shards[src], v_shards[src], scale, False, 0, dtype)
                no, nl = combine(acc_o[:, c:], acc_l[:, :, c:], o, l, True)
                acc_o = torch.cat([acc_o[:, :c], no], dim=1)
                acc_l = torch.cat([acc_l[:, :, :c], nl], dim=2)
        outs.append(acc_o)
        lses.append(acc_l)
    return outs, lses


def ring_zigzag_bwd(q_shards, k_shards, v_shards, do_shards, o_shards, lse_shards, scale: float,
                    dtype=torch.float32):
    """Zigzag backward: per rank dQ; dK/dV summed into the owner of each KV shard."""
    cp = len(q_shards)
    dqs = [torch.zeros_like(q.to(dtype)) for q in q_shards]
    dks = [torch.zeros_like(k.to(dtype)) for k in k_shards]
    dvs = [torch.zeros_like(v.to(dtype)) for v in v_shards]
    for r in range(cp):
        c = q_shards[r].shape[1] // 2
        dl = delta(o_shards[r], do_shards[r], dtype)
        for step in range(cp):
            src = (r - step) % cp
            kind = zigzag_step_kind(r, src)
            if kind == "causal":
                dq, dk, dv = attention_bwd(q_shards[r], k_shards[src], v_shards[src], do_shards[r], lse_shards[r], dl,
                                           scale, True, 0, dtype)
                dqs[r] += dq; dks[src] += dk; dvs[src] += dv
            elif kind == "kv_first_half":
                dq, dk, dv = attention_bwd(q_shards[r], k_shards[src][:, :c], v_shards[src][:, :c], do_shards[r],
                                           lse_shards[r], dl, scale, False, 0, dtype)
                dqs[r] += dq; dks[src][:, :c] += dk; dvs[src][:, :c] += dv
            else:
                dq, dk, dv = attention_bwd(q_shards[r][:, c:], k_shards[src], v_shards[src], do_shards[r][:, c:],
                                           lse_shards[r][:, :, c:], dl[:, :, c:], scale, False, 0, dtype)
                dqs[r][:, c:] += dq; dks[src] += dk; dvs[src] += dv
    return dqs, dks, dvs


def fwd_flops(b: int, h: int, s: int, dqk: int, dv: int) -> float:
    """Causal forward FLOPs, the reference's convention (benchmarks/operators/mla/test_triton.py:7-12)."""
    return float(b) * h * s * s * (dqk + dv)


def fwd_bwd_flops(b: int, h: int, s: int, dqk: int, dv: int) -> float:
    """Forward + 2.5 x forward for the backward (same file, :13-14)."""
    return 3.5 * fwd_flops(b, h, s, dqk, dv)


def cosine_error(a: torch.Tensor, b: torch.Tensor) -> float:
    """1 - cosine similarity of the flattened tensors (tests/test_ring_attention.py metric)."""
    a = a.double().flatten()
    b = b.double().flatten()
    return float(1.0 - torch.dot(a, b) / (a.norm() * b.norm() + 1e-300))


__all__ = [name for name in dir() if not name.startswith("_")]
