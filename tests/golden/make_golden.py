"""Generates the golden vectors under tests/golden/ by running the REFERENCE's own code on CPU.

Run once where a PithTrain checkout is available:

    python tests/golden/make_golden.py /path/to/PithTrain      (or set PITHTRAIN_ROOT)

What is executed from the reference (nothing is copied):
  * pithtrain.operators.ring_attention.standard._online_softmax_combine          (natural-log merge)
  * pithtrain.operators.ring_attention.mla._online_softmax_combine_log2          (log2 merge)
  * tests.operators.mla.test_triton_non_causal._reference_attention + autograd   (attention ground truth)
The reference's GPU kernels (flash-attn, Triton) cannot run without a GPU; its CPU-runnable pieces above
are what pin the oracle. ``torch.cuda.get_device_capability`` is stubbed during import because
pithtrain/operators/mla/__init__.py:3 calls it at import time.

  * pithtrain.models.qwen3_30b_a3b.apply_rotary_pos_emb, Qwen3MoeRotaryEmbedding, with torch.nn.RMSNorm as the
    model constructs it                                                          (q/k norm + rotary, fwd + autograd)

  * pithtrain.models.deepseek_v2_lite.apply_rotary_pos_emb, DeepseekV2LiteYarnRotaryEmbedding
                                                              (MLA rotary + input assembly, fwd + autograd)

Outputs (small, committed): golden_combine.npz, golden_attention.npz, golden_qk_norm_rope.npz,
golden_mla_assemble.npz.
"""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def import_reference(root: str):
    sys.path.insert(0, root)
    real = torch.cuda.get_device_capability
    torch.cuda.get_device_capability = lambda *a, **k: (10, 0)
    try:
        from pithtrain.operators.ring_attention.mla import _online_softmax_combine_log2
        from pithtrain.operators.ring_attention.standard import _online_softmax_combine
        from tests.operators.mla.test_triton_non_causal import _reference_attention
    finally:
        torch.cuda.get_device_capability = real
    return _online_softmax_combine, _online_softmax_combine_log2, _reference_attention


def bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().bfloat16().view(torch.int16).numpy().view(np.uint16)


def main() -> None:
    import os
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("PITHTRAIN_ROOT")
    if not root:
        raise SystemExit("usage: make_golden.py /path/to/PithTrain (or set PITHTRAIN_ROOT)")
    combine_nat, combine_log2, ref_attention = import_reference(root)

    # ---- combine: random partials, plus the sentinels the ring uses (-inf and finfo.min)
    g = torch.Generator().manual_seed(1234)
    B, S, H, D = 2, 24, 3, 16
    out1 = torch.randn(B, S, H, D, generator=g)
    out2 = torch.randn(B, S, H, D, generator=g).bfloat16()
    lse1 = torch.randn(B, H, S, generator=g) * 4
    lse2 = torch.randn(B, H, S, generator=g) * 4
    lse1[0, 0, :4] = float("-inf")
    lse2[1, 2, 5:9] = torch.finfo(torch.float32).min
    o_nat, l_nat = combine_nat(out1, lse1, out2, lse2)
    o_l2, l_l2 = combine_log2(out1, lse1, out2, lse2)
    np.savez_compressed(
        HERE / "golden_combine.npz",
        out1=out1.numpy(), out2=out2.float().numpy(), lse1=lse1.numpy(), lse2=lse2.numpy(),
        out_nat=o_nat.numpy(), lse_nat=l_nat.numpy(), out_log2=o_l2.numpy(), lse_log2=l_l2.numpy())

    # ---- attention: the reference's manual attention (MHA, since that function has no GQA), fwd + autograd
    cases = {}
    for name, (b, s, h, dq, dv, causal) in {
        "mla_causal": (1, 48, 1, 192, 128, True),
        "mla_full": (1, 32, 1, 192, 128, False),
        "d128_causal": (2, 40, 1, 128, 128, True),
    }.items():
        g = torch.Generator().manual_seed(42)
        q = torch.randn(b, s, h, dq, generator=g).bfloat16().float().requires_grad_()
        k = torch.randn(b, s, h, dq, generator=g).bfloat16().float().requires_grad_()
        v = torch.randn(b, s, h, dv, generator=g).bfloat16().float().requires_grad_()
        do = torch.randn(b, s, h, dv, generator=g).bfloat16().float()
        scale = dq ** -0.5
        o = ref_attention(q, k, v, scale, causal=causal)
        o.backward(do)
        cases.update({
            # inputs are bf16-exact: stored as bf16 bit patterns (uint16)
            f"{name}.q": bits(q), f"{name}.k": bits(k), f"{name}.v": bits(v),
            f"{name}.do": bits(do), f"{name}.o": o.detach().numpy(), f"{name}.dq": q.grad.numpy(),
            f"{name}.dk": k.grad.numpy(), f"{name}.dv": v.grad.numpy(),
            f"{name}.meta": np.array([b, s, h, dq, dv, int(causal)], dtype=np.int64),
        })
    np.savez_compressed(HERE / "golden_attention.npz", **cases)
    make_qk_norm_rope()
    make_mla_assemble()
    for f in ("golden_combine.npz", "golden_attention.npz", "golden_qk_norm_rope.npz", "golden_mla_assemble.npz"):
        print(f, (HERE / f).stat().st_size, "bytes")


def make_mla_assemble() -> None:
    """Rotary embedding + assembly of the MLA operator's inputs with the reference's own ``apply_rotary_pos_emb``
    and ``DeepseekV2LiteYarnRotaryEmbedding`` (pithtrain/models/deepseek_v2_lite.py:173-187, :103-163), following
    the statements of the attention layer's forward (:426-454, :463) one by one, on CPU in fp32 with autograd."""
    from pithtrain.models.deepseek_v2_lite import DeepseekV2LiteYarnRotaryEmbedding, apply_rotary_pos_emb
    g = torch.Generator().manual_seed(11)
    B, S, H = 2, 10, 3
    q = torch.randn(B, S, H, 192, generator=g).bfloat16().float().requires_grad_()
    kv = torch.randn(B, S, H, 256, generator=g).bfloat16().float().requires_grad_()
    k_pe = torch.randn(B, S, 1, 64, generator=g).bfloat16().float().requires_grad_()
    position_ids = torch.stack([torch.arange(S) + 3, torch.arange(S) * 29 + 500])
    rotary = DeepseekV2LiteYarnRotaryEmbedding(64, max_position_embeddings=2048, scaling_factor=40.0, base=10000,
                                               original_max_position_embeddings=4096, beta_fast=32, beta_slow=1,
                                               mscale=0.707, mscale_all_dim=0.707)
    q_nope, q_pe = torch.split(q, [128, 64], dim=-1)
    k_nope, value_states = torch.split(kv, [128, 128], dim=-1)
    cos, sin = rotary(value_states, seq_len=int(position_ids.max()) + 1)
    q_rot, k_rot = apply_rotary_pos_emb(q_pe, k_pe, cos, sin, position_ids, unsqueeze_dim=2)
    query_states = k_rot.new_empty(B, S, H, 192)
    query_states[:, :, :, :128] = q_nope
    query_states[:, :, :, 128:] = q_rot
    key_states = k_rot.new_empty(B, S, H, 192)
    key_states[:, :, :, :128] = k_nope
    key_states[:, :, :, 128:] = k_rot
    value = value_states.contiguous()
    grads = [torch.randn(t.shape, generator=g).bfloat16().float() for t in (query_states, key_states, value)]
    torch.autograd.backward([query_states, key_states, value], grads)
    np.savez_compressed(
        HERE / "golden_mla_assemble.npz",
        q=bits(q), kv=bits(kv), k_pe=bits(k_pe[:, :, 0]), position_ids=position_ids.numpy(),
        cos=cos[position_ids].detach().float().numpy(), sin=sin[position_ids].detach().float().numpy(),
        query=query_states.detach().numpy(), key=key_states.detach().numpy(), value=value.detach().numpy(),
        dquery=bits(grads[0]), dkey=bits(grads[1]), dvalue=bits(grads[2]),
        dq=q.grad.numpy(), dkv=kv.grad.numpy(), dk_pe=k_pe.grad[:, :, 0].numpy())


def make_qk_norm_rope() -> None:
    """q/k RMSNorm + rotary embedding exactly as the reference's attention layer runs them
    (pithtrain/models/qwen3_30b_a3b.py:381-382 modules, :417-421 calls), on CPU: once in fp32 with autograd (pins the
    oracle) and once in bf16 (the dtype the model runs in; shows the rounding the reference takes between kernels)."""
    from pithtrain.models.qwen3_30b_a3b import Qwen3MoeRotaryEmbedding, apply_rotary_pos_emb
    g = torch.Generator().manual_seed(7)
    B, S, Hq, Hkv, D, eps = 2, 12, 4, 2, 128, 1e-6
    q = torch.randn(B, S, Hq, D, generator=g).bfloat16().float().requires_grad_()
    k = (torch.randn(B, S, Hkv, D, generator=g) * 3).bfloat16().float().requires_grad_()
    q_norm, k_norm = torch.nn.RMSNorm(D, eps=eps), torch.nn.RMSNorm(D, eps=eps)
    with torch.no_grad():
        q_norm.weight.copy_((1 + 0.25 * torch.randn(D, generator=g)).bfloat16().float())
        k_norm.weight.copy_((1 + 0.25 * torch.randn(D, generator=g)).bfloat16().float())
    position_ids = torch.stack([torch.arange(S) + 5, torch.arange(S) * 37 + 1000])  # [B, S], two different offsets
    rotary = Qwen3MoeRotaryEmbedding(D, max_position_embeddings=4096)
    cos, sin = rotary(q, position_ids)
    qe, ke = apply_rotary_pos_emb(q_norm(q), k_norm(k), cos, sin)
    dqe = torch.randn(qe.shape, generator=g).bfloat16().float()
    dke = torch.randn(ke.shape, generator=g).bfloat16().float()
    torch.autograd.backward([qe, ke], [dqe, dke])
    with torch.no_grad():  # the same in bf16, as the model runs it
        qb, kb = q.detach().bfloat16(), k.detach().bfloat16()
        qn, kn = torch.nn.RMSNorm(D, eps=eps).bfloat16(), torch.nn.RMSNorm(D, eps=eps).bfloat16()
        qn.weight.copy_(q_norm.weight); kn.weight.copy_(k_norm.weight)
        cos_b, sin_b = rotary(qb, position_ids)
        qe_b, ke_b = apply_rotary_pos_emb(qn(qb), kn(kb), cos_b, sin_b)
    np.savez_compressed(
        HERE / "golden_qk_norm_rope.npz",
        q=bits(q), k=bits(k), q_weight=bits(q_norm.weight), k_weight=bits(k_norm.weight),
        position_ids=position_ids.numpy(), cos=cos.numpy(), sin=sin.numpy(), eps=np.float64(eps),
        q_embed=qe.detach().numpy(), k_embed=ke.detach().numpy(), dq_embed=bits(dqe), dk_embed=bits(dke),
        dq=q.grad.numpy(), dk=k.grad.numpy(), dq_weight=q_norm.weight.grad.numpy(), dk_weight=k_norm.weight.grad.numpy(),
        q_embed_bf16=bits(qe_b), k_embed_bf16=bits(ke_b))


if __name__ == "__main__":
    main()
