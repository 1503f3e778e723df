"""Generates the golden vectors under tests/golden/ by running the REFERENCE's own code on CPU.

Run once in a container that has the PithTrain checkout (default /root/reference):

    python tests/golden/make_golden.py [/path/to/PithTrain]

What is executed from the reference (nothing is copied):
  * pithtrain.operators.ring_attention.standard._online_softmax_combine          (natural-log merge)
  * pithtrain.operators.ring_attention.mla._online_softmax_combine_log2          (log2 merge)
  * tests.operators.mla.test_triton_non_causal._reference_attention + autograd   (attention ground truth)
The reference's GPU kernels (flash-attn, Triton) cannot run without a GPU; its CPU-runnable pieces above
are what pin the oracle. ``torch.cuda.get_device_capability`` is stubbed during import because
pithtrain/operators/mla/__init__.py:3 calls it at import time.

Outputs (small, committed): golden_combine.npz, golden_attention.npz.
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
    root = sys.argv[1] if len(sys.argv) > 1 else "/root/reference"
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
    for f in ("golden_combine.npz", "golden_attention.npz"):
        print(f, (HERE / f).stat().st_size, "bytes")


if __name__ == "__main__":
    main()
