"""A fixed, small workload for profilers: one causal forward + backward of each attention kernel.

    python -m pithtrain_b200.profile_case [--shape qwen3|mla] [--seq 8192] [--repeat 2]

Launch order per repeat: attn_fwd_kernel, delta_kernel, attn_bwd_kernel<kDkDv>, attn_bwd_kernel<kDq>,
3 x cast_kernel, combine_kernel, and qk_norm_rope_kernel (head_dim 128) or mla_assemble_kernel (MLA) forward and backward. The working set (a few hundred MB) is larger than the 126 MB L2 and far below the
sizes at which a multi-pass profiler capture gets slow. Prints the CUDA-event time of each launch.

A measurement aid: nothing in the package imports this module; it only calls the public wrappers in ``kernels``.
``--rows / --keys / --non-causal / --merge`` select the shapes of one ring step (for example 4096 queries against
2048 keys, non-causal, merging into a running fp32 result) instead of the square causal block.
"""

from __future__ import annotations

import argparse

import torch

from . import kernels as K


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", choices=["qwen3", "mla"], default="qwen3")
    ap.add_argument("--seq", type=int, default=8192)
    ap.add_argument("--repeat", type=int, default=2)
    ap.add_argument("--rows", type=int, default=0, help="query rows (default: --seq)")
    ap.add_argument("--keys", type=int, default=0, help="key rows (default: --seq)")
    ap.add_argument("--non-causal", action="store_true")
    ap.add_argument("--merge", action="store_true", help="forward merges into a running fp32 (O, LSE), as a ring step")
    args = ap.parse_args()
    hq, hkv, dqk = (32, 4, 128) if args.shape == "qwen3" else (16, 16, 192)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(42)
    S = args.seq
    if args.rows or args.keys or args.non_causal or args.merge:
        ring_step(args, hq, hkv, dqk, dev, g)
        return
    q = torch.randn(1, S, hq, dqk, generator=g).bfloat16().to(dev)
    k = torch.randn(1, S, hkv, dqk, generator=g).bfloat16().to(dev)
    v = torch.randn(1, S, hkv, 128, generator=g).bfloat16().to(dev)
    do = torch.randn(1, S, hq, 128, generator=g).bfloat16().to(dev)
    scale = dqk ** -0.5
    out = torch.empty(1, S, hq, 128, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(1, hq, S, dtype=torch.float32, device=dev)
    delta = torch.empty_like(lse)
    dq, dk, dv = (torch.zeros(t.shape, dtype=torch.float32, device=dev) for t in (q, k, v))
    acc = torch.randn(1, S, hq, 128, device=dev)

    w_norm = torch.ones(dqk, dtype=torch.bfloat16, device=dev)
    emb = torch.outer(torch.arange(S, dtype=torch.float32),
                      1.0 / (1e6 ** (torch.arange(0, dqk, 2, dtype=torch.float32) / dqk))).repeat(1, 2)[None]
    cos, sin = emb.cos().bfloat16().to(dev), emb.sin().bfloat16().to(dev)
    kv_in = torch.randn(1, S, hq, 256, generator=g).bfloat16().to(dev)
    kpe_in = torch.randn(1, S, 64, generator=g).bfloat16().to(dev)

    def timed(name, fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        print(f"{name:28s} {e0.elapsed_time(e1) * 1e3:9.1f} us")

    for rep in range(args.repeat):
        print(f"-- repeat {rep}")
        timed("attn_fwd_kernel", lambda: K.attn_fwd(q, k, v, scale, True, 0, out=out, lse=lse))
        timed("delta_kernel", lambda: K.bwd_preprocess(out, do, delta))
        timed("attn_bwd_kernel<kDkDv>", lambda: K.attn_bwd(q, k, v, do, lse, delta, scale, True, 0, None, dk, dv))
        timed("attn_bwd_kernel<kDq>", lambda: K.attn_bwd(q, k, v, do, lse, delta, scale, True, 0, dq, None, None))
        timed("cast_kernel x3", lambda: (K.cast_to_bf16(dq), K.cast_to_bf16(dk), K.cast_to_bf16(dv)))
        timed("combine_kernel", lambda: K.combine(acc, lse, out, lse, natural=False))
        if dqk == 128:
            timed("qk_norm_rope_kernel fwd", lambda: K.qk_norm_rope_fwd(q, k, w_norm, w_norm, cos, sin, 1e-6))
            timed("qk_norm_rope_kernel bwd", lambda: K.qk_norm_rope_bwd(q, k, w_norm, w_norm, cos, sin, 1e-6, do, k))
        else:
            timed("mla_assemble_kernel fwd", lambda: K.mla_assemble_fwd(q, kv_in, kpe_in, cos[..., :64], sin[..., :64]))
            timed("mla_assemble_kernel bwd", lambda: K.mla_assemble_bwd(cos[..., :64], sin[..., :64], q, k, v))
    K.check_device_status(dev)


def ring_step(args, hq, hkv, dqk, dev, g) -> None:
    """The attention launches of one ring step: Sq x Sk block, optionally non-causal and merging."""
    Sq, Sk, causal = args.rows or args.seq, args.keys or args.seq, not args.non_causal
    q = torch.randn(1, Sq, hq, dqk, generator=g).bfloat16().to(dev)
    k = torch.randn(1, Sk, hkv, dqk, generator=g).bfloat16().to(dev)
    v = torch.randn(1, Sk, hkv, 128, generator=g).bfloat16().to(dev)
    do = torch.randn(1, Sq, hq, 128, generator=g).bfloat16().to(dev)
    scale = dqk ** -0.5
    out = torch.zeros(1, Sq, hq, 128, dtype=torch.float32 if args.merge else torch.bfloat16, device=dev)
    lse = torch.zeros(1, hq, Sq, dtype=torch.float32, device=dev)
    delta = torch.zeros_like(lse)
    dq, dk, dv = (torch.zeros(t.shape, dtype=torch.float32, device=dev) for t in (q, k, v))
    prev = dict(prev_o=out, prev_lse=lse) if args.merge else {}
    for rep in range(args.repeat):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        e[0].record()
        K.attn_fwd(q, k, v, scale, causal, 0, out=out, lse=lse, **prev)
        e[1].record()
        K.attn_bwd(q, k, v, do, lse, delta, scale, causal, 0, None, dk, dv)
        e[2].record()
        K.attn_bwd(q, k, v, do, lse, delta, scale, causal, 0, dq, None, None)
        e[3].record()
        torch.cuda.synchronize()
        print(f"-- repeat {rep}: fwd {e[0].elapsed_time(e[1]) * 1e3:.1f} us, dK/dV {e[1].elapsed_time(e[2]) * 1e3:.1f} us, "
              f"dQ {e[2].elapsed_time(e[3]) * 1e3:.1f} us")
    K.check_device_status(dev)


if __name__ == "__main__":
    main()
