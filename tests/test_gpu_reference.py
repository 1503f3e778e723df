"""This library beside the reference's own GPU path, on identical seeded inputs.

The reference (PithTrain) is imported from ``baseline/_ref`` (``python baseline/install_reference.py <checkout>``);
without it these tests skip. Covered:

* the reference's Triton MLA kernels ``_mla_fwd``, ``_mla_bwd_preprocess``, ``_mla_bwd_dk_dv``, ``_mla_bwd_dq``
  (pithtrain/operators/mla/triton.py:552-603) against the same-named helpers here, at 16 heads and S = 4096;
* how far the reference's kernels (Triton MLA, flash-attn) and ours each sit from the fp32 oracle, which is what
  justifies the half-ulp allowance for bf16-rounded tensors in ``helpers.assert_bf16_close``;
* the reference's attention modules (pithtrain/models/qwen3_30b_a3b.py:347-442,
  pithtrain/models/deepseek_v2_lite.py:352-472) run stock and with the import swaps of INTEGRATION.md patched in.

Bars: O, dQ, dK, dV max-abs <= 2e-2 (+ half a bf16 ulp per rounded operand), mean-abs <= 2e-3; LSE <= 1e-3.
"""

import sys
from pathlib import Path

import pytest
import torch

from helpers import assert_bf16_close, assert_lse_close
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu

REF = Path(__file__).resolve().parent.parent / "baseline" / "_ref"


@pytest.fixture(scope="module")
def ref(cuda_device):
    if not (REF / "pithtrain").is_dir():
        pytest.skip("the reference is not installed under baseline/_ref (python baseline/install_reference.py <checkout>)")
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))
    import pithtrain  # noqa: F401
    return REF


def _mla_inputs(dev, S=4096, H=16, seed=42):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(1, S, H, 192, generator=g).bfloat16().to(dev)
    k = torch.randn(1, S, H, 192, generator=g).bfloat16().to(dev)
    v = torch.randn(1, S, H, 128, generator=g).bfloat16().to(dev)
    do = torch.randn(1, S, H, 128, generator=g).bfloat16().to(dev)
    return q, k, v, do


def _errs(got, want):
    d = (got.float().cpu() - want.float().cpu()).abs()
    return d.max().item(), d.mean().item()


def test_triton_mla_kernels_against_ours_and_the_oracle(ref, cuda_device, capsys):
    from pithtrain.operators.mla import triton as T
    from pithtrain_b200.operators import mla as M
    q, k, v, do = _mla_inputs(cuda_device)
    scale = 192 ** -0.5
    ro, rl = T._mla_fwd(q, k, v, scale, True)
    rdelta = T._mla_bwd_preprocess(ro, do)
    rdk, rdv = T._mla_bwd_dk_dv(q, k, v, do, rl, rdelta, scale, True)
    rdq = T._mla_bwd_dq(q, k, v, do, rl, rdelta, scale, True)
    oo, ol = M._mla_fwd(q, k, v, scale, True)
    odelta = M._mla_bwd_preprocess(oo, do)
    odk, odv = M._mla_bwd_dk_dv(q, k, v, do, ol, odelta, scale, True)
    odq = M._mla_bwd_dq(q, k, v, do, ol, odelta, scale, True)
    torch.cuda.synchronize()
    # ours against the reference's kernels: both sides are rounded to bf16
    assert_lse_close(ol, rl, "LSE (log2) vs Triton")
    assert torch.allclose(odelta, rdelta, atol=2e-2, rtol=1e-2)
    for name, a, b in (("O", oo, ro), ("dQ", odq, rdq), ("dK", odk, rdk), ("dV", odv, rdv)):
        assert_bf16_close(a, b, name + " vs Triton")
        assert O.cosine_error(a, b) < 1e-5, name
    # both against the fp32 oracle on two heads (the CPU takes seconds for these)
    heads = [3, 12]
    qc, kc, vc, dc = (t[:, :, heads].cpu() for t in (q, k, v, do))
    fo, fl = O.attention_fwd(qc, kc, vc, scale, True, 0)
    fdq, fdk, fdv = O.attention_bwd(qc, kc, vc, dc, fl, O.delta(fo, dc), scale, True, 0)
    rows = []
    for name, want, mine, theirs in (("O", fo, oo, ro), ("dQ", fdq, odq, rdq), ("dK", fdk, odk, rdk), ("dV", fdv, odv, rdv)):
        assert_bf16_close(mine[:, :, heads], want, name + " vs oracle")
        rows.append((name, _errs(mine[:, :, heads], want), _errs(theirs[:, :, heads], want)))
    with capsys.disabled():
        print("\nMLA S=4096 H=16, error against the fp32 oracle (max-abs / mean-abs), heads 3 and 12:")
        for name, mine, theirs in rows:
            print(f"  {name:3s} this library {mine[0]:.3e} / {mine[1]:.3e}   reference Triton {theirs[0]:.3e} / {theirs[1]:.3e}")
    for name, mine, theirs in rows:  # not further from the oracle than the reference's own kernels, up to rounding noise
        assert mine[1] <= theirs[1] * 1.5 + 1e-5, (name, mine, theirs)


def test_flash_attn_and_ours_against_the_oracle(cuda_device, capsys):
    """The arithmetic behind the reference's GQA path is flash-attn (ring_attention/standard.py:26,:91,:134). On the last
    128 queries of two heads of the Qwen3 layer at S = 8192, where the oracle is cheap, record both distances."""
    fa = pytest.importorskip("flash_attn")
    from pithtrain_b200.operators.attention import flash_attn_func as ours
    g = torch.Generator().manual_seed(42)
    S, Hq, Hkv, D = 8192, 32, 4, 128
    q = torch.randn(1, S, Hq, D, generator=g).bfloat16().to(cuda_device)
    k = torch.randn(1, S, Hkv, D, generator=g).bfloat16().to(cuda_device)
    v = torch.randn(1, S, Hkv, D, generator=g).bfloat16().to(cuda_device)
    do = torch.randn(1, S, Hq, D, generator=g).bfloat16().to(cuda_device)
    scale = D ** -0.5
    res = {}
    for name, fn in (("flash-attn", fa.flash_attn_func), ("this library", ours)):
        ql, kl, vl = (t.clone().requires_grad_() for t in (q, k, v))
        out = fn(ql, kl, vl, softmax_scale=scale, causal=True)
        out.backward(do)
        res[name] = (out.detach(), ql.grad, kl.grad, vl.grad)
    torch.cuda.synchronize()
    heads, kv = [5, 31], [0, 3]
    n = 128
    qc, dc = q[:, -n:, heads].cpu(), do[:, -n:, heads].cpu()
    fo, fl = O.attention_fwd(qc, k[:, :, kv].cpu(), v[:, :, kv].cpu(), scale, True, S - n)
    # dK, dV of the last 128 keys depend on the last 128 queries of the whole GQA group only
    grp = list(range(24, 32))
    qg, dg = q[:, -n:, grp].cpu(), do[:, -n:, grp].cpu()
    go, gl = O.attention_fwd(q[:, :, grp].cpu()[:, -n:], k[:, :, [3]].cpu(), v[:, :, [3]].cpu(), scale, True, S - n)
    _, gdk, gdv = O.attention_bwd(qg, k[:, -n:, [3]].cpu(), v[:, -n:, [3]].cpu(), dg, gl, O.delta(go, dg), scale, True, 0)
    rows = []
    for name, (out, dq, dk, dv) in res.items():
        rows.append((name, _errs(out[:, -n:, heads], fo), _errs(dk[:, -n:, [3]], gdk), _errs(dv[:, -n:, [3]], gdv)))
    with capsys.disabled():
        print("\nQwen3 layer S=8192, error against the fp32 oracle (max-abs / mean-abs):")
        for name, eo, edk, edv in rows:
            print(f"  {name:13s} O[-128:] {eo[0]:.3e} / {eo[1]:.3e}   dK[-128:] {edk[0]:.3e} / {edk[1]:.3e}   "
                  f"dV[-128:] {edv[0]:.3e} / {edv[1]:.3e}")
    mine, theirs = rows[1], rows[0]
    for a, b in zip(mine[1:], theirs[1:]):
        assert a[1] <= b[1] * 1.5 + 1e-5, rows
    assert_bf16_close(res["this library"][0][:, -n:, heads], fo, "O vs oracle")
    assert_bf16_close(res["this library"][2][:, -n:, [3]], gdk, "dK vs oracle")
    assert_bf16_close(res["this library"][3][:, -n:, [3]], gdv, "dV vs oracle")


def _layer_io(module, x, run):
    """Forward + backward of an attention module: returns (output, dx, {parameter name: grad})."""
    module.zero_grad(set_to_none=True)
    xl = x.detach().clone().requires_grad_()
    out = run(module, xl)
    g = torch.Generator().manual_seed(1)
    dout = torch.randn(out.shape, generator=g).to(out.dtype).to(out.device)
    out.backward(dout)
    return out.detach(), xl.grad, {n: p.grad.detach().clone() for n, p in module.named_parameters() if p.grad is not None}


def _compare_layers(stock, swapped, what):
    (o1, dx1, g1), (o2, dx2, g2) = stock, swapped
    assert_bf16_close(o2, o1, f"{what}: layer output")
    assert O.cosine_error(o2, o1) < 1e-4
    assert O.cosine_error(dx2, dx1) < 1e-4, what
    assert set(g1) == set(g2)
    for n in g1:  # weight gradients are sums over thousands of tokens: compare direction and size, not single ulps
        assert O.cosine_error(g2[n], g1[n]) < 1e-4, (what, n)


def test_qwen3_attention_layer_with_the_import_swap(ref, cuda_device):
    """pithtrain/models/qwen3_30b_a3b.py:347-442 with `flash_attn_func` replaced the way INTEGRATION.md says."""
    import pithtrain.models.qwen3_30b_a3b as M
    from pithtrain_b200.operators.attention import flash_attn_func as ours
    torch.manual_seed(0)
    layer = M.Qwen3MoeAttention(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128)
    layer = layer.to(cuda_device).bfloat16()
    S = 1024
    x = torch.randn(1, S, 512, device=cuda_device).bfloat16()
    inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, device=cuda_device, dtype=torch.float32) / 128))
    emb = torch.outer(torch.arange(S, device=cuda_device, dtype=torch.float32), inv).repeat(1, 2)[None]
    pos = (emb.cos().bfloat16(), emb.sin().bfloat16())
    run = lambda m, xl: m(xl, pos)  # noqa: E731
    stock = _layer_io(layer, x, run)
    original = M.flash_attn_func
    M.flash_attn_func = ours
    try:
        swapped = _layer_io(layer, x, run)
    finally:
        M.flash_attn_func = original
    _compare_layers(stock, swapped, "Qwen3MoeAttention")


def test_deepseek_attention_layer_with_the_import_swap(ref, cuda_device):
    """pithtrain/models/deepseek_v2_lite.py:352-472 with its `MLA` operator replaced by this library's."""
    import pithtrain.models.deepseek_v2_lite as M
    from transformers.models.deepseek_v3.configuration_deepseek_v3 import DeepseekV3Config
    from pithtrain_b200.operators.mla import MLA as OurMLA
    cfg = DeepseekV3Config(hidden_size=512, num_attention_heads=16, num_key_value_heads=16, qk_rope_head_dim=64,
                           qk_nope_head_dim=128, v_head_dim=128, kv_lora_rank=512, q_lora_rank=None,
                           max_position_embeddings=8192, rms_norm_eps=1e-6, rope_theta=10000.0,
                           rope_scaling={"type": "yarn", "rope_type": "yarn", "factor": 40.0, "rope_theta": 10000.0,
                                         "original_max_position_embeddings": 4096, "beta_fast": 32, "beta_slow": 1,
                                         "mscale": 0.707, "mscale_all_dim": 0.707})
    torch.manual_seed(0)
    layer = M.DeepseekV2LiteAttention(cfg).to(cuda_device).bfloat16()
    S = 4096  # the shape the kernel test above already tuned the reference's Triton kernels for
    x = torch.randn(1, S, 512, device=cuda_device).bfloat16()
    pos = torch.arange(S, device=cuda_device)[None]
    run = lambda m, xl: m(xl, position_ids=pos)  # noqa: E731
    stock = _layer_io(layer, x, run)
    original = layer.attn
    layer.attn = OurMLA(layer.num_heads, layer.q_head_dim, layer.v_head_dim, layer.softmax_scale)
    try:
        swapped = _layer_io(layer, x, run)
    finally:
        layer.attn = original
    _compare_layers(stock, swapped, "DeepseekV2LiteAttention")


# ----------------------------------------------------------------------------- zigzag through the reference's caller
def _cp_layer_worker(rank, world, port, path, ref_dir):
    """One CP rank: the reference's Qwen3MoeAttention with a CP group, its `ring_attention_func` replaced by this
    library's with zigzag sharding, fed the zigzag slice of the hidden states and zigzag position ids."""
    import os
    import torch.distributed as dist
    sys.path.insert(0, ref_dir)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import pithtrain.models.qwen3_30b_a3b as M
        from pithtrain_b200.modules.distributed import cp_position_ids
        from pithtrain_b200.operators.ring_attention import ring_attention_func, sharding as sh
        group = dist.new_group(list(range(world)))
        M.ring_attention_func = lambda q, k, v, softmax_scale, cp_group: ring_attention_func(  # the import swap
            q, k, v, softmax_scale, cp_group, "zigzag")
        torch.manual_seed(0)
        layer = M.Qwen3MoeAttention(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                                    cp_group=group).to(dev).bfloat16()
        assert layer.use_ring_attn
        S = 1024 * world
        g = torch.Generator().manual_seed(7)
        x = torch.randn(1, S, 512, generator=g).bfloat16()
        dout = torch.randn(1, S, 512, generator=g).bfloat16()
        xl = sh.shard_sequence(x, world, rank, "zigzag").contiguous().to(dev).requires_grad_()
        dl = sh.shard_sequence(dout, world, rank, "zigzag").contiguous().to(dev)
        pos = cp_position_ids(S // world, rank, world, "zigzag", device=dev)[0].float()
        inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, device=dev, dtype=torch.float32) / 128))
        emb = torch.outer(pos, inv).repeat(1, 2)[None]
        out = layer(xl, (emb.cos().bfloat16(), emb.sin().bfloat16()))
        out.backward(dl)
        torch.cuda.synchronize()
        grads = {n: p.grad.detach().float() for n, p in layer.named_parameters()}
        for t in grads.values():  # what FSDP / DDP would do across the CP ranks
            dist.all_reduce(t)
        torch.save({"out": out.detach().cpu(), "dx": xl.grad.cpu(), "grads": {n: t.cpu() for n, t in grads.items()}},
                   os.path.join(path, f"rank{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_reference_layer_under_zigzag_cp_equals_single_gpu(ref, cuda_device, tmp_path):
    """Config-3 plumbing through a real caller (pithtrain/models/qwen3_30b_a3b.py:432): the reference's attention layer
    on 2+ GPUs with zigzag token slices, zigzag position ids and this library's ring operator must reproduce the same
    layer on one GPU with its stock flash-attn path over the whole sequence."""
    import socket
    import torch.multiprocessing as mp
    from pithtrain_b200.operators.ring_attention import sharding as sh
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_cp_layer_worker, args=(world, port, str(tmp_path), str(ref)), nprocs=world, join=True)
    res = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    import pithtrain.models.qwen3_30b_a3b as M
    torch.manual_seed(0)
    layer = M.Qwen3MoeAttention(hidden_size=512, num_attention_heads=8, num_key_value_heads=2, head_dim=128)
    layer = layer.to(cuda_device).bfloat16()
    S = 1024 * world
    g = torch.Generator().manual_seed(7)
    x = torch.randn(1, S, 512, generator=g).bfloat16().to(cuda_device).requires_grad_()
    dout = torch.randn(1, S, 512, generator=g).bfloat16().to(cuda_device)
    inv = 1.0 / (1e6 ** (torch.arange(0, 128, 2, device=cuda_device, dtype=torch.float32) / 128))
    emb = torch.outer(torch.arange(S, device=cuda_device, dtype=torch.float32), inv).repeat(1, 2)[None]
    out = layer(x, (emb.cos().bfloat16(), emb.sin().bfloat16()))  # stock: flash_attn_func over the whole sequence
    out.backward(dout)
    got_out = sh.unshard_sequence([r["out"] for r in res], "zigzag", seq_dim=1)
    got_dx = sh.unshard_sequence([r["dx"] for r in res], "zigzag", seq_dim=1)
    assert_bf16_close(got_out, out.detach(), "layer output, zigzag CP vs single GPU")
    assert O.cosine_error(got_out, out.detach().cpu()) < 1e-4
    assert O.cosine_error(got_dx, x.grad.cpu()) < 1e-4
    for n, p in layer.named_parameters():
        assert O.cosine_error(res[0]["grads"][n], p.grad.float().cpu()) < 1e-4, n
