"""Parity of the sm_100a kernels, called through the C ABI, against the CPU oracle and the golden vectors.

Tolerances are the path's bars: bf16 tensors max-abs <= 2e-2 and mean-abs <= 2e-3, LSE within 1e-3 (fp32)."""

import math

import pytest
import torch

from helpers import (GOLDEN, assert_bf16_close, assert_lse_close, load_golden_attention)
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K(cuda_device):
    from pithtrain_b200 import kernels
    yield kernels
    kernels.check_device_status(cuda_device)


def _rand(shape, dev, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randn(shape, generator=g).bfloat16().to(dev)


def _inputs(B, Sq, Sk, Hq, Hkv, Dqk, dev, seed=42):
    return (_rand((B, Sq, Hq, Dqk), dev, seed), _rand((B, Sk, Hkv, Dqk), dev, seed + 1),
            _rand((B, Sk, Hkv, 128), dev, seed + 2), _rand((B, Sq, Hq, 128), dev, seed + 3))


FWD_CASES = [
    # B, Sq, Sk, Hq, Hkv, Dqk, causal, offset
    (1, 128, 128, 1, 1, 128, False, 0),
    (1, 256, 256, 2, 1, 128, True, 0),
    (1, 1024, 1024, 8, 2, 128, True, 0),       # GQA 4:1
    (2, 1000, 1000, 4, 4, 128, True, 0),       # ragged tail, batch 2
    (1, 512, 1024, 8, 1, 128, False, 0),       # GQA 8:1, Sq != Sk
    (1, 512, 1024, 4, 1, 128, True, 512),      # causal, bottom-right aligned
    (1, 384, 200, 4, 2, 128, False, 0),        # key tail inside one block
    (1, 64, 72, 2, 2, 128, True, 8),           # smaller than one tile
    (1, 768, 256, 2, 1, 128, True, -512),      # early queries see nothing: O = 0, LSE = -inf
    (1, 2048, 2048, 4, 4, 192, True, 0),       # MLA head dims
    (1, 512, 520, 16, 16, 192, False, 0),
    (1, 1, 1, 1, 1, 128, True, 0),             # single token
]


@pytest.mark.parametrize("single_cta", [False, True], ids=["cta_pair", "single_cta"])
@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,Dqk,causal,off", FWD_CASES)
def test_forward_matches_oracle(K, cuda_device, B, Sq, Sk, Hq, Hkv, Dqk, causal, off, single_cta):
    q, k, v, _ = _inputs(B, Sq, Sk, Hq, Hkv, Dqk, cuda_device)
    scale = Dqk ** -0.5
    out, lse = K.attn_fwd(q, k, v, scale, causal, off, single_cta=single_cta)
    ro, rl = O.attention_fwd(q.cpu(), k.cpu(), v.cpu(), scale, causal, off)
    assert out.dtype == torch.bfloat16 and lse.dtype == torch.float32
    assert_bf16_close(out, ro, "O")
    assert_lse_close(lse, rl)
    K.check_device_status(cuda_device)


BWD_CASES = [
    (1, 128, 128, 1, 1, 128, False, 0),
    (1, 256, 256, 2, 1, 128, True, 0),
    (1, 1024, 1024, 8, 2, 128, True, 0),
    (2, 1000, 1000, 4, 4, 128, True, 0),
    (1, 512, 1024, 8, 1, 128, False, 0),
    (1, 512, 1024, 4, 1, 128, True, 512),
    (1, 384, 200, 4, 2, 128, False, 0),
    (1, 768, 256, 2, 1, 128, True, -512),
    (1, 2048, 2048, 4, 4, 192, True, 0),
    (1, 1000, 520, 2, 2, 192, False, 0),
    (1, 1, 1, 1, 1, 128, True, 0),
]


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,Dqk,causal,off", BWD_CASES)
def test_backward_matches_oracle(K, cuda_device, B, Sq, Sk, Hq, Hkv, Dqk, causal, off):
    q, k, v, do = _inputs(B, Sq, Sk, Hq, Hkv, Dqk, cuda_device)
    scale = Dqk ** -0.5
    out, lse = K.attn_fwd(q, k, v, scale, causal, off)
    delta = K.bwd_preprocess(out, do)
    dq = torch.zeros(q.shape, device=cuda_device)
    dk = torch.zeros(k.shape, device=cuda_device)
    dv = torch.zeros(v.shape, device=cuda_device)
    K.attn_bwd(q, k, v, do, lse, delta, scale, causal, off, dq, dk, dv)
    ro, rl = O.attention_fwd(q.cpu(), k.cpu(), v.cpu(), scale, causal, off)
    rd = O.delta(ro, do.cpu())
    assert torch.allclose(delta.cpu(), O.delta(out.cpu(), do.cpu()), atol=1e-4, rtol=1e-5)
    rdq, rdk, rdv = O.attention_bwd(q.cpu(), k.cpu(), v.cpu(), do.cpu(), rl, rd, scale, causal, off)
    for acc, ref, name in ((dq, rdq, "dQ"), (dk, rdk, "dK"), (dv, rdv, "dV")):
        assert_bf16_close(acc, ref, name + " (fp32 accumulator)")
        assert_bf16_close(K.cast_to_bf16(acc), ref, name)
    K.check_device_status(cuda_device)


def test_backward_accumulates_and_can_skip_halves(K, cuda_device):
    q, k, v, do = _inputs(1, 256, 256, 4, 2, 128, cuda_device)
    scale = 128 ** -0.5
    out, lse = K.attn_fwd(q, k, v, scale, True, 0)
    delta = K.bwd_preprocess(out, do)
    z = lambda t: torch.zeros(t.shape, device=cuda_device)  # noqa: E731
    dq, dk, dv = z(q), z(k), z(v)
    K.attn_bwd(q, k, v, do, lse, delta, scale, True, 0, dq, dk, dv)
    dq2, dk2, dv2 = dq.clone(), dk.clone(), dv.clone()
    K.attn_bwd(q, k, v, do, lse, delta, scale, True, 0, dq2, None, None)     # dQ only, accumulating
    K.attn_bwd(q, k, v, do, lse, delta, scale, True, 0, None, dk2, dv2)      # dK/dV only
    for a, b in ((dq2, dq), (dk2, dk), (dv2, dv)):
        assert torch.allclose(a, 2 * b, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("name", ["mla_causal", "mla_full", "d128_causal"])
def test_golden_vectors(K, cuda_device, name):
    g = load_golden_attention(name)
    q, k, v, do = (g[x].to(cuda_device) for x in ("q", "k", "v", "do"))
    out, lse = K.attn_fwd(q, k, v, g["scale"], g["causal"], 0)
    assert_bf16_close(out, g["o"], "O")
    delta = K.bwd_preprocess(out, do)
    dq, dk, dv = (torch.zeros(t.shape, device=cuda_device) for t in (q, k, v))
    K.attn_bwd(q, k, v, do, lse, delta, g["scale"], g["causal"], 0, dq, dk, dv)
    assert_bf16_close(dq, g["dq"], "dQ")
    assert_bf16_close(dk, g["dk"], "dK")
    assert_bf16_close(dv, g["dv"], "dV")


def test_fused_merge_equals_separate_combine(K, cuda_device):
    """Attention over two KV halves: the second call merges into the first in its epilogue."""
    q, k, v, _ = _inputs(1, 512, 1024, 8, 2, 128, cuda_device)
    scale = 128 ** -0.5
    acc, lse = K.attn_fwd(q, k[:, :512], v[:, :512], scale, False, 0, out_fp32=True)
    o2, l2 = K.attn_fwd(q, k[:, 512:], v[:, 512:], scale, False, 0, out_fp32=True)
    ref_o, ref_l = K.combine(acc, lse, o2, l2, natural=False)
    K.attn_fwd(q, k[:, 512:], v[:, 512:], scale, False, 0, out=acc, lse=lse, prev_o=acc, prev_lse=lse)
    assert torch.allclose(acc, ref_o, atol=2e-6, rtol=1e-5)
    assert torch.allclose(lse, ref_l, atol=1e-5)
    full_o, full_l = O.attention_fwd(q.cpu(), k.cpu(), v.cpu(), scale, False, 0)
    assert_bf16_close(acc, full_o, "merged O")
    assert_lse_close(lse, full_l)


def test_natural_log_lse_flag(K, cuda_device):
    q, k, v, _ = _inputs(1, 256, 256, 2, 2, 128, cuda_device)
    _, l2 = K.attn_fwd(q, k, v, 0.1, True, 0)
    _, ln = K.attn_fwd(q, k, v, 0.1, True, 0, lse_natural=True)
    assert torch.allclose(ln, l2 * math.log(2.0), atol=1e-5)


# ------------------------------------------------------------------ combine (tests/test_online_softmax_combine_log2.py)
def test_combine_golden(K, cuda_device):
    import numpy as np
    z = np.load(GOLDEN / "golden_combine.npz")
    t = {k: torch.from_numpy(z[k]).to(cuda_device) for k in z.files}
    for natural, suffix in ((True, "nat"), (False, "log2")):
        for out2 in (t["out2"], t["out2"].bfloat16()):
            out, lse = K.combine(t["out1"], t["lse1"], out2, t["lse2"], natural=natural)
            assert torch.allclose(out, t[f"out_{suffix}"], atol=1e-5, equal_nan=True)
            assert torch.allclose(lse, t[f"lse_{suffix}"], atol=1e-5, equal_nan=True)


def test_combine_partials_matches_pairwise_oracle(K, cuda_device):
    """The one-pass merge of the forward ring: partials that cover different row ranges (the zigzag steps), rows that
    saw no key in some partials (LSE = -inf) or in all of them, against the oracle's pairwise combine in fp32."""
    B, S, H, D = 2, 300, 3, 128
    g = torch.Generator().manual_seed(11)
    spans = [(0, S), (0, S), (150, S - 150), (150, S - 150), (0, S)]
    parts = []
    for i, (r0, rows) in enumerate(spans):
        o = torch.randn(B, rows, H, D, generator=g).bfloat16()
        l = torch.randn(B, H, rows, generator=g) * 3
        if i == 1:
            l[:, :, :40] = -math.inf       # these rows saw no key in this partial
        if i != 2 and i != 3:
            l[:, 1, 7] = -math.inf         # row 7 of head 1: no key anywhere (partials 2, 3 do not cover it)
        parts.append((o, l, r0))
    out, lse = K.combine_partials([(o.to(cuda_device), l.to(cuda_device), r0) for o, l, r0 in parts], B, S, H, D)
    K.check_device_status(cuda_device)
    ref_o = torch.zeros(B, S, H, D)
    ref_l = torch.full((B, H, S), -math.inf)
    for o, l, r0 in parts:
        rows = o.shape[1]
        old_l = ref_l[:, :, r0:r0 + rows]
        co, cl = O.combine(ref_o[:, r0:r0 + rows], old_l, o.float(), l, log2=True)
        dead = (old_l == -math.inf) & (l == -math.inf)          # both sides empty (the formula gives NaN): zeros, -inf
        co = torch.where(dead.permute(0, 2, 1).unsqueeze(-1), torch.zeros_like(co), co)
        cl = torch.where(dead, torch.full_like(cl, -math.inf), cl)
        ref_o[:, r0:r0 + rows] = co
        ref_l[:, :, r0:r0 + rows] = cl
    assert out.dtype == torch.bfloat16 and lse.dtype == torch.float32
    assert_bf16_close(out, ref_o, "combined O", max_abs=1e-2)
    assert_lse_close(lse, ref_l)
    assert (out[:, 7, 1] == 0).all() and torch.isinf(lse[:, 1, 7]).all()


def test_combine_two_halves_identity_commutativity(cuda_device):
    from pithtrain_b200.operators.mla import _mla_fwd
    from pithtrain_b200.operators.ring_attention import _online_softmax_combine, _online_softmax_combine_log2
    B, S, H = 1, 256, 16
    q, k, v, _ = _inputs(B, S // 2, S, H, H, 192, cuda_device, seed=123)
    scale = 192 ** -0.5
    o1, l1 = _mla_fwd(q, k[:, :128], v[:, :128], scale, causal=False)
    o2, l2 = _mla_fwd(q, k[:, 128:], v[:, 128:], scale, causal=False)
    co, cl = _online_softmax_combine_log2(o1, l1, o2, l2)
    assert co.dtype == torch.float32 and co.is_contiguous()
    ro, rl = O.attention_fwd(q.cpu(), k.cpu(), v.cpu(), scale, False)
    assert_bf16_close(co, ro, "two halves")
    assert_lse_close(cl, rl)
    # identity: merging with an empty partial (LSE = -inf) changes nothing
    io, il = _online_softmax_combine_log2(o1, l1, torch.zeros_like(o1), torch.full_like(l1, float("-inf")))
    assert torch.allclose(io, o1.float(), atol=1e-5) and torch.allclose(il, l1, atol=1e-5)
    # commutativity
    ab = _online_softmax_combine_log2(o1, l1, o2, l2)
    ba = _online_softmax_combine_log2(o2, l2, o1, l1)
    assert torch.allclose(ab[0], ba[0], atol=1e-5) and torch.allclose(ab[1], ba[1], atol=1e-5)
    # natural-log variant agrees after converting the LSEs
    no, nl = _online_softmax_combine(o1, l1 * math.log(2.0), o2, l2 * math.log(2.0))
    assert torch.allclose(no, co, atol=1e-5) and torch.allclose(nl, cl * math.log(2.0), atol=1e-4)
    # empty input
    e = torch.empty(1, 0, 2, 128, device=cuda_device)
    eo, el = _online_softmax_combine_log2(e, torch.empty(1, 2, 0, device=cuda_device), e, torch.empty(1, 2, 0, device=cuda_device))
    assert eo.shape == (1, 0, 2, 128) and el.shape == (1, 2, 0)


# ------------------------------------------------------------------ operator layer (CP = 1)
def test_custom_op_autograd_and_mla_module(cuda_device):
    from pithtrain_b200.operators.attention import flash_attn_func
    from pithtrain_b200.operators.mla import MLA
    q, k, v, do = _inputs(1, 512, 512, 8, 2, 128, cuda_device)
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    out = flash_attn_func(q, k, v, softmax_scale=128 ** -0.5, causal=True)
    out.backward(do)
    ref = O.full_attention_fwd_bwd(q.detach().cpu(), k.detach().cpu(), v.detach().cpu(), do.cpu(), 128 ** -0.5)
    assert_bf16_close(out, ref["o"], "O")
    assert_bf16_close(q.grad, ref["dq"], "dQ")
    assert_bf16_close(k.grad, ref["dk"], "dK")
    assert_bf16_close(v.grad, ref["dv"], "dV")
    q, k, v, do = _inputs(1, 256, 256, 16, 16, 192, cuda_device)
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    MLA.autotune(1, 256, 16, 192, 128, 192 ** -0.5)
    out = MLA(16, 192, 128)(q, k, v)
    out.backward(do)
    ref = O.full_attention_fwd_bwd(q.detach().cpu(), k.detach().cpu(), v.detach().cpu(), do.cpu(), 192 ** -0.5)
    assert_bf16_close(out, ref["o"], "MLA O")
    assert_bf16_close(q.grad, ref["dq"], "MLA dQ")
    assert_bf16_close(k.grad, ref["dk"], "MLA dK")
    assert_bf16_close(v.grad, ref["dv"], "MLA dV")


def test_mla_helpers_match_reference_decomposition(cuda_device):
    from pithtrain_b200.operators.mla import _mla_bwd_dk_dv, _mla_bwd_dq, _mla_bwd_preprocess, _mla_fwd
    q, k, v, do = _inputs(2, 512, 512, 16, 16, 192, cuda_device)
    scale = 192 ** -0.5
    for causal in (True, False):
        out, lse = _mla_fwd(q, k, v, scale, causal=causal)
        delta = _mla_bwd_preprocess(out, do)
        dk, dv = _mla_bwd_dk_dv(q, k, v, do, lse, delta, scale, causal=causal)
        dq = _mla_bwd_dq(q, k, v, do, lse, delta, scale, causal=causal)
        ro, rl = O.attention_fwd(q.cpu(), k.cpu(), v.cpu(), scale, causal)
        rdq, rdk, rdv = O.attention_bwd(q.cpu(), k.cpu(), v.cpu(), do.cpu(), rl, O.delta(ro, do.cpu()), scale, causal)
        assert_bf16_close(out, ro, "O"); assert_lse_close(lse, rl)
        assert_bf16_close(dq, rdq, "dQ"); assert_bf16_close(dk, rdk, "dK"); assert_bf16_close(dv, rdv, "dV")


# ------------------------------------------------------------------ full size (Qwen3-30B-A3B layer, S = 8192)
@pytest.fixture(scope="module")
def qwen3_full(K, cuda_device):
    q, k, v, do = _inputs(1, 8192, 8192, 32, 4, 128, cuda_device, seed=42)
    scale = 128 ** -0.5
    out, lse = K.attn_fwd(q, k, v, scale, True, 0)
    delta = K.bwd_preprocess(out, do)
    dq, dk, dv = (torch.zeros(t.shape, device=cuda_device) for t in (q, k, v))
    K.attn_bwd(q, k, v, do, lse, delta, scale, True, 0, dq, dk, dv)
    return dict(q=q, k=k, v=v, do=do, scale=scale, out=out, lse=lse, delta=delta, dq=dq, dk=dk, dv=dv)


def test_full_size_slices_match_oracle(qwen3_full):
    """Rows whose dependencies are small enough for the CPU: the first 256 queries (keys 0..255 only) and the last
    128 queries of two heads against all 8192 keys."""
    f = qwen3_full
    q, k, v = f["q"].cpu(), f["k"].cpu(), f["v"].cpu()
    ro, rl = O.attention_fwd(q[:, :256], k[:, :256], v[:, :256], f["scale"], True, 0)
    assert_bf16_close(f["out"][:, :256], ro, "O[:256]")
    assert_lse_close(f["lse"][:, :, :256], rl)
    heads = [5, 31]
    kv = [h // 8 for h in heads]
    ro, rl = O.attention_fwd(q[:, -128:, heads], k[:, :, kv], v[:, :, kv], f["scale"], True, 8192 - 128)
    assert_bf16_close(f["out"][:, -128:, heads], ro, "O[-128:]")
    assert_lse_close(f["lse"][:, heads, -128:], rl)
    # gradients of the last 128 keys depend on the last 128 queries only
    do = f["do"].cpu()
    o_full, l_full = f["out"].cpu().float(), f["lse"].cpu()
    dl = O.delta(o_full[:, -128:], do[:, -128:])
    _, rdk, rdv = O.attention_bwd(q[:, -128:], k[:, -128:], v[:, -128:], do[:, -128:], l_full[:, :, -128:], dl,
                                  f["scale"], True, 0)
    assert_bf16_close(f["dk"][:, -128:], rdk, "dK[-128:]")
    assert_bf16_close(f["dv"][:, -128:], rdv, "dV[-128:]")
    # dQ of the first 256 queries depends on the first 256 keys only
    dl = O.delta(o_full[:, :256], do[:, :256])
    rdq, _, _ = O.attention_bwd(q[:, :256], k[:, :256], v[:, :256], do[:, :256], l_full[:, :, :256], dl,
                                f["scale"], True, 0)
    assert_bf16_close(f["dq"][:, :256], rdq, "dQ[:256]")


def test_full_size_properties(K, cuda_device, qwen3_full):
    f = qwen3_full
    # softmax rows sum to one: V = 1 gives O = 1 up to bf16 rounding of P
    ones = torch.ones_like(f["v"])
    o1, _ = K.attn_fwd(f["q"], f["k"], ones, f["scale"], True, 0)
    assert (o1.float() - 1).abs().max().item() <= 8e-3
    # scaling V by 2 scales O by exactly 2 (powers of two are exact in bf16 and fp32)
    o2, l2 = K.attn_fwd(f["q"], f["k"], f["v"] * 2, f["scale"], True, 0)
    assert torch.equal(o2, f["out"] * 2) and torch.equal(l2, f["lse"])
    # the backward is linear in dO
    do2 = f["do"] * 2
    delta2 = K.bwd_preprocess(f["out"], do2)
    assert torch.equal(delta2, f["delta"] * 2)
    dq, dk, dv = (torch.zeros_like(f[n]) for n in ("dq", "dk", "dv"))
    K.attn_bwd(f["q"], f["k"], f["v"], do2, f["lse"], delta2, f["scale"], True, 0, dq, dk, dv)
    for a, n in ((dq, "dq"), (dk, "dk"), (dv, "dv")):
        err = (a - 2 * f[n]).abs().max().item()
        assert err <= 1e-3 * f[n].abs().max().item(), (n, err)   # fp32 atomics: summation order differs per run
    # sum over queries of dO equals... dV column sums: sum_n dV[n] = sum_m dO[m] per kv-head group (rows of P sum to 1)
    g = f["do"].float().view(1, 8192, 4, 8, 128).sum(dim=(1, 3))
    assert torch.allclose(f["dv"].sum(dim=1), g, rtol=2e-2, atol=0.5)
    K.check_device_status(cuda_device)


def test_full_size_against_flash_attn(qwen3_full):
    """flash-attn is the arithmetic behind the reference's GQA path (ring_attention/standard.py:26,:91,:134)."""
    fa = pytest.importorskip("flash_attn")
    f = qwen3_full
    q, k, v = (f[n].clone().requires_grad_() for n in ("q", "k", "v"))
    out, lse, _ = fa.flash_attn_func(q, k, v, softmax_scale=f["scale"], causal=True, return_attn_probs=True)
    out.backward(f["do"])
    K = __import__("pithtrain_b200.kernels", fromlist=["x"])
    assert_bf16_close(f["out"], out, "O vs flash-attn")
    assert_lse_close(f["lse"] * math.log(2.0), lse, "LSE vs flash-attn (natural log)")
    assert_bf16_close(K.cast_to_bf16(f["dq"]), q.grad, "dQ vs flash-attn")
    assert_bf16_close(K.cast_to_bf16(f["dk"]), k.grad, "dK vs flash-attn")
    assert_bf16_close(K.cast_to_bf16(f["dv"]), v.grad, "dV vs flash-attn")


# Launches long enough for the dK/dV pass to give one CTA several query heads of a GQA group (its launcher picks 1, 2
# or 4 by a cost model; the small cases above always get 1): a 2:1 group over a long causal launch takes 2, the
# non-causal ring-step shapes of the 8:1 Qwen3 group take 4.
@pytest.mark.parametrize("Sq,Sk,Hq,Hkv,causal", [(4096, 4096, 32, 16, True), (2048, 4096, 32, 4, False),
                                                 (4096, 2048, 32, 4, False)])
def test_several_heads_per_cta_against_flash_attn_and_oracle(K, cuda_device, Sq, Sk, Hq, Hkv, causal):
    fa = pytest.importorskip("flash_attn")
    q, k, v, do = _inputs(1, Sq, Sk, Hq, Hkv, 128, cuda_device, seed=7)
    scale = 128 ** -0.5
    out, lse = K.attn_fwd(q, k, v, scale, causal, 0)
    delta = K.bwd_preprocess(out, do)
    dq, dk, dv = (torch.zeros(t.shape, device=cuda_device) for t in (q, k, v))
    K.attn_bwd(q, k, v, do, lse, delta, scale, causal, 0, dq, dk, dv)
    K.check_device_status(cuda_device)
    qr, kr, vr = (t.clone().requires_grad_() for t in (q, k, v))
    ro = fa.flash_attn_func(qr, kr, vr, softmax_scale=scale, causal=causal)
    ro.backward(do)
    assert_bf16_close(out, ro, "O vs flash-attn")
    assert_bf16_close(K.cast_to_bf16(dq), qr.grad, "dQ vs flash-attn")
    assert_bf16_close(K.cast_to_bf16(dk), kr.grad, "dK vs flash-attn")
    assert_bf16_close(K.cast_to_bf16(dv), vr.grad, "dV vs flash-attn")
    # the last 128 keys of the last kv head against the oracle: every query head of its group adds into them
    g = Hq // Hkv
    heads = list(range(Hq - g, Hq))
    q0 = Sq - 128 if causal else 0  # causal: only the last 128 queries see those keys
    dl = O.delta(out[:, q0:, heads].cpu().float(), do[:, q0:, heads].cpu())
    _, rdk, rdv = O.attention_bwd(q[:, q0:, heads].cpu(), k[:, -128:, -1:].cpu(), v[:, -128:, -1:].cpu(),
                                  do[:, q0:, heads].cpu(), lse[:, heads, q0:].cpu(), dl, scale, causal, 0)
    assert_bf16_close(dk[:, -128:, -1:], rdk, "dK[-128:] vs oracle")
    assert_bf16_close(dv[:, -128:, -1:], rdv, "dV[-128:] vs oracle")


# ----------------------------------------------------------------------------- q/k RMSNorm + rotary embedding
def _qk_golden(dev):
    import numpy as np
    from helpers import bf16_from_bits
    z = np.load(GOLDEN / "golden_qk_norm_rope.npz")
    t = {k: (bf16_from_bits(z[k]) if z[k].dtype == np.uint16 else torch.from_numpy(np.asarray(z[k])))
         for k in z.files}
    return t, float(z["eps"])


@pytest.mark.parametrize("w_dtype,cs_dtype", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32),
                                              (torch.float32, torch.bfloat16)])
def test_qk_norm_rope_golden(cuda_device, w_dtype, cs_dtype):
    """Forward and backward against what the reference's own modules produced (fp32 on CPU)."""
    from pithtrain_b200.operators.qk_norm_rope import qk_norm_rope
    g, eps = _qk_golden(cuda_device)
    dev = cuda_device
    q = g["q"].to(dev).requires_grad_()
    k = g["k"].to(dev).requires_grad_()
    wq = g["q_weight"].to(dev, w_dtype).requires_grad_()   # bf16-exact values
    wk = g["k_weight"].to(dev, w_dtype).requires_grad_()
    cos, sin = g["cos"].to(dev, cs_dtype), g["sin"].to(dev, cs_dtype)
    qe, ke = qk_norm_rope(q, k, wq, wk, cos, sin, eps)
    torch.autograd.backward([qe, ke], [g["dq_embed"].to(dev), g["dk_embed"].to(dev)])
    if cs_dtype == torch.float32:
        ref = g
    else:  # bf16 tables: the expected values are the oracle's on the rounded tables
        from oracle import qk_norm_rope_oracle as R
        c32, s32 = cos.float().cpu(), sin.float().cpu()
        args = (g["q"].float(), g["k"].float(), g["q_weight"].float(), g["k_weight"].float(), c32, s32, eps)
        ref = dict(zip(("q_embed", "k_embed"), R.qk_norm_rope(*args)))
        ref.update(zip(("dq", "dk", "dq_weight", "dk_weight"),
                       R.qk_norm_rope_bwd(*args, g["dq_embed"].float(), g["dk_embed"].float())))
    assert_bf16_close(qe, ref["q_embed"], "q_embed")
    assert_bf16_close(ke, ref["k_embed"], "k_embed")
    assert_bf16_close(q.grad, ref["dq"], "dq")
    assert_bf16_close(k.grad, ref["dk"], "dk")
    for got, name in ((wq.grad, "dq_weight"), (wk.grad, "dk_weight")):
        assert got.dtype == w_dtype
        e = ref[name]
        assert (got.float().cpu() - e).abs().max() <= 2e-2 + 2.0 ** -7 * e.abs().max(), name


def test_qk_norm_rope_full_size_strided(K, cuda_device):
    """The Qwen3 layer's shape (S = 8192, 32 + 4 heads) with q and k as views of one fused projection output (so
    their rows are strided) and one cos/sin table broadcast over the batch; checked against the oracle on a slice
    of positions, plus two size-independent properties: rotation preserves the norm of every row
    (|z| = |y|), and with unit weights every output row has mean square 1."""
    from oracle import qk_norm_rope_oracle as R
    dev = cuda_device
    B, S, Hq, Hkv, D, eps = 1, 8192, 32, 4, 128, 1e-6
    gen = torch.Generator().manual_seed(42)
    qkv = (torch.randn(B, S, (Hq + 2 * Hkv) * D, generator=gen) * 2).bfloat16().to(dev)
    q = qkv[..., :Hq * D].view(B, S, Hq, D)
    k = qkv[..., Hq * D:(Hq + Hkv) * D].view(B, S, Hkv, D)
    wq = (1 + 0.2 * torch.randn(D, generator=gen)).bfloat16().to(dev)
    wk = (1 + 0.2 * torch.randn(D, generator=gen)).bfloat16().to(dev)
    cos, sin = (t.bfloat16().to(dev) for t in R.rope_tables(torch.arange(S) + 24576, D))
    dqe = torch.randn(B, S, Hq, D, generator=gen).bfloat16().to(dev)
    dke = torch.randn(B, S, Hkv, D, generator=gen).bfloat16().to(dev)
    qe, ke = K.qk_norm_rope_fwd(q, k, wq, wk, cos, sin, eps)
    dq, dk, dwq, dwk = K.qk_norm_rope_bwd(q, k, wq, wk, cos, sin, eps, dqe, dke)
    assert qe.is_contiguous() and ke.is_contiguous()
    sl = slice(4000, 4128)
    args = [t.float().cpu() for t in (q[:, sl], k[:, sl], wq, wk, cos[:, sl], sin[:, sl])]
    rq, rk = R.qk_norm_rope(*args, eps)
    assert_bf16_close(qe[:, sl], rq, "q_embed slice")
    assert_bf16_close(ke[:, sl], rk, "k_embed slice")
    rdq, rdk, _, _ = R.qk_norm_rope_bwd(*args, eps, dqe[:, sl].float().cpu(), dke[:, sl].float().cpu())
    assert_bf16_close(dq[:, sl], rdq, "dq slice")
    assert_bf16_close(dk[:, sl], rdk, "dk slice")
    # weight gradients over ALL rows, against a float64 reduction on the GPU of the same closed form
    for x, g, w, got in ((q, dqe, wq, dwq), (k, dke, wk, dwk)):
        x64, g64 = x.double(), g.double()
        c, s = cos.double().unsqueeze(2), sin.double().unsqueeze(2)
        t = g64 * s
        dy = g64 * c + torch.cat((t[..., 64:], -t[..., :64]), dim=-1)
        xh = x64 * torch.rsqrt(x64.pow(2).mean(-1, keepdim=True) + eps)
        want = (dy * xh).sum((0, 1, 2))
        assert (got.double() - want).abs().max() <= 1e-3 * want.abs().max() + 1e-2
    # properties at full size
    ones = torch.ones(D, dtype=torch.bfloat16, device=dev)
    q1, k1 = K.qk_norm_rope_fwd(q, k, ones, ones, cos, sin, eps)
    for z in (q1, k1):
        ms = z.float().pow(2).mean(-1)
        assert (ms - 1).abs().max() < 2e-2          # rotation keeps |y|, and |y|^2 / D = 1 after the norm
    K.check_device_status(dev)


def test_qk_norm_rope_edges(K, cuda_device):
    """Empty tensors, a row count that is not a multiple of the 16 rows a block handles at a time, zero rows
    (finite output thanks to eps), and rejected arguments."""
    dev = cuda_device
    w = torch.ones(128, dtype=torch.bfloat16, device=dev)
    cs = torch.ones(1, 0, 128, dtype=torch.bfloat16, device=dev)
    e = torch.empty(1, 0, 2, 128, dtype=torch.bfloat16, device=dev)
    qe, ke = K.qk_norm_rope_fwd(e, e, w, w, cs, cs, 1e-6)
    assert qe.shape == e.shape and ke.shape == e.shape
    from oracle import qk_norm_rope_oracle as R
    q = torch.randn(3, 7, 5, 128).bfloat16().to(dev)
    k = torch.zeros(3, 7, 1, 128, dtype=torch.bfloat16, device=dev)
    cos, sin = (t.to(dev) for t in R.rope_tables(torch.arange(7), 128))
    qe, ke = K.qk_norm_rope_fwd(q, k, w, w, cos, sin, 1e-6)
    rq, _ = R.qk_norm_rope(q.float().cpu(), k.float().cpu(), w.float().cpu(), w.float().cpu(), cos.cpu(), sin.cpu(),
                           1e-6)
    assert_bf16_close(qe, rq, "ragged q_embed")
    assert torch.equal(ke, torch.zeros_like(ke))
    with pytest.raises(RuntimeError, match="128 only"):
        K.qk_norm_rope_fwd(q[..., :64].contiguous(), k[..., :64].contiguous(), w[:64].contiguous(),
                           w[:64].contiguous(), cos[..., :64].contiguous(), sin[..., :64].contiguous(), 1e-6)
    with pytest.raises(ValueError):
        K.qk_norm_rope_fwd(q, k, w, w, cos[:, :5], sin[:, :5], 1e-6)


# ----------------------------------------------------------------------------- MLA rotary + input assembly
@pytest.mark.parametrize("cs_dtype", [torch.float32, torch.bfloat16])
def test_mla_assemble_golden(cuda_device, cs_dtype):
    """Forward and backward against what the reference's own functions produced (fp32 on CPU)."""
    import numpy as np
    from helpers import bf16_from_bits
    from oracle import mla_assemble_oracle as M
    from pithtrain_b200.operators.mla import mla_assemble
    z = np.load(GOLDEN / "golden_mla_assemble.npz")
    g = {k: (bf16_from_bits(z[k]) if z[k].dtype == np.uint16 else torch.from_numpy(np.asarray(z[k]))) for k in z.files}
    dev = cuda_device
    q, kv = g["q"].to(dev).requires_grad_(), g["kv"].to(dev).requires_grad_()
    k_pe = g["k_pe"].to(dev).unsqueeze(2).requires_grad_()           # [B,S,1,64] as the layer has it
    cos, sin = g["cos"].to(dev, cs_dtype), g["sin"].to(dev, cs_dtype)
    query, key, value = mla_assemble(q, kv, k_pe, cos, sin)
    torch.autograd.backward([query, key, value], [g[n].to(dev) for n in ("dquery", "dkey", "dvalue")])
    if cs_dtype == torch.float32:
        ref = g
    else:
        args = (g["q"].float(), g["kv"].float(), g["k_pe"].float(), cos.float().cpu(), sin.float().cpu())
        ref = dict(zip(("query", "key", "value"), M.mla_assemble(*args)))
        ref.update(zip(("dq", "dkv", "dk_pe"), M.mla_assemble_bwd(*args, g["dquery"].float(), g["dkey"].float(),
                                                                  g["dvalue"].float())))
    assert_bf16_close(query, ref["query"], "query")
    assert_bf16_close(key, ref["key"], "key")
    assert torch.equal(value.cpu(), g["kv"][..., 128:])               # a pure copy: bit-exact
    assert torch.equal(query[..., :128].cpu(), g["q"][..., :128])
    assert torch.equal(key[..., :128].cpu(), g["kv"][..., :128])
    assert_bf16_close(q.grad, ref["dq"], "dq")
    assert_bf16_close(kv.grad, ref["dkv"], "dkv")
    assert k_pe.grad.shape == k_pe.shape
    assert_bf16_close(k_pe.grad[:, :, 0], ref["dk_pe"], "dk_pe")


def test_mla_assemble_full_size(K, cuda_device):
    """DeepSeek-V2-Lite's shape at 4096 tokens per rank with strided inputs (q and kv as views of wider projection
    outputs, k_pe as the tail of the compressed-kv projection), the rotary tables given with position_ids as the
    reference passes them; oracle on a slice, plus: rotation preserves the norm of every rope row, the rope part of
    key is the same for all heads, and dk_pe equals the head-sum property (zero dkey rope part -> zero dk_pe)."""
    from oracle import mla_assemble_oracle as M
    from pithtrain_b200.operators.mla import mla_assemble
    dev = cuda_device
    B, S, H = 1, 4096, 16
    gen = torch.Generator().manual_seed(5)
    qbuf = torch.randn(B, S, H * 192 + 64, generator=gen).bfloat16().to(dev)
    kvbuf = torch.randn(B, S, H * 256, generator=gen).bfloat16().to(dev)
    ckv = torch.randn(B, S, 512 + 64, generator=gen).bfloat16().to(dev)
    q = qbuf[..., :H * 192].view(B, S, H, 192)
    kv = kvbuf.view(B, S, H, 256)
    k_pe = ckv[..., 512:].view(B, S, 1, 64)
    pos = torch.arange(S, device=dev).view(1, S) + 28672
    inv = 1.0 / (10000 ** (torch.arange(0, 64, 2, dtype=torch.float32, device=dev) / 64))
    emb = torch.outer(torch.arange(32768, dtype=torch.float32, device=dev), inv).repeat(1, 2)
    cos_t, sin_t = (emb.cos() * 1.1).bfloat16(), (emb.sin() * 1.1).bfloat16()
    query, key, value = mla_assemble(q, kv, k_pe, cos_t, sin_t, pos)
    assert query.is_contiguous() and key.is_contiguous() and value.is_contiguous()
    sl = slice(1000, 1064)
    cos_g, sin_g = cos_t[pos][:, sl].float().cpu(), sin_t[pos][:, sl].float().cpu()
    rq, rk, rv = M.mla_assemble(q[:, sl].float().cpu(), kv[:, sl].float().cpu(), k_pe[:, sl, 0].float().cpu(), cos_g, sin_g)
    assert_bf16_close(query[:, sl], rq, "query slice")
    assert_bf16_close(key[:, sl], rk, "key slice")
    assert torch.equal(value.cpu(), kv[..., 128:].cpu())
    assert torch.equal(key[..., 128:], key[:, :, :1, 128:].expand(-1, -1, H, -1))
    # |rope(x)|^2 = 1.1^2 |x|^2 up to bf16 rounding of the tables and the outputs
    n_in = q[..., 128:].float().pow(2).sum(-1)
    n_out = query[..., 128:].float().pow(2).sum(-1)
    assert ((n_out / n_in).sqrt() - 1.1).abs().max() < 2e-2
    dquery = torch.randn(B, S, H, 192, generator=gen).bfloat16().to(dev)
    dkey = torch.randn(B, S, H, 192, generator=gen).bfloat16().to(dev)
    dvalue = torch.randn(B, S, H, 128, generator=gen).bfloat16().to(dev)
    dq, dkv, dk_pe = K.mla_assemble_bwd(cos_t[pos], sin_t[pos], dquery, dkey, dvalue)
    rdq, rdkv, rdkpe = M.mla_assemble_bwd(q[:, sl].float().cpu(), kv[:, sl].float().cpu(), k_pe[:, sl, 0].float().cpu(),
                                          cos_g, sin_g, dquery[:, sl].float().cpu(), dkey[:, sl].float().cpu(),
                                          dvalue[:, sl].float().cpu())
    assert_bf16_close(dq[:, sl], rdq, "dq slice")
    assert_bf16_close(dkv[:, sl], rdkv, "dkv slice")
    # dk_pe sums 16 heads: its entries are ~4x larger, so its share of bf16 rounding in the mean is too
    assert_bf16_close(dk_pe[:, sl], rdkpe, "dk_pe slice", mean_abs=2e-3 + 2.0 ** -9 * rdkpe.abs().mean().item())
    dkey0 = dkey.clone()
    dkey0[..., 128:] = 0
    assert not K.mla_assemble_bwd(cos_t[pos], sin_t[pos], dquery, dkey0, dvalue)[2].any()
    # empty input and rejected sizes
    e = torch.empty(1, 0, H, 192, dtype=torch.bfloat16, device=dev)
    out = K.mla_assemble_fwd(e, torch.empty(1, 0, H, 256, dtype=torch.bfloat16, device=dev),
                             torch.empty(1, 0, 64, dtype=torch.bfloat16, device=dev),
                             torch.empty(1, 0, 64, device=dev), torch.empty(1, 0, 64, device=dev))
    assert out[0].shape == (1, 0, H, 192)
    with pytest.raises(ValueError):
        K.mla_assemble_fwd(q[..., :128], kv, k_pe, cos_t[pos], sin_t[pos])
    K.check_device_status(dev)


@pytest.mark.parametrize("Sq,Sk,causal,off", [(512, 512, True, 0), (384, 640, False, 0), (200, 333, True, 133),
                                              (512, 256, True, -300)])
def test_backward_direct_dq_store(K, cuda_device, Sq, Sk, causal, off):
    """PITH_BWD_DQ_STORE_BF16: the dQ pass stores bf16 directly. Must equal the rounded fp32 accumulator bit for bit
    (one CTA owns a row block, so the sum is the same), including rows that see no key at all (zeros) and ragged
    tile edges; and it must not touch dK/dV."""
    dev = cuda_device
    q, k, v, do = _inputs(1, Sq, Sk, 8, 2, 128, dev, seed=7)
    scale = 128 ** -0.5
    o, lse = K.attn_fwd(q, k, v, scale, causal, off)
    lse = torch.nan_to_num(lse, nan=0.0, neginf=0.0)  # rows without keys: any finite value, their P is masked anyway
    o = torch.nan_to_num(o)
    delta = K.bwd_preprocess(o, do)
    acc = [torch.zeros(t.shape, dtype=torch.float32, device=dev) for t in (q, k, v)]
    K.attn_bwd(q, k, v, do, lse, delta, scale, causal, off, acc[0], acc[1], acc[2])
    dq = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device=dev)
    dk2, dv2 = (torch.zeros_like(t) for t in acc[1:])
    K.attn_bwd(q, k, v, do, lse, delta, scale, causal, off, None, dk2, dv2, dq_out=dq)
    assert torch.equal(dq, acc[0].bfloat16())
    assert torch.allclose(dk2, acc[1], atol=1e-4, rtol=1e-4) and torch.allclose(dv2, acc[2], atol=1e-4, rtol=1e-4)
    if off < 0:
        assert not dq[:, : -off].any()  # queries before the first visible key
    with pytest.raises(ValueError):
        K.attn_bwd(q, k, v, do, lse, delta, scale, causal, off, acc[0], None, None, dq_out=dq)
