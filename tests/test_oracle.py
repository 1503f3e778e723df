"""The CPU oracle against the golden vectors produced by the reference's own code, and against itself."""

import numpy as np
import pytest
import torch

from helpers import GOLDEN, load_golden_attention
from oracle import attention_oracle as O


def test_combine_matches_reference_golden():
    z = np.load(GOLDEN / "golden_combine.npz")
    t = {k: torch.from_numpy(z[k]) for k in z.files}
    for log2, suffix in ((False, "nat"), (True, "log2")):
        out, lse = O.combine(t["out1"], t["lse1"], t["out2"], t["lse2"], log2=log2)
        assert torch.allclose(out, t[f"out_{suffix}"], rtol=0, atol=1e-6, equal_nan=True)
        assert torch.allclose(lse, t[f"lse_{suffix}"], rtol=0, atol=1e-6, equal_nan=True)


@pytest.mark.parametrize("name", ["mla_causal", "mla_full", "d128_causal"])
def test_attention_matches_reference_golden(name):
    g = load_golden_attention(name)
    q, k, v, do = (g[x].float() for x in ("q", "k", "v", "do"))
    o, lse = O.attention_fwd(q, k, v, g["scale"], g["causal"])
    assert torch.allclose(o, g["o"], rtol=1e-5, atol=2e-6)
    dl = O.delta(o, do)
    dq, dk, dv = O.attention_bwd(q, k, v, do, lse, dl, g["scale"], g["causal"])
    assert torch.allclose(dq, g["dq"], rtol=1e-4, atol=2e-5)
    assert torch.allclose(dk, g["dk"], rtol=1e-4, atol=2e-5)
    assert torch.allclose(dv, g["dv"], rtol=1e-4, atol=2e-5)


def _config1():
    """B=1, S=1024, Hq=8, Hkv=2, D=64, N(0,1) from seed 0, scale 1/sqrt(64)."""
    torch.manual_seed(0)
    q = torch.randn(1, 1024, 8, 64)
    k = torch.randn(1, 1024, 2, 64)
    v = torch.randn(1, 1024, 2, 64)
    do = torch.randn(1, 1024, 8, 64)
    return q, k, v, do, 64 ** -0.5


def test_config1_split_kv_combine_equals_full_attention():
    """KV split into two chunks, each attended separately, merged with the log2 combine, equals full attention
    for O, LSE, dQ, dK and dV."""
    q, k, v, do, scale = _config1()
    full = O.full_attention_fwd_bwd(q, k, v, do, scale)
    # the second chunk is entirely in the future of the first 512 queries: rows with no visible key give LSE=-inf
    o1, l1 = O.attention_fwd(q, k[:, :512], v[:, :512], scale, True, 0)
    o2, l2 = O.attention_fwd(q, k[:, 512:], v[:, 512:], scale, True, -512)
    o, lse = O.combine(o1, l1, o2, l2, log2=True)
    assert torch.allclose(o, full["o"], atol=2e-6)
    assert torch.allclose(lse, full["lse_log2"], atol=1e-5)
    dl = O.delta(o, do)
    dq1, dk1, dv1 = O.attention_bwd(q, k[:, :512], v[:, :512], do, lse, dl, scale, True, 0)
    dq2, dk2, dv2 = O.attention_bwd(q, k[:, 512:], v[:, 512:], do, lse, dl, scale, True, -512)
    assert torch.allclose(dq1 + dq2, full["dq"], atol=2e-5)
    assert torch.allclose(torch.cat([dk1, dk2], 1), full["dk"], atol=2e-5)
    assert torch.allclose(torch.cat([dv1, dv2], 1), full["dv"], atol=2e-5)


def test_backward_formulas_match_autograd():
    torch.manual_seed(3)
    q = torch.randn(2, 64, 4, 32, dtype=torch.float64, requires_grad=True)
    k = torch.randn(2, 64, 2, 32, dtype=torch.float64, requires_grad=True)
    v = torch.randn(2, 64, 2, 16, dtype=torch.float64, requires_grad=True)
    do = torch.randn(2, 64, 4, 16, dtype=torch.float64)
    o, _ = O.attention_fwd(q, k, v, 0.2, True, 0, torch.float64)
    o.backward(do)
    r = O.full_attention_fwd_bwd(q.detach(), k.detach(), v.detach(), do, 0.2, torch.float64)
    for a, b in ((r["dq"], q.grad), (r["dk"], k.grad), (r["dv"], v.grad)):
        assert torch.allclose(a, b, atol=1e-10)


@pytest.mark.parametrize("cp", [2, 4])
def test_ring_schedules_equal_full_attention(cp):
    torch.manual_seed(42)
    S = 128
    q = torch.randn(1, S, 4, 32, dtype=torch.float64)
    k = torch.randn(1, S, 2, 32, dtype=torch.float64)
    v = torch.randn(1, S, 2, 32, dtype=torch.float64)
    do = torch.randn(1, S, 4, 32, dtype=torch.float64)
    full = O.full_attention_fwd_bwd(q, k, v, do, 0.3, torch.float64)
    idx = [O.contiguous_indices(S, cp, r) for r in range(cp)]
    outs, _ = O.ring_contiguous_fwd([q[:, i] for i in idx], [k[:, i] for i in idx], [v[:, i] for i in idx], 0.3,
                                    log2=True, dtype=torch.float64)
    for r in range(cp):
        assert torch.allclose(outs[r], full["o"][:, idx[r]], atol=1e-12)
    idx = [O.zigzag_indices(S, cp, r) for r in range(cp)]
    sh = lambda t: [t[:, i] for i in idx]  # noqa: E731
    outs, lses = O.ring_zigzag_fwd(sh(q), sh(k), sh(v), 0.3, torch.float64)
    dqs, dks, dvs = O.ring_zigzag_bwd(sh(q), sh(k), sh(v), sh(do), outs, lses, 0.3, torch.float64)
    for r in range(cp):
        assert torch.allclose(outs[r], full["o"][:, idx[r]], atol=1e-12)
        assert torch.allclose(lses[r], full["lse_log2"][:, :, idx[r]], atol=1e-12)
        assert torch.allclose(dqs[r], full["dq"][:, idx[r]], atol=1e-12)
        assert torch.allclose(dks[r], full["dk"][:, idx[r]], atol=1e-12)
        assert torch.allclose(dvs[r], full["dv"][:, idx[r]], atol=1e-12)


def test_flop_conventions():
    # Qwen3-30B-A3B attention at S=8192: 5.498e11 forward, x3.5 for forward + backward
    assert abs(O.fwd_flops(1, 32, 8192, 128, 128) - 5.498e11) / 5.498e11 < 1e-3
    assert abs(O.fwd_bwd_flops(1, 32, 8192, 128, 128) - 1.924e12) / 1.924e12 < 1e-3


def _golden_qk():
    from helpers import bf16_from_bits
    z = np.load(GOLDEN / "golden_qk_norm_rope.npz")
    t = {k: (bf16_from_bits(z[k]) if z[k].dtype == np.uint16 else torch.from_numpy(np.asarray(z[k])))
         for k in z.files}
    t["eps"] = float(z["eps"])
    return t


def test_qk_norm_rope_matches_reference_golden():
    """The oracle against nn.RMSNorm + the reference's apply_rotary_pos_emb (fp32 on CPU, with autograd), and the
    oracle's cos/sin tables against Qwen3MoeRotaryEmbedding's."""
    from oracle import qk_norm_rope_oracle as R
    g = _golden_qk()
    q, k, wq, wk = (g[x].float() for x in ("q", "k", "q_weight", "k_weight"))
    qe, ke = R.qk_norm_rope(q, k, wq, wk, g["cos"], g["sin"], g["eps"])
    assert torch.allclose(qe, g["q_embed"], rtol=1e-5, atol=2e-6)
    assert torch.allclose(ke, g["k_embed"], rtol=1e-5, atol=2e-6)
    dq, dk, dwq, dwk = R.qk_norm_rope_bwd(q, k, wq, wk, g["cos"], g["sin"], g["eps"], g["dq_embed"].float(),
                                          g["dk_embed"].float())
    for got, name in ((dq, "dq"), (dk, "dk"), (dwq, "dq_weight"), (dwk, "dk_weight")):
        assert torch.allclose(got, g[name], rtol=1e-4, atol=2e-5), name
    for b in range(2):
        cos, sin = R.rope_tables(g["position_ids"][b], 128)
        assert torch.allclose(cos[0], g["cos"][b], atol=1e-6) and torch.allclose(sin[0], g["sin"][b], atol=1e-6)
    # the reference's own bf16 flow (a rounding after every elementwise kernel) stays within bf16 rounding of it
    assert (g["q_embed_bf16"].float() - qe).abs().max() <= 3 * 2.0 ** -8 * qe.abs().max()
    assert (g["k_embed_bf16"].float() - ke).abs().max() <= 3 * 2.0 ** -8 * ke.abs().max()


def test_qk_norm_rope_backward_formula():
    """The closed form the CUDA backward uses (dy = dz*cos + rotate_half^T(dz*sin); dx = r*(g - xhat*mean(g*xhat)),
    g = dy*w; dw = sum dy*xhat) against autograd through the oracle, in fp64."""
    from oracle import qk_norm_rope_oracle as R
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(2, 5, 3, 128, generator=gen, dtype=torch.float64)
    w = 1 + 0.3 * torch.randn(128, generator=gen, dtype=torch.float64)
    cos, sin = R.rope_tables(torch.arange(5) * 11, 128, dtype=torch.float64)
    dz = torch.randn(x.shape, generator=gen, dtype=torch.float64)
    dx_ref, _, dw_ref, _ = R.qk_norm_rope_bwd(x, x, w, w, cos, sin, 1e-6, dz, torch.zeros_like(dz))
    c, s = cos.unsqueeze(2), sin.unsqueeze(2)
    t = dz * s
    dy = dz * c + torch.cat((t[..., 64:], -t[..., :64]), dim=-1)
    r = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)
    xh = x * r
    g = dy * w
    dx = r * (g - xh * (g * xh).mean(-1, keepdim=True))
    assert torch.allclose(dx, dx_ref, rtol=1e-10, atol=1e-12)
    assert torch.allclose((dy * xh).sum((0, 1, 2)), dw_ref, rtol=1e-10, atol=1e-12)


def _golden_npz(name):
    from helpers import bf16_from_bits
    z = np.load(GOLDEN / name)
    return {k: (bf16_from_bits(z[k]) if z[k].dtype == np.uint16 else torch.from_numpy(np.asarray(z[k])))
            for k in z.files}


def test_mla_assemble_matches_reference_golden():
    """The oracle against the reference's apply_rotary_pos_emb (DeepSeek form) + the layer's assembly statements,
    fp32 on CPU with autograd."""
    from oracle import mla_assemble_oracle as M
    g = _golden_npz("golden_mla_assemble.npz")
    q, kv, k_pe = g["q"].float(), g["kv"].float(), g["k_pe"].float()
    query, key, value = M.mla_assemble(q, kv, k_pe, g["cos"], g["sin"])
    for got, name in ((query, "query"), (key, "key"), (value, "value")):
        assert torch.allclose(got, g[name], rtol=1e-6, atol=1e-6), name
    grads = M.mla_assemble_bwd(q, kv, k_pe, g["cos"], g["sin"], g["dquery"].float(), g["dkey"].float(),
                               g["dvalue"].float())
    for got, name in zip(grads, ("dq", "dkv", "dk_pe")):
        assert torch.allclose(got, g[name], rtol=1e-5, atol=1e-5), name
