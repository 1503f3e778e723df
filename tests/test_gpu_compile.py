"""The CP = 1 operators inside ``torch.compile(fullgraph=True)``: the reference compiles the region that contains its
attention call (pithtrain/models/qwen3_30b_a3b.py:518 around flash_attn_func at :424; the Triton MLA custom op at
pithtrain/operators/mla/triton.py:445-508), so the replacements must trace without a graph break and their fake
kernels must describe the real outputs (shape, dtype, strides)."""

import pytest
import torch

from helpers import assert_bf16_close

pytestmark = pytest.mark.gpu


def _run(fn, inputs, do):
    leaves = [t.detach().clone().requires_grad_() for t in inputs]
    out = fn(*leaves)
    out.backward(do)
    return out.detach(), [t.grad for t in leaves]


@pytest.mark.parametrize("kind", ["gqa", "mla"])
def test_fullgraph_compile_matches_eager(cuda_device, kind):
    from pithtrain_b200.operators.attention import flash_attn_func
    from pithtrain_b200.operators.mla import MLA
    g = torch.Generator().manual_seed(9)
    if kind == "gqa":
        S, Hq, Hkv, Dqk = 512, 8, 2, 128
        scale = Dqk ** -0.5
        fn = lambda q, k, v: flash_attn_func(q * 1.0, k, v, softmax_scale=scale, causal=True) + 0.0  # noqa: E731
    else:
        S, Hq, Hkv, Dqk = 512, 4, 4, 192
        mla = MLA(Hq, Dqk, 128)
        fn = lambda q, k, v: mla(q * 1.0, k, v) + 0.0  # noqa: E731
    q = torch.randn(1, S, Hq, Dqk, generator=g).bfloat16().to(cuda_device)
    k = torch.randn(1, S, Hkv, Dqk, generator=g).bfloat16().to(cuda_device)
    v = torch.randn(1, S, Hkv, 128, generator=g).bfloat16().to(cuda_device)
    do = torch.randn(1, S, Hq, 128, generator=g).bfloat16().to(cuda_device)
    eager_out, eager_grads = _run(fn, (q, k, v), do)
    compiled = torch.compile(fn, fullgraph=True)  # raises on any graph break
    out, grads = _run(compiled, (q, k, v), do)
    assert out.shape == eager_out.shape and out.dtype == torch.bfloat16 and out.stride() == eager_out.stride()
    assert torch.equal(out, eager_out)  # the forward is deterministic
    for name, a, b in zip(("dq", "dk", "dv"), grads, eager_grads):
        assert a.shape == b.shape and a.dtype == b.dtype
        assert_bf16_close(a, b, name + " (compiled vs eager)")  # fp32 atomics: last bits may differ


def test_fake_kernels_describe_the_real_outputs(cuda_device):
    from pithtrain_b200.operators.attention import attn_bwd_op, attn_fwd_op
    q = torch.zeros(2, 256, 8, 128, dtype=torch.bfloat16, device=cuda_device)
    k = torch.zeros(2, 256, 2, 128, dtype=torch.bfloat16, device=cuda_device)
    torch.library.opcheck(attn_fwd_op, (q, k, k, 0.1, True), test_utils=("test_schema", "test_faketensor"))
    o, lse = attn_fwd_op(q, k, k, 0.1, True)
    torch.library.opcheck(attn_bwd_op, (q, k, k, o, lse, o, 0.1, True), test_utils=("test_schema", "test_faketensor"))
