"""Host-side behaviour of the operator layer that needs no GPU: API surface, argument checks, loud failure on
CPU tensors (there is no CPU fallback), and the CP plumbing helpers."""

import inspect

import pytest
import torch

from pithtrain_b200.modules import distributed as D
from pithtrain_b200.operators import attention, mla, ring_attention
from pithtrain_b200.operators.ring_attention import mla as ring_mla
from pithtrain_b200.operators.ring_attention import standard


def test_reference_names_and_argument_order():
    assert list(inspect.signature(standard.ring_attention_func).parameters)[:5] == \
        ["q", "k", "v", "softmax_scale", "cp_group"]
    assert list(inspect.signature(ring_mla.ring_mla_attention_func).parameters)[:5] == \
        ["q", "k", "v", "softmax_scale", "cp_group"]
    assert list(inspect.signature(standard._online_softmax_combine).parameters) == ["out1", "lse1", "out2", "lse2"]
    assert list(inspect.signature(ring_mla._online_softmax_combine_log2).parameters) == ["out1", "lse1", "out2", "lse2"]
    assert list(inspect.signature(standard._ring_send_recv_kv).parameters) == \
        ["send_k", "send_v", "next_global", "prev_global"]
    assert list(inspect.signature(mla.MLA.__init__).parameters) == ["self", "h", "dq", "dv", "softmax_scale"]
    assert list(inspect.signature(mla.MLA.autotune).parameters) == \
        ["b", "s", "h", "dq", "dv", "softmax_scale", "include_non_causal"]
    for name in ("_mla_fwd", "_mla_bwd_preprocess", "_mla_bwd_dk_dv", "_mla_bwd_dq"):
        assert hasattr(mla, name)
    for name in ("RingAttentionFunc", "RingMLAAttentionFunc", "ring_attention_func", "ring_mla_attention_func"):
        assert hasattr(ring_attention, name)


def test_mla_module_default_scale():
    m = mla.MLA(16, 192, 128)
    assert abs(m.softmax_scale - 192 ** -0.5) < 1e-12
    assert mla.MLA(16, 192, 128, 0.25).softmax_scale == 0.25
    with pytest.raises(AssertionError):
        mla.MLA.autotune(1, 128, 16, 128, 128, 0.1)


def test_no_cpu_fallback(built_library):
    q = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        attention.flash_attn_func(q, q, q, causal=True)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        standard._online_softmax_combine(q.float(), torch.zeros(1, 2, 128), q.float(), torch.zeros(1, 2, 128))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        standard.RingAttentionFunc.apply(q, q, q, 0.1, 0, 1, [0])
    with pytest.raises(NotImplementedError):
        attention.flash_attn_func(q, q, q, dropout_p=0.1)
    from pithtrain_b200.operators.qk_norm_rope import qk_norm_rope
    w, cs = torch.ones(128), torch.ones(1, 128, 128)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        qk_norm_rope(q, q, w, w, cs, cs, 1e-6)
    from pithtrain_b200.operators.mla import mla_assemble
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        mla_assemble(torch.zeros(1, 8, 2, 192, dtype=torch.bfloat16), torch.zeros(1, 8, 2, 256, dtype=torch.bfloat16),
                     torch.zeros(1, 8, 1, 64, dtype=torch.bfloat16), torch.ones(1, 8, 64), torch.ones(1, 8, 64))


def test_contiguity_assertion_matches_reference_message():
    k = torch.zeros(1, 128, 4, 128, dtype=torch.bfloat16).transpose(1, 2).transpose(1, 2)[:, ::2]
    q = torch.zeros(1, 64, 4, 128, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="ring attention k or v is not contiguous"):
        standard.RingAttentionFunc.apply(q, k, k, 0.1, 0, 1, [0])
    with pytest.raises(AssertionError, match="ring MLA attention k or v is not contiguous"):
        ring_mla.RingMLAAttentionFunc.apply(q, k, k, 0.1, 0, 1, [0])


def test_cp_batch_slicing_and_positions():
    tokens = torch.arange(2 * 32).view(2, 32)
    labels = tokens + 1
    t, l = D.shard_batch_for_cp(tokens, labels, 1, 4, "contiguous")
    assert torch.equal(t, tokens[:, 8:16]) and torch.equal(l, labels[:, 8:16])
    t, l = D.shard_batch_for_cp(tokens, labels, 1, 4, "zigzag")
    assert torch.equal(t, torch.cat([tokens[:, 4:8], tokens[:, 24:28]], 1))
    assert torch.equal(D.cp_position_ids(8, 1, 4, "contiguous"), torch.arange(8, 16).unsqueeze(0))
    assert torch.equal(D.cp_position_ids(8, 1, 4, "zigzag")[0], torch.cat([torch.arange(4, 8), torch.arange(24, 28)]))
    assert D.shard_batch_for_cp(tokens, labels, 0, 1)[0] is tokens
    with pytest.raises(AssertionError, match="must be divisible"):
        D.check_sequence_length(30, 4)
    with pytest.raises(AssertionError, match="2 \\* context_parallel_size"):
        D.check_sequence_length(36, 8, "zigzag")
    assert D.use_ring_attn(None) is False
    loss = torch.tensor(3.0)
    assert D.average_loss_over_cp(loss, None, 1) is loss
