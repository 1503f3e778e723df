"""How the operators share the GPU with work on other streams, and how device-side anomalies reach the host.

DualPipeV runs expert-parallel all-to-all traffic on its own ``comm_stream`` (pithtrain/dualpipe/dualpipev.py:87,
waited for at pithtrain/dualpipe/execution.py:152-158) while attention runs on the default stream. The attention
backward forks a side stream of its own (dQ pass beside the dK/dV pass); these tests check that a third stream at
default priority keeps making progress next to it, that attention is not held up by more than that stream's own
work, and that on return everything the operator launched is ordered before later work on the caller's stream.
"""

import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ms(fn, stream=None):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s = stream or torch.cuda.current_stream()
    e0.record(s)
    fn()
    e1.record(s)
    return e0, e1


def test_backward_side_stream_coexists_with_a_comm_like_stream(cuda_device):
    from pithtrain_b200 import _lib, kernels as K
    g = torch.Generator().manual_seed(3)
    B, S, Hq, Hkv, D = 1, 4096, 32, 4, 128
    q = torch.randn(B, S, Hq, D, generator=g).bfloat16().to(cuda_device)
    k = torch.randn(B, S, Hkv, D, generator=g).bfloat16().to(cuda_device)
    v = torch.randn(B, S, Hkv, D, generator=g).bfloat16().to(cuda_device)
    do = torch.randn(B, S, Hq, D, generator=g).bfloat16().to(cuda_device)
    scale = D ** -0.5
    out, lse = K.attn_fwd(q, k, v, scale, True, 0)
    delta = K.bwd_preprocess(out, do)
    dq, dk, dv = (torch.zeros(t.shape, device=cuda_device) for t in (q, k, v))
    comm_stream = torch.cuda.Stream()                       # default priority, like dualpipev.py:87
    a = torch.ones(64 << 20, device=cuda_device)             # 256 MB per pass: stands in for all-to-all traffic
    b = torch.empty_like(a)

    def attention(n=8):
        for _ in range(n):  # both passes side by side: the library's own side stream is in play
            K.attn_bwd(q, k, v, do, lse, delta, scale, True, 0, dq, dk, dv, serial=False)

    def traffic(n=12):
        with torch.cuda.stream(comm_stream):
            for _ in range(n):
                torch.add(a, 1.0, out=b)

    attention(2); traffic(2)
    torch.cuda.synchronize()
    ea = _ms(attention); torch.cuda.synchronize(); t_attn = ea[0].elapsed_time(ea[1])
    ec = _ms(traffic, comm_stream); torch.cuda.synchronize(); t_comm = ec[0].elapsed_time(ec[1])
    # both at once
    comm_stream.wait_stream(torch.cuda.current_stream())
    ec = _ms(traffic, comm_stream)
    ea = _ms(attention)
    torch.cuda.synchronize()
    both_attn, both_comm = ea[0].elapsed_time(ea[1]), ec[0].elapsed_time(ec[1])
    # neither side is starved: each finishes within the serial sum (plus scheduling slack), not after the other's
    # whole backlog plus its own
    assert both_attn <= (t_attn + t_comm) * 1.25 + 0.5, (t_attn, t_comm, both_attn, both_comm)
    assert both_comm <= (t_attn + t_comm) * 1.25 + 0.5, (t_attn, t_comm, both_attn, both_comm)
    K.check_device_status(cuda_device)
    # on return the side stream has been joined: work enqueued next on the caller's stream sees complete gradients
    dq.zero_(); dk.zero_(); dv.zero_()
    K.attn_bwd(q, k, v, do, lse, delta, scale, True, 0, dq, dk, dv, serial=False)
    snap = dq.clone()                                        # ordered after the join on the same stream
    dq2, dk2, dv2 = (torch.zeros(t.shape, device=cuda_device) for t in (q, k, v))
    K.attn_bwd(q, k, v, do, lse, delta, scale, True, 0, dq2, dk2, dv2, serial=True)
    torch.cuda.synchronize()
    assert (snap - dq2).abs().max().item() <= 1e-3 * dq2.abs().max().item()
    assert _lib.BWD_CONCURRENT == 2


def test_anomaly_reaches_the_next_operator_call_without_a_sync(cuda_device):
    """A bounded wait that ran out sets the device status word; the operators copy it to pinned memory after a backward
    and look at the copy on their next entry, so a loop that never calls check_device_status still stops."""
    from pithtrain_b200 import _lib, kernels as K
    from pithtrain_b200.operators.attention import flash_attn_func
    lib = _lib.load()
    K.check_device_status(cuda_device)
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(1, 256, 4, 128, generator=g).bfloat16().to(cuda_device).requires_grad_() for _ in range(3))
    flash_attn_func(q, k, v, causal=True).sum().backward()      # healthy step: posts a copy of a zero status word
    torch.cuda.synchronize()
    flash_attn_func(q, k, v, causal=True)                        # reads it: nothing to report
    # make a wait run out: a flag that nothing sets, 0.1 s limit, reporting into the operators' status word
    flag = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    ctr = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    s = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.pith_flag_wait(flag.data_ptr(), ctr.data_ptr(), 0.1, K.status_word(cuda_device).data_ptr(), s), "wait")
    q.grad = None
    t0 = time.perf_counter()
    flash_attn_func(q, k, v, causal=True).sum().backward()      # kernels skip their work; the backward posts the copy
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    with pytest.raises(RuntimeError, match="ring neighbour"):
        flash_attn_func(q, k, v, causal=True)
    K.check_device_status(cuda_device)                            # the word was cleared when the error was raised
    out = flash_attn_func(q, k, v, causal=True)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
