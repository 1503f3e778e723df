"""The allocation-free attention backward (``pith_attn_bwd_noalloc``) against the regular entry points and the
CPU oracle.

Some hosts cannot allocate device memory at the point where the backward runs: their memory pool was frozen
after start-up, or the runtime they are embedded in owns every device allocation, or they cannot take the
device-wide synchronisation that cudaMalloc / cudaFree imply. For them the library carries a fixed 32 MiB scratch
area in its own image; this test drives that entry point through the C ABI twice in a row (the area keeps the
previous call's contents and must be re-zeroed by the callee) and compares with the caller-allocated path.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""

import ctypes

import pytest
import torch

from helpers import assert_bf16_close
from oracle import attention_oracle as O

pytestmark = pytest.mark.gpu


def _strides(t):
    from pithtrain_b200._lib import I64x3
    return I64x3(t.stride(0), t.stride(1), t.stride(2))


def _noalloc_backward(q, k, v, o, do, lse, scale, causal, status):
    from pithtrain_b200 import _lib
    lib = _lib.load()
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)   # outputs belong to the caller
    a = _lib.AttnBwdNoallocArgs()
    a.q, a.k, a.v, a.o, a.dout, a.lse = (t.data_ptr() for t in (q, k, v, o, do, lse))
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.status = status.data_ptr()
    a.B, a.Sq, a.Hq, a.Dqk = q.shape
    _, a.Sk, a.Hkv, a.Dv = v.shape
    a.causal, a.causal_offset, a.softmax_scale = int(causal), 0, scale
    a.q_stride, a.k_stride, a.v_stride, a.o_stride, a.do_stride = (_strides(t) for t in (q, k, v, o, do))
    a.dq_stride, a.dk_stride, a.dv_stride = _strides(dq), _strides(dk), _strides(dv)
    a.lse_stride = _lib.I64x2(lse.stride(0), lse.stride(1))
    rc = lib.pith_attn_bwd_noalloc(ctypes.byref(a), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc, "pith_attn_bwd_noalloc")
    return dq, dk, dv


def _regular_backward(K, q, k, v, o, do, lse, scale, causal):
    delta = K.bwd_preprocess(o, do)
    dq, dk, dv = (torch.zeros(t.shape, dtype=torch.float32, device=t.device) for t in (q, k, v))
    K.attn_bwd(q, k, v, do, lse, delta, scale, causal, 0, dq, dk, dv)
    return K.cast_to_bf16(dq), K.cast_to_bf16(dk), K.cast_to_bf16(dv)


def test_noalloc_backward_matches_regular_entry_points_twice(cuda_device):
    from pithtrain_b200 import _lib, kernels as K
    lib = _lib.load()
    status = K.status_word(cuda_device)
    # two different problems back to back: the second must not see the first one's accumulators
    problems = [(1, 1024, 1024, 8, 2, 128, True, 7), (2, 384, 512, 4, 4, 192, False, 11)]
    for B, Sq, Sk, Hq, Hkv, Dqk, causal, seed in problems:
        g = torch.Generator().manual_seed(seed)
        q = torch.randn(B, Sq, Hq, Dqk, generator=g).bfloat16().to(cuda_device)
        k = torch.randn(B, Sk, Hkv, Dqk, generator=g).bfloat16().to(cuda_device)
        v = torch.randn(B, Sk, Hkv, 128, generator=g).bfloat16().to(cuda_device)
        do = torch.randn(B, Sq, Hq, 128, generator=g).bfloat16().to(cuda_device)
        scale = Dqk ** -0.5
        o, lse = K.attn_fwd(q, k, v, scale, causal, 0)
        assert lib.pith_attn_bwd_noalloc_scratch_bytes(B, Sq, Sk, Hq, Hkv, Dqk, 128) <= _lib.NOALLOC_SCRATCH_BYTES
        ref = _regular_backward(K, q, k, v, o, do, lse, scale, causal)
        # two CUDA paths agreeing is not parity: the oracle (fp32 on the CPU, from its own forward) decides
        ro, rl = O.attention_fwd(q.cpu(), k.cpu(), v.cpu(), scale, causal, 0)
        oracle = O.attention_bwd(q.cpu(), k.cpu(), v.cpu(), do.cpu(), rl, O.delta(ro, do.cpu()), scale, causal, 0)
        for call in range(2):
            got = _noalloc_backward(q, k, v, o, do, lse, scale, causal, status)
            torch.cuda.synchronize()
            for name, a, b, c in zip(("dQ", "dK", "dV"), got, ref, oracle):
                # same kernels, same inputs; only the order of the fp32 atomic additions may differ
                assert_bf16_close(a, b, f"{name} vs regular entry points (call {call})")
                assert_bf16_close(a, c, f"{name} vs oracle (call {call})")
    K.check_device_status(cuda_device)


def test_noalloc_rejects_problems_beyond_the_scratch_area(cuda_device):
    from pithtrain_b200 import _lib
    lib = _lib.load()
    assert lib.pith_attn_bwd_noalloc_scratch_bytes(1, 8192, 8192, 32, 4, 128, 128) > _lib.NOALLOC_SCRATCH_BYTES
    a = _lib.AttnBwdNoallocArgs()
    for f in ("q", "k", "v", "o", "dout", "lse", "dq", "dk", "dv"):
        setattr(a, f, 0x1000)
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.Dqk, a.Dv = 1, 8192, 8192, 32, 4, 128, 128
    a.softmax_scale = 0.1
    assert lib.pith_attn_bwd_noalloc(ctypes.byref(a), None) < 0
    msg = lib.pith_last_error().decode()
    assert "scratch" in msg and str(_lib.NOALLOC_SCRATCH_BYTES) in msg
    # a shape whose byte count would wrap around 64 bits is "does not fit", not a small number
    huge = lib.pith_attn_bwd_noalloc_scratch_bytes(65535, 2 ** 31 - 1, 2 ** 31 - 1, 65535, 1, 192, 128)
    assert huge > _lib.NOALLOC_SCRATCH_BYTES
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv = 65535, 2 ** 31 - 1, 2 ** 31 - 1, 65535, 1
    assert lib.pith_attn_bwd_noalloc(ctypes.byref(a), None) < 0 and "scratch" in lib.pith_last_error().decode()
    # checks of the regular entry point are made before the shared area is touched
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.Dqk = 1, 128, 128, 4, 4, 96
    assert lib.pith_attn_bwd_noalloc(ctypes.byref(a), None) < 0 and "head dims" in lib.pith_last_error().decode()
