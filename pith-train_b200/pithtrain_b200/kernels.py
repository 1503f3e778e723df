"""Thin tensor-level wrappers over the C ABI: pointer / stride marshalling and nothing else.

All functions enqueue on the current CUDA stream of the tensors' device and return immediately.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import I64x2, I64x3

_status_words: dict[int, torch.Tensor] = {}

# Kernels of libpith_b200.so enqueued by this process so far (benchmarks report the per-step count).
launch_count = 0


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device uint32 the kernels write to when a bounded wait gives up (0 = healthy)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    w = _status_words.get(idx)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status_words[idx] = w
    return w


def check_device_status(device=None) -> None:
    """Synchronises and raises if any kernel launched so far reported a device-side anomaly."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = status_word(device)
    val = int(w.item()) & 0xFFFFFFFF
    if val != 0:
        w.zero_()
        text = _lib.load().pith_status_string(val).decode()
        raise RuntimeError(f"pith_b200 kernel reported: {text}")


# Host mirror of the status word: (pinned int32 tensor, event recorded after the last device-to-host copy).
_status_mirrors: dict[int, list] = {}


def post_status_copy(device=None) -> None:
    """Enqueues, on the current stream, a copy of the status word into pinned host memory and records an event
    behind it. Costs one 4-byte copy and no synchronisation; the operators call it when a backward has been
    enqueued, and ``poll_device_status`` reads the mirror later. Skipped while a stream is being captured."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if torch.cuda.is_current_stream_capturing():
        return
    idx = device.index if device.index is not None else torch.cuda.current_device()
    m = _status_mirrors.get(idx)
    if m is None:
        m = _status_mirrors[idx] = [torch.zeros(1, dtype=torch.int32).pin_memory(), torch.cuda.Event(), False]
    elif m[2] and not m[1].query():
        return  # the previous copy has not landed yet: its value is still to be read
    m[0].copy_(status_word(device), non_blocking=True)
    m[1].record(torch.cuda.current_stream(device))
    m[2] = True


def poll_device_status(device=None) -> None:
    """Raises if a kernel enqueued before the last ``post_status_copy`` reported a device-side anomaly (a bounded
    wait that gave up), without synchronising: it looks at the host mirror only when its copy has completed.
    The operators call it on entry, so a training loop that never calls ``check_device_status`` still stops at the
    next attention call instead of training on the output of kernels that skipped their work."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    m = _status_mirrors.get(idx)
    if m is None or not m[2] or not m[1].query():
        return
    m[2] = False
    val = int(m[0].item()) & 0xFFFFFFFF
    if val != 0:
        status_word(device).zero_()
        text = _lib.load().pith_status_string(val).decode()
        raise RuntimeError(f"pith_b200 kernel reported: {text}")


def _count(n: int) -> None:
    global launch_count
    launch_count += n


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _bshd(t: torch.Tensor, name: str) -> I64x3:
    if t.dim() != 4 or t.stride(3) != 1:
        raise ValueError(f"{name} must be [B,S,H,D] with a contiguous last dimension, got {tuple(t.shape)} "
                         f"strides {t.stride()}")
    return I64x3(t.stride(0), t.stride(1), t.stride(2))


def _bhs(t: torch.Tensor, name: str) -> I64x2:
    if t.dim() != 3 or t.stride(2) != 1 or t.dtype != torch.float32:
        raise ValueError(f"{name} must be fp32 [B,H,S] with unit stride along S")
    return I64x2(t.stride(0), t.stride(1))


def _expect(t, shape, name: str) -> None:
    """A mismatch would otherwise become a TMA map that reads past the tensor: refuse it here."""
    if t is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("pith_b200 operators run on CUDA tensors only (no CPU fallback)")


def attn_fwd(q, k, v, softmax_scale: float, causal: bool, causal_offset: int = 0, *, out=None, lse=None,
             prev_o=None, prev_lse=None, out_fp32: bool = False, lse_natural: bool = False, single_cta=None):
    """One attention block: returns (O [B,Sq,Hq,Dv], LSE [B,Hq,Sq]); see ``pith_attn_fwd``.

    ``single_cta=True`` selects the kernel that keeps every MMA inside one CTA (``PITH_FWD_SINGLE_CTA``),
    ``single_cta=False`` the CTA-pair kernel (``PITH_FWD_CTA_PAIR``); ``None`` lets the library choose."""
    _require_cuda(q, k, v, out, lse, prev_o, prev_lse)
    B, Sq, Hq, Dqk = q.shape
    _, Sk, Hkv, Dv = v.shape
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise TypeError("q, k, v must be bfloat16")
    _expect(k, (B, Sk, Hkv, Dqk), "k")
    _expect(v, (B, Sk, Hkv, Dv), "v")
    _expect(out, (B, Sq, Hq, Dv), "out")
    _expect(lse, (B, Hq, Sq), "lse")
    _expect(prev_o, (B, Sq, Hq, Dv), "prev_o")
    _expect(prev_lse, (B, Hq, Sq), "prev_lse")
    if (prev_o is None) != (prev_lse is None):
        raise ValueError("prev_o and prev_lse must be given together")
    if out is None:
        out = torch.empty((B, Sq, Hq, Dv), dtype=torch.float32 if out_fp32 else torch.bfloat16, device=q.device)
    else:
        out_fp32 = out.dtype == torch.float32
    if lse is None:
        lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device)
    a = _lib.AttnFwdArgs()
    a.q, a.k, a.v, a.o, a.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr()
    a.prev_o = prev_o.data_ptr() if prev_o is not None else None
    a.prev_lse = prev_lse.data_ptr() if prev_lse is not None else None
    a.status = status_word(q.device).data_ptr()
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.Dqk, a.Dv = B, Sq, Sk, Hq, Hkv, Dqk, Dv
    a.causal, a.causal_offset = int(bool(causal)), int(causal_offset)
    a.flags = ((_lib.FWD_O_FP32 if out_fp32 else 0) | (_lib.FWD_LSE_NATURAL if lse_natural else 0)
               | (0 if single_cta is None else _lib.FWD_SINGLE_CTA if single_cta else _lib.FWD_CTA_PAIR))
    a.softmax_scale = float(softmax_scale)
    a.q_stride, a.k_stride, a.v_stride = _bshd(q, "q"), _bshd(k, "k"), _bshd(v, "v")
    a.o_stride = _bshd(out, "out")
    a.lse_stride = _bhs(lse, "lse")
    if prev_o is not None:
        if prev_o.dtype != torch.float32:
            raise TypeError("prev_o must be float32")
        a.prev_o_stride = _bshd(prev_o, "prev_o")
        a.prev_lse_stride = _bhs(prev_lse, "prev_lse")
    _lib.check(_lib.load().pith_attn_fwd(ctypes.byref(a), _stream(q)), "pith_attn_fwd")
    _count(1)
    return out, lse


def bwd_preprocess(o, dout, delta=None):
    """delta [B,H,S] = rowsum(o * dout); see ``pith_attn_bwd_preprocess``."""
    _require_cuda(o, dout, delta)
    B, S, H, Dv = o.shape
    _expect(dout, (B, S, H, Dv), "dout")
    _expect(delta, (B, H, S), "delta")
    if delta is None:
        delta = torch.empty((B, H, S), dtype=torch.float32, device=o.device)
    a = _lib.BwdPreprocessArgs()
    a.o, a.dout, a.delta = o.data_ptr(), dout.data_ptr(), delta.data_ptr()
    a.B, a.S, a.H, a.Dv = B, S, H, Dv
    a.o_stride, a.do_stride, a.delta_stride = _bshd(o, "o"), _bshd(dout, "dout"), _bhs(delta, "delta")
    _lib.check(_lib.load().pith_attn_bwd_preprocess(ctypes.byref(a), _stream(o)), "pith_attn_bwd_preprocess")
    _count(1 if o.numel() else 0)
    return delta


def attn_bwd(q, k, v, dout, lse_log2, delta, softmax_scale: float, causal: bool, causal_offset: int,
             dq_acc, dk_acc, dv_acc, serial=None, dq_out=None):
    """Adds this block's dQ/dK/dV into the fp32 accumulators; see ``pith_attn_bwd``.

    ``serial=True`` runs the two passes one after the other on the current stream (``PITH_BWD_SERIAL``),
    ``serial=False`` side by side (``PITH_BWD_CONCURRENT``); ``None`` lets the library decide by problem size.

    ``dq_out`` (bf16, shape of q; head_dim 128 only; instead of ``dq_acc``): the dQ pass stores this block's complete
    dQ there (``PITH_BWD_DQ_STORE_BF16``) — for a backward that consists of this one block."""
    if dq_out is not None:
        if dq_acc is not None:
            raise ValueError("give dq_acc (accumulate, fp32) or dq_out (store, bf16), not both")
        if dq_out.dtype != torch.bfloat16 or dq_out.shape != q.shape:
            raise ValueError("dq_out must be bfloat16 with the shape of q")
        _require_cuda(dq_out)
    _require_cuda(q, k, v, dout, lse_log2, delta, dq_acc, dk_acc, dv_acc)
    B, Sq, Hq, Dqk = q.shape
    _, Sk, Hkv, Dv = v.shape
    for t, n in ((dq_acc, "dq_acc"), (dk_acc, "dk_acc"), (dv_acc, "dv_acc")):
        if t is not None and t.dtype != torch.float32:
            raise TypeError(f"{n} must be float32")
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (dout, "dout")):
        if t.dtype != torch.bfloat16:
            raise TypeError(f"{n} must be bfloat16")
    _expect(k, (B, Sk, Hkv, Dqk), "k")
    _expect(v, (B, Sk, Hkv, Dv), "v")
    _expect(dout, (B, Sq, Hq, Dv), "dout")
    _expect(lse_log2, (B, Hq, Sq), "lse")
    _expect(delta, (B, Hq, Sq), "delta")
    _expect(dq_acc, (B, Sq, Hq, Dqk), "dq_acc")
    _expect(dk_acc, (B, Sk, Hkv, Dqk), "dk_acc")
    _expect(dv_acc, (B, Sk, Hkv, Dv), "dv_acc")
    if (dk_acc is None) != (dv_acc is None):
        raise ValueError("dk_acc and dv_acc must be given together")
    a = _lib.AttnBwdArgs()
    a.q, a.k, a.v, a.dout = q.data_ptr(), k.data_ptr(), v.data_ptr(), dout.data_ptr()
    a.lse, a.delta = lse_log2.data_ptr(), delta.data_ptr()
    a.dq_acc = dq_out.data_ptr() if dq_out is not None else dq_acc.data_ptr() if dq_acc is not None else None
    a.dk_acc = dk_acc.data_ptr() if dk_acc is not None else None
    a.dv_acc = dv_acc.data_ptr() if dv_acc is not None else None
    a.status = status_word(q.device).data_ptr()
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.Dqk, a.Dv = B, Sq, Sk, Hq, Hkv, Dqk, Dv
    a.causal, a.causal_offset, a.flags = int(bool(causal)), int(causal_offset), ((0 if serial is None else _lib.BWD_SERIAL if serial else _lib.BWD_CONCURRENT)
                                                        | (_lib.BWD_DQ_STORE_BF16 if dq_out is not None else 0))
    a.softmax_scale = float(softmax_scale)
    a.q_stride, a.k_stride, a.v_stride, a.do_stride = _bshd(q, "q"), _bshd(k, "k"), _bshd(v, "v"), _bshd(dout, "dout")
    if dq_out is not None:
        a.dq_stride = _bshd(dq_out, "dq_out")
    elif dq_acc is not None:
        a.dq_stride = _bshd(dq_acc, "dq_acc")
    if dk_acc is not None:
        a.dk_stride, a.dv_stride = _bshd(dk_acc, "dk_acc"), _bshd(dv_acc, "dv_acc")
    a.lse_stride, a.delta_stride = _bhs(lse_log2, "lse"), _bhs(delta, "delta")
    _lib.check(_lib.load().pith_attn_bwd(ctypes.byref(a), _stream(q)), "pith_attn_bwd")
    _count((dq_acc is not None or dq_out is not None) + (dk_acc is not None))


def cast_to_bf16(acc, out=None, scale: float = 1.0):
    """bf16(acc * scale) for an fp32 [B,S,H,D] accumulator; see ``pith_cast_f32_to_bf16``."""
    _require_cuda(acc, out)
    B, S, H, D = acc.shape
    if out is None:
        out = torch.empty((B, S, H, D), dtype=torch.bfloat16, device=acc.device)
    _lib.check(_lib.load().pith_cast_f32_to_bf16(acc.data_ptr(), out.data_ptr(), B, S, H, D, _bshd(acc, "acc"),
                                                 _bshd(out, "out"), float(scale), _stream(acc)),
               "pith_cast_f32_to_bf16")
    _count(1 if acc.numel() else 0)
    return out


def combine(out1, lse1, out2, lse2, natural: bool):
    """Online-softmax merge; returns (fp32 out [B,S,H,D], fp32 lse [B,H,S]); see ``pith_combine``."""
    _require_cuda(out1, lse1, out2, lse2)
    B, S, H, D = out1.shape
    dt = {torch.bfloat16: _lib.DTYPE_BF16, torch.float32: _lib.DTYPE_F32}
    if out1.dtype not in dt or out2.dtype not in dt:
        raise TypeError("combine inputs must be bfloat16 or float32")
    out = torch.empty((B, S, H, D), dtype=torch.float32, device=out1.device)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=out1.device)
    a = _lib.CombineArgs()
    a.out1, a.lse1, a.out2, a.lse2 = out1.data_ptr(), lse1.data_ptr(), out2.data_ptr(), lse2.data_ptr()
    a.out, a.lse = out.data_ptr(), lse.data_ptr()
    a.out1_dtype, a.out2_dtype = dt[out1.dtype], dt[out2.dtype]
    a.B, a.S, a.H, a.D = B, S, H, D
    a.flags = _lib.COMBINE_NATURAL if natural else 0
    a.out1_stride, a.out2_stride = _bshd(out1, "out1"), _bshd(out2, "out2")
    a.lse1_stride, a.lse2_stride = _bhs(lse1, "lse1"), _bhs(lse2, "lse2")
    _lib.check(_lib.load().pith_combine(ctypes.byref(a), _stream(out1)), "pith_combine")
    _count(1 if out1.numel() else 0)
    return out, lse


def combine_partials(parts, B: int, S: int, H: int, D: int):
    """Merges partial attention results in one pass; see ``pith_combine_partials``.

    ``parts``: sequence of ``(o, lse, row_begin)`` with ``o`` bf16 [B, rows, H, D] and ``lse`` fp32 [B, H, rows] (log2
    domain), the partial result of query rows ``row_begin .. row_begin + rows`` over one K/V block.
    Returns (bf16 out [B, S, H, D], fp32 lse [B, H, S])."""
    parts = list(parts)
    if not 1 <= len(parts) <= _lib.MAX_PARTIALS:
        raise ValueError(f"combine_partials takes 1 .. {_lib.MAX_PARTIALS} partial results, got {len(parts)}")
    _require_cuda(*[t for o, l, _ in parts for t in (o, l)])
    dev = parts[0][0].device
    out = torch.empty((B, S, H, D), dtype=torch.bfloat16, device=dev)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=dev)
    a = _lib.CombinePartialsArgs()
    a.n = len(parts)
    a.B, a.S, a.H, a.D = B, S, H, D
    a.out, a.lse = out.data_ptr(), lse.data_ptr()
    for i, (o, l, row_begin) in enumerate(parts):
        if o.dtype != torch.bfloat16:
            raise TypeError(f"partial {i} must be bfloat16")
        _expect(o, (B, o.shape[1], H, D), f"partial {i}")
        _expect(l, (B, H, o.shape[1]), f"lse of partial {i}")
        pt = a.part[i]
        pt.o, pt.lse = o.data_ptr(), l.data_ptr()
        pt.row_begin, pt.rows = int(row_begin), int(o.shape[1])
        pt.o_stride, pt.lse_stride = _bshd(o, f"partial {i}"), _bhs(l, f"lse of partial {i}")
    _lib.check(_lib.load().pith_combine_partials(ctypes.byref(a), _stream(out)), "pith_combine_partials")
    _count(1 if out.numel() else 0)
    return out, lse


def _qk_args(q, k, q_weight, k_weight, cos, sin, eps):
    _require_cuda(q, k, q_weight, k_weight, cos, sin)
    B, S, Hq, D = q.shape
    Hkv = k.shape[2]
    if k.shape[0] != B or k.shape[1] != S or k.shape[3] != D:
        raise ValueError(f"q {tuple(q.shape)} and k {tuple(k.shape)} disagree in batch, sequence or head_dim")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16:
        raise TypeError("q and k must be bfloat16")
    dt = {torch.bfloat16: _lib.DTYPE_BF16, torch.float32: _lib.DTYPE_F32}
    if q_weight.dtype not in dt or k_weight.dtype != q_weight.dtype or cos.dtype not in dt or sin.dtype != cos.dtype:
        raise TypeError("weights and cos/sin must be bfloat16 or float32 (both weights alike, cos and sin alike)")
    if tuple(q_weight.shape) != (D,) or tuple(k_weight.shape) != (D,) or not (q_weight.is_contiguous()
                                                                               and k_weight.is_contiguous()):
        raise ValueError(f"norm weights must be contiguous [{D}]")
    if cos.dim() != 3 or cos.shape[0] not in (1, B) or cos.shape[1] != S or cos.shape[2] != D or cos.stride(2) != 1 \
            or sin.shape != cos.shape or sin.stride() != cos.stride():
        raise ValueError(f"cos/sin must be [B or 1, {S}, {D}] with a contiguous last dimension and equal strides")
    a = _lib.QkNormRopeArgs()
    a.q, a.k, a.q_weight, a.k_weight = q.data_ptr(), k.data_ptr(), q_weight.data_ptr(), k_weight.data_ptr()
    a.cos, a.sin = cos.data_ptr(), sin.data_ptr()
    a.B, a.S, a.Hq, a.Hkv, a.D = B, S, Hq, Hkv, D
    a.weight_dtype, a.cs_dtype, a.eps = dt[q_weight.dtype], dt[cos.dtype], float(eps)
    a.q_stride, a.k_stride = _bshd(q, "q"), _bshd(k, "k")
    a.cs_stride = I64x2(cos.stride(0) if cos.shape[0] == B and B > 1 else 0, cos.stride(1))
    return a


def qk_norm_rope_fwd(q, k, q_weight, k_weight, cos, sin, eps: float):
    """Per-head RMSNorm of q and k, then rotary embedding; returns (q_embed, k_embed) bf16 contiguous.
    See ``pith_qk_norm_rope_fwd``."""
    a = _qk_args(q, k, q_weight, k_weight, cos, sin, eps)
    q_out, k_out = torch.empty(q.shape, dtype=q.dtype, device=q.device), torch.empty(k.shape, dtype=k.dtype,
                                                                                     device=k.device)
    a.q_out, a.k_out = q_out.data_ptr(), k_out.data_ptr()
    a.q_out_stride, a.k_out_stride = _bshd(q_out, "q_out"), _bshd(k_out, "k_out")
    _lib.check(_lib.load().pith_qk_norm_rope_fwd(ctypes.byref(a), _stream(q)), "pith_qk_norm_rope_fwd")
    _count(1 if q.numel() + k.numel() else 0)
    return q_out, k_out


def qk_norm_rope_bwd(q, k, q_weight, k_weight, cos, sin, eps: float, dq_embed, dk_embed):
    """Backward of ``qk_norm_rope_fwd``: returns (dq, dk bf16; dq_weight, dk_weight fp32 [D])."""
    _require_cuda(dq_embed, dk_embed)
    a = _qk_args(q, k, q_weight, k_weight, cos, sin, eps)
    if dq_embed.shape != q.shape or dk_embed.shape != k.shape or dq_embed.dtype != torch.bfloat16 \
            or dk_embed.dtype != torch.bfloat16:
        raise ValueError("output gradients must be bfloat16 with the shapes of q and k")
    dq, dk = torch.empty(q.shape, dtype=q.dtype, device=q.device), torch.empty(k.shape, dtype=k.dtype, device=k.device)
    dw = torch.zeros(2, q.shape[3], dtype=torch.float32, device=q.device)
    a.q_out, a.k_out = dq.data_ptr(), dk.data_ptr()
    a.q_out_stride, a.k_out_stride = _bshd(dq, "dq"), _bshd(dk, "dk")
    a.dq_out, a.dk_out = dq_embed.data_ptr(), dk_embed.data_ptr()
    a.dq_out_stride, a.dk_out_stride = _bshd(dq_embed, "dq_embed"), _bshd(dk_embed, "dk_embed")
    a.dq_weight, a.dk_weight = dw[0].data_ptr(), dw[1].data_ptr()
    _lib.check(_lib.load().pith_qk_norm_rope_bwd(ctypes.byref(a), _stream(q)), "pith_qk_norm_rope_bwd")
    _count(1 if q.numel() + k.numel() else 0)
    return dq, dk, dw[0], dw[1]


def _mla_asm_args(B, S, H, cos, sin):
    _require_cuda(cos, sin)
    dt = {torch.bfloat16: _lib.DTYPE_BF16, torch.float32: _lib.DTYPE_F32}
    if cos.dtype not in dt or sin.dtype != cos.dtype:
        raise TypeError("cos and sin must both be bfloat16 or float32")
    if cos.dim() != 3 or cos.shape[0] not in (1, B) or tuple(cos.shape[1:]) != (S, 64) or cos.stride(2) != 1 \
            or sin.shape != cos.shape or sin.stride() != cos.stride():
        raise ValueError(f"cos/sin must be [B or 1, {S}, 64] (gathered by position) with equal strides")
    a = _lib.MlaAssembleArgs()
    a.cos, a.sin = cos.data_ptr(), sin.data_ptr()
    a.B, a.S, a.H, a.Dnope, a.Drope, a.Dv, a.cs_dtype = B, S, H, 128, 64, 128, dt[cos.dtype]
    a.cs_stride = I64x2(cos.stride(0) if cos.shape[0] == B and B > 1 else 0, cos.stride(1))
    return a


def mla_assemble_fwd(q, kv, k_pe, cos, sin):
    """(query [B,S,H,192], key [B,S,H,192], value [B,S,H,128]) from q = [q_nope | q_pe], kv = [k_nope | v] and the
    per-position rotary key k_pe; see ``pith_mla_assemble_fwd``."""
    _require_cuda(q, kv, k_pe)
    if q.dim() != 4 or q.shape[3] != 192 or tuple(kv.shape) != (*q.shape[:3], 256):
        raise ValueError(f"q must be [B,S,H,192] and kv [B,S,H,256], got {tuple(q.shape)} and {tuple(kv.shape)}")
    B, S, H, _ = q.shape
    if k_pe.dim() == 4 and k_pe.shape[2] == 1:
        k_pe = k_pe[:, :, 0]
    if tuple(k_pe.shape) != (B, S, 64) or k_pe.stride(2) != 1:
        raise ValueError(f"k_pe must be [B,S,64] or [B,S,1,64] with a contiguous last dimension, got {tuple(k_pe.shape)}")
    if not (q.dtype == kv.dtype == k_pe.dtype == torch.bfloat16):
        raise TypeError("q, kv and k_pe must be bfloat16")
    a = _mla_asm_args(B, S, H, cos, sin)
    query, key = (torch.empty((B, S, H, 192), dtype=q.dtype, device=q.device) for _ in range(2))
    value = torch.empty((B, S, H, 128), dtype=q.dtype, device=q.device)
    a.q, a.kv, a.k_pe = q.data_ptr(), kv.data_ptr(), k_pe.data_ptr()
    a.query, a.key, a.value = query.data_ptr(), key.data_ptr(), value.data_ptr()
    a.q_stride, a.kv_stride = _bshd(q, "q"), _bshd(kv, "kv")
    a.query_stride, a.key_stride, a.value_stride = _bshd(query, "query"), _bshd(key, "key"), _bshd(value, "value")
    a.k_pe_stride = I64x2(k_pe.stride(0), k_pe.stride(1))
    _lib.check(_lib.load().pith_mla_assemble_fwd(ctypes.byref(a), _stream(q)), "pith_mla_assemble_fwd")
    _count(1 if q.numel() else 0)
    return query, key, value


def mla_assemble_bwd(cos, sin, dquery, dkey, dvalue):
    """Gradients (dq [B,S,H,192], dkv [B,S,H,256], dk_pe [B,S,64]; contiguous) from the gradients of
    query / key / value; see ``pith_mla_assemble_bwd``."""
    _require_cuda(dquery, dkey, dvalue)
    if dquery.dim() != 4 or dquery.shape[3] != 192:
        raise ValueError(f"dquery must be [B,S,H,192], got {tuple(dquery.shape)}")
    B, S, H, _ = dquery.shape
    for t, d, n in ((dquery, 192, "dquery"), (dkey, 192, "dkey"), (dvalue, 128, "dvalue")):
        if tuple(t.shape) != (B, S, H, d) or t.dtype != torch.bfloat16:
            raise ValueError(f"{n} must be bfloat16 [{B},{S},{H},{d}]")
    a = _mla_asm_args(B, S, H, cos, sin)
    dq = torch.empty((B, S, H, 192), dtype=torch.bfloat16, device=dquery.device)
    dkv = torch.empty((B, S, H, 256), dtype=torch.bfloat16, device=dquery.device)
    dk_pe = torch.empty((B, S, 64), dtype=torch.bfloat16, device=dquery.device)
    a.dq, a.dkv, a.dk_pe = dq.data_ptr(), dkv.data_ptr(), dk_pe.data_ptr()
    a.dquery, a.dkey, a.dvalue = dquery.data_ptr(), dkey.data_ptr(), dvalue.data_ptr()
    a.q_stride, a.kv_stride = _bshd(dq, "dq"), _bshd(dkv, "dkv")
    a.query_stride, a.key_stride, a.value_stride = _bshd(dquery, "dquery"), _bshd(dkey, "dkey"), _bshd(dvalue, "dvalue")
    a.k_pe_stride = I64x2(dk_pe.stride(0), dk_pe.stride(1))
    _lib.check(_lib.load().pith_mla_assemble_bwd(ctypes.byref(a), _stream(dquery)), "pith_mla_assemble_bwd")
    _count(1 if dq.numel() else 0)
    return dq, dkv, dk_pe
