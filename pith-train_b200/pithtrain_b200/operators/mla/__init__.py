"""MLA attention operator (q/k head dim 192, v head dim 128) on the sm_100a kernels.

Mirrors ``pithtrain.operators.mla``: the ``MLA`` module (pithtrain/operators/mla/pytorch.py:8-63,
pithtrain/operators/mla/triton.py:510-549) and the raw helpers ``_mla_fwd``, ``_mla_bwd_preprocess``,
``_mla_bwd_dk_dv``, ``_mla_bwd_dq`` (triton.py:552-603). There is one backend, sm_100a; the reference's
import-time dispatch on the device's compute capability (pithtrain/operators/mla/__init__.py:3-11) is gone.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..attention import attn_fwd_op


def _kernels():
    from ... import kernels
    return kernels


class MLA(nn.Module):
    """Causal MLA attention, BSHD layout. ``MLA(h, dq, dv, softmax_scale=0.0)``; 0.0 means ``1/sqrt(dq)``."""

    def __init__(self, h: int, dq: int, dv: int, softmax_scale: float = 0.0):
        super().__init__()
        self.h = h
        self.dq = dq
        self.dv = dv
        self.softmax_scale = softmax_scale if softmax_scale != 0.0 else math.sqrt(1.0 / dq)

    @staticmethod
    def causal(b: int, h: int, qidx: int, kidx: int) -> bool:
        return qidx >= kidx

    @staticmethod
    def autotune(b: int, s: int, h: int, dq: int, dv: int, softmax_scale: float,
                 include_non_causal: bool = False) -> None:
        """The kernels have one fixed configuration, so there is nothing to tune; the call (made by the
        reference's launcher, pithtrain/tasks/pretrain_language_model.py:497-501) only validates the shape
        and loads the library so that the first training step does not pay for it."""
        assert dq == 192 and dv == 128, f"MLA kernel assumes dq=192 and dv=128, got dq={dq} and dv={dv}"
        from ... import _lib
        _lib.load()

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        o, _ = attn_fwd_op(q, k, v, float(self.softmax_scale), True)
        return o


def _mla_fwd(q, k, v, softmax_scale: float, causal: bool = True):
    """Raw MLA forward. Returns (out bf16 [b,s,h,dv], lse fp32 log2 [b,h,s])."""
    return _kernels().attn_fwd(q, k, v, softmax_scale, causal, 0)


def _mla_bwd_preprocess(out, dout):
    """delta = rowsum(out * dout), fp32 [b,h,s]."""
    return _kernels().bwd_preprocess(out, dout)


def _mla_bwd_dk_dv(q, k, v, dout, lse, delta, softmax_scale: float, causal: bool = True):
    """dK, dV (bf16) from external lse (log2) and delta."""
    K = _kernels()
    dk = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
    dv = torch.zeros(v.shape, dtype=torch.float32, device=v.device)
    K.attn_bwd(q, k, v, dout, lse, delta, softmax_scale, causal, 0, None, dk, dv)
    return K.cast_to_bf16(dk), K.cast_to_bf16(dv)


def _mla_bwd_dq(q, k, v, dout, lse, delta, softmax_scale: float, causal: bool = True):
    """dQ (bf16) from external lse (log2) and delta."""
    K = _kernels()
    dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    K.attn_bwd(q, k, v, dout, lse, delta, softmax_scale, causal, 0, dq, None, None)
    return K.cast_to_bf16(dq)


from .assemble import MLAAssembleFunc, mla_assemble  # noqa: E402

__all__ = ["MLA", "_mla_fwd", "_mla_bwd_preprocess", "_mla_bwd_dk_dv", "_mla_bwd_dq", "MLAAssembleFunc", "mla_assemble"]
