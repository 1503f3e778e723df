"""ctypes binding of ``libpith_b200.so`` (declared in ``include/pith_b200.h``).

There is no fallback: if the library is missing or a call is rejected, an exception is raised.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_uint32, c_void_p
from pathlib import Path

import os

# PITH_B200_LIB overrides the library location (used to compare builds); the default is the in-tree build.
LIB_PATH = Path(os.environ.get("PITH_B200_LIB", Path(__file__).resolve().parent / "libpith_b200.so"))

I64x3 = c_int64 * 3
I64x2 = c_int64 * 2


class AttnFwdArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("o", c_void_p), ("lse", c_void_p),
        ("prev_o", c_void_p), ("prev_lse", c_void_p), ("status", c_void_p),
        ("B", c_int32), ("Sq", c_int32), ("Sk", c_int32), ("Hq", c_int32), ("Hkv", c_int32),
        ("Dqk", c_int32), ("Dv", c_int32),
        ("causal", c_int32), ("causal_offset", c_int32), ("flags", c_uint32), ("softmax_scale", c_float),
        ("q_stride", I64x3), ("k_stride", I64x3), ("v_stride", I64x3), ("o_stride", I64x3),
        ("prev_o_stride", I64x3),
        ("lse_stride", I64x2), ("prev_lse_stride", I64x2),
    ]


class BwdPreprocessArgs(Structure):
    _fields_ = [
        ("o", c_void_p), ("dout", c_void_p), ("delta", c_void_p),
        ("B", c_int32), ("S", c_int32), ("H", c_int32), ("Dv", c_int32),
        ("o_stride", I64x3), ("do_stride", I64x3), ("delta_stride", I64x2),
    ]


class AttnBwdArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("dout", c_void_p), ("lse", c_void_p),
        ("delta", c_void_p), ("dq_acc", c_void_p), ("dk_acc", c_void_p), ("dv_acc", c_void_p),
        ("status", c_void_p),
        ("B", c_int32), ("Sq", c_int32), ("Sk", c_int32), ("Hq", c_int32), ("Hkv", c_int32),
        ("Dqk", c_int32), ("Dv", c_int32),
        ("causal", c_int32), ("causal_offset", c_int32), ("flags", c_uint32), ("softmax_scale", c_float),
        ("q_stride", I64x3), ("k_stride", I64x3), ("v_stride", I64x3), ("do_stride", I64x3),
        ("dq_stride", I64x3), ("dk_stride", I64x3), ("dv_stride", I64x3),
        ("lse_stride", I64x2), ("delta_stride", I64x2),
    ]


class CombineArgs(Structure):
    _fields_ = [
        ("out1", c_void_p), ("lse1", c_void_p), ("out2", c_void_p), ("lse2", c_void_p),
        ("out", c_void_p), ("lse", c_void_p),
        ("out1_dtype", c_int32), ("out2_dtype", c_int32),
        ("B", c_int32), ("S", c_int32), ("H", c_int32), ("D", c_int32), ("flags", c_uint32),
        ("out1_stride", I64x3), ("out2_stride", I64x3), ("lse1_stride", I64x2), ("lse2_stride", I64x2),
    ]


MAX_PARTIALS = 16


class Partial(Structure):
    _fields_ = [
        ("o", c_void_p), ("lse", c_void_p), ("row_begin", c_int32), ("rows", c_int32),
        ("o_stride", I64x3), ("lse_stride", I64x2),
    ]


class CombinePartialsArgs(Structure):
    _fields_ = [
        ("part", Partial * MAX_PARTIALS), ("n", c_int32),
        ("B", c_int32), ("S", c_int32), ("H", c_int32), ("D", c_int32),
        ("out", c_void_p), ("lse", c_void_p),
    ]


class AttnBwdNoallocArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("o", c_void_p), ("dout", c_void_p), ("lse", c_void_p),
        ("dq", c_void_p), ("dk", c_void_p), ("dv", c_void_p), ("status", c_void_p),
        ("B", c_int32), ("Sq", c_int32), ("Sk", c_int32), ("Hq", c_int32), ("Hkv", c_int32),
        ("Dqk", c_int32), ("Dv", c_int32),
        ("causal", c_int32), ("causal_offset", c_int32), ("softmax_scale", c_float),
        ("q_stride", I64x3), ("k_stride", I64x3), ("v_stride", I64x3), ("o_stride", I64x3), ("do_stride", I64x3),
        ("dq_stride", I64x3), ("dk_stride", I64x3), ("dv_stride", I64x3),
        ("lse_stride", I64x2),
    ]


class QkNormRopeArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("q_weight", c_void_p), ("k_weight", c_void_p),
        ("cos", c_void_p), ("sin", c_void_p), ("q_out", c_void_p), ("k_out", c_void_p),
        ("dq_out", c_void_p), ("dk_out", c_void_p), ("dq_weight", c_void_p), ("dk_weight", c_void_p),
        ("B", c_int32), ("S", c_int32), ("Hq", c_int32), ("Hkv", c_int32), ("D", c_int32),
        ("weight_dtype", c_int32), ("cs_dtype", c_int32), ("eps", c_float),
        ("q_stride", I64x3), ("k_stride", I64x3), ("q_out_stride", I64x3), ("k_out_stride", I64x3),
        ("dq_out_stride", I64x3), ("dk_out_stride", I64x3),
        ("cs_stride", I64x2),
    ]


class MlaAssembleArgs(Structure):
    _fields_ = [
        ("q", c_void_p), ("kv", c_void_p), ("k_pe", c_void_p), ("cos", c_void_p), ("sin", c_void_p),
        ("query", c_void_p), ("key", c_void_p), ("value", c_void_p),
        ("dquery", c_void_p), ("dkey", c_void_p), ("dvalue", c_void_p),
        ("dq", c_void_p), ("dkv", c_void_p), ("dk_pe", c_void_p),
        ("B", c_int32), ("S", c_int32), ("H", c_int32),
        ("Dnope", c_int32), ("Drope", c_int32), ("Dv", c_int32), ("cs_dtype", c_int32),
        ("q_stride", I64x3), ("kv_stride", I64x3), ("query_stride", I64x3), ("key_stride", I64x3),
        ("value_stride", I64x3),
        ("k_pe_stride", I64x2), ("cs_stride", I64x2),
    ]


NOALLOC_SCRATCH_BYTES = 32 << 20
FWD_O_FP32 = 1
BWD_SERIAL = 1
BWD_CONCURRENT = 2
BWD_DQ_STORE_BF16 = 4
FWD_LSE_NATURAL = 2
FWD_SINGLE_CTA = 4
FWD_CTA_PAIR = 8
COMBINE_NATURAL = 1
DTYPE_BF16 = 0
DTYPE_F32 = 1

# Every symbol include/pith_b200.h declares: name -> (restype, argtypes)
EXPORTS = {
    "pith_attn_fwd": (c_int, [POINTER(AttnFwdArgs), c_void_p]),
    "pith_attn_bwd_preprocess": (c_int, [POINTER(BwdPreprocessArgs), c_void_p]),
    "pith_attn_bwd": (c_int, [POINTER(AttnBwdArgs), c_void_p]),
    "pith_cast_f32_to_bf16": (c_int, [c_void_p, c_void_p, c_int32, c_int32, c_int32, c_int32,
                                      POINTER(c_int64), POINTER(c_int64), c_float, c_void_p]),
    "pith_combine": (c_int, [POINTER(CombineArgs), c_void_p]),
    "pith_combine_partials": (c_int, [POINTER(CombinePartialsArgs), c_void_p]),
    "pith_attn_bwd_noalloc": (c_int, [POINTER(AttnBwdNoallocArgs), c_void_p]),
    "pith_attn_bwd_noalloc_scratch_bytes": (ctypes.c_size_t, [c_int32] * 7),
    "pith_flag_signal": (c_int, [c_void_p, c_void_p, c_void_p]),
    "pith_flag_wait": (c_int, [c_void_p, c_void_p, ctypes.c_double, c_void_p, c_void_p]),
    "pith_enable_peer_access": (c_int, [c_int32]),
    "pith_ipc_export": (c_int, [c_void_p, c_void_p, POINTER(ctypes.c_uint64)]),
    "pith_ipc_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "pith_ipc_close": (c_int, [c_void_p]),
    "pith_peer_copy": (c_int, [c_void_p, c_void_p, ctypes.c_size_t, c_void_p]),
    "pith_qk_norm_rope_fwd": (c_int, [POINTER(QkNormRopeArgs), c_void_p]),
    "pith_qk_norm_rope_bwd": (c_int, [POINTER(QkNormRopeArgs), c_void_p]),
    "pith_mla_assemble_fwd": (c_int, [POINTER(MlaAssembleArgs), c_void_p]),
    "pith_mla_assemble_bwd": (c_int, [POINTER(MlaAssembleArgs), c_void_p]),
    "pith_last_error": (c_char_p, []),
    "pith_status_string": (c_char_p, [c_uint32]),
    "pith_abi_version": (c_int, []),
}

_lib = None


class PithLibraryError(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Loads the library (once) and types every export. Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise PithLibraryError(
                f"{LIB_PATH} is missing: build it with `python -m pithtrain_b200.build` "
                "(there is no CPU or PyTorch fallback for these operators)")
        lib = ctypes.CDLL(str(LIB_PATH))
        for name, (res, args) in EXPORTS.items():
            fn = getattr(lib, name)  # AttributeError if the export is missing
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().pith_last_error()
        raise PithLibraryError(f"{what} rejected (code {rc}): {msg.decode() if msg else ''}")
