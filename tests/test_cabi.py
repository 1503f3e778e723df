"""The C-ABI library: builds, loads on a machine without a GPU, exports what the header declares, and rejects
bad arguments on the host with a message (no kernel is launched here)."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "pith_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pith_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_all_exported(built_library):
    from pithtrain_b200 import _lib
    lib = ctypes.CDLL(str(built_library))
    names = declared_symbols()
    assert "pith_attn_fwd" in names and "pith_attn_bwd" in names and "pith_combine" in names
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/pith_b200.h but not exported"
        assert n in _lib.EXPORTS, f"{n} has no ctypes signature in pithtrain_b200._lib"
    assert sorted(_lib.EXPORTS) == names


def test_abi_version_and_status_strings(built_library):
    from pithtrain_b200 import _lib
    lib = _lib.load()
    assert lib.pith_abi_version() == 2
    assert lib.pith_status_string(0) == b"ok"
    assert b"timed out" in lib.pith_status_string((1 << 24) | 0x700)


def test_struct_sizes_match_the_header(built_library):
    """ctypes mirrors of the argument structs must have the C layout (checked against a compiled sizeof)."""
    import subprocess, tempfile, textwrap
    from pithtrain_b200 import _lib
    src = textwrap.dedent("""
        #include <stdio.h>
        #include "pith_b200.h"
        int main(void) {
          printf("%zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(pith_attn_fwd_args), sizeof(pith_bwd_preprocess_args),
                 sizeof(pith_attn_bwd_args), sizeof(pith_combine_args), sizeof(pith_attn_bwd_noalloc_args),
                 sizeof(pith_qk_norm_rope_args), sizeof(pith_mla_assemble_args), sizeof(pith_combine_partials_args));
          return 0;
        }""")
    with tempfile.TemporaryDirectory() as d:
        (Path(d) / "s.c").write_text(src)
        subprocess.run(["gcc", "-I", str(ROOT / "include"), str(Path(d) / "s.c"), "-o", str(Path(d) / "s")], check=True)
        sizes = [int(x) for x in subprocess.run([str(Path(d) / "s")], capture_output=True, text=True, check=True).stdout.split()]
    assert sizes == [ctypes.sizeof(_lib.AttnFwdArgs), ctypes.sizeof(_lib.BwdPreprocessArgs),
                     ctypes.sizeof(_lib.AttnBwdArgs), ctypes.sizeof(_lib.CombineArgs),
                     ctypes.sizeof(_lib.AttnBwdNoallocArgs), ctypes.sizeof(_lib.QkNormRopeArgs),
                     ctypes.sizeof(_lib.MlaAssembleArgs), ctypes.sizeof(_lib.CombinePartialsArgs)]


def test_host_side_rejections(built_library):
    from pithtrain_b200 import _lib
    lib = _lib.load()
    assert lib.pith_attn_fwd(None, None) < 0
    assert b"null args" in lib.pith_last_error()
    a = _lib.AttnFwdArgs()
    assert lib.pith_attn_fwd(ctypes.byref(a), None) < 0
    assert b"null tensor pointer" in lib.pith_last_error()
    a.q = a.k = a.v = a.o = a.lse = 0x1000
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.Dqk, a.Dv = 1, 128, 128, 6, 4, 128, 128
    a.softmax_scale = 0.1
    assert lib.pith_attn_fwd(ctypes.byref(a), None) < 0
    assert b"not a multiple" in lib.pith_last_error()
    a.Hq, a.Dqk = 8, 96
    assert lib.pith_attn_fwd(ctypes.byref(a), None) < 0
    assert b"unsupported head dims" in lib.pith_last_error()
    c = _lib.CombineArgs()
    c.out1 = c.out2 = c.lse1 = c.lse2 = c.out = c.lse = 0x1000
    c.B, c.S, c.H, c.D = 1, 4, 2, 12
    assert lib.pith_combine(ctypes.byref(c), None) < 0
    assert b"bad shape" in lib.pith_last_error()
    e = _lib.CombineArgs()
    e.B, e.S, e.H, e.D = 1, 0, 2, 128
    assert lib.pith_combine(ctypes.byref(e), None) == 0  # empty input: nothing to do, null pointers accepted
    cp = _lib.CombinePartialsArgs()
    cp.B, cp.S, cp.H, cp.D = 1, 256, 2, 128
    assert lib.pith_combine_partials(ctypes.byref(cp), None) < 0 and b"partials" in lib.pith_last_error()  # n = 0
    cp.n = _lib.MAX_PARTIALS + 1
    assert lib.pith_combine_partials(ctypes.byref(cp), None) < 0 and b"partials" in lib.pith_last_error()
    cp.n = 1
    cp.out = cp.lse = 0x1000
    cp.part[0].row_begin, cp.part[0].rows = 128, 256                       # runs past the 256 output rows
    assert lib.pith_combine_partials(ctypes.byref(cp), None) < 0 and b"covers rows" in lib.pith_last_error()
    cp.part[0].rows = 128
    assert lib.pith_combine_partials(ctypes.byref(cp), None) < 0 and b"null tensor pointer" in lib.pith_last_error()
    cp.S = 0
    assert lib.pith_combine_partials(ctypes.byref(cp), None) == 0          # empty output: nothing to do
    b = _lib.AttnBwdArgs()
    b.q = b.k = b.v = b.dout = b.lse = b.delta = 0x1000
    assert lib.pith_attn_bwd(ctypes.byref(b), None) < 0
    assert b"no gradient accumulator" in lib.pith_last_error()
    with pytest.raises(_lib.PithLibraryError):
        _lib.check(-1, "demo")


def test_host_side_rejections_of_the_front_end_and_peer_entries(built_library):
    from pithtrain_b200 import _lib
    lib = _lib.load()
    r = _lib.QkNormRopeArgs()
    r.B, r.S, r.Hq, r.Hkv, r.D = 1, 8, 2, 1, 64
    assert lib.pith_qk_norm_rope_fwd(ctypes.byref(r), None) < 0
    assert b"128 only" in lib.pith_last_error()
    r.D, r.S = 128, 0
    assert lib.pith_qk_norm_rope_fwd(ctypes.byref(r), None) == 0          # empty: nothing to do
    r.S = 8
    assert lib.pith_qk_norm_rope_bwd(ctypes.byref(r), None) < 0
    assert b"null weight" in lib.pith_last_error()
    m = _lib.MlaAssembleArgs()
    m.B, m.S, m.H, m.Dnope, m.Drope, m.Dv = 1, 8, 2, 128, 32, 128
    assert lib.pith_mla_assemble_fwd(ctypes.byref(m), None) < 0
    assert b"supported" in lib.pith_last_error()
    m.Drope, m.H = 64, 0
    assert lib.pith_mla_assemble_bwd(ctypes.byref(m), None) == 0           # empty
    assert lib.pith_flag_signal(None, None, None) < 0 and b"null flag" in lib.pith_last_error()
    assert lib.pith_flag_wait(0x1000, 0x1000, 0.0, None, None) < 0 and b"max_seconds" in lib.pith_last_error()
    assert lib.pith_ipc_open(None, None) < 0 and lib.pith_ipc_close(None) < 0
    assert lib.pith_peer_copy(None, None, 0, None) == 0                    # nothing to copy
    assert lib.pith_peer_copy(None, 0x1000, 16, None) < 0
