"""CPU-side checks of the C ABI: the library loads without a GPU, exports every symbol
the header declares, and the layout / argument validation behave (no compute calls)."""
import ctypes as C
import os
import re

import pytest

from mini_mega_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    _lib.build()
    return _lib.lib()


def _declared_functions():
    src = open(os.path.join(ROOT, "include", "mxk_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(mxk_[a-z0-9_]+)\s*\(", src)))


def test_every_declared_symbol_is_exported(lib):
    names = _declared_functions()
    assert len(names) >= 20
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/mxk_b200.h but not exported"
    assert sorted(_lib.EXPORTS) == names


def test_layout_is_consistent(lib):
    L = _lib.compute_layout(8, 3, 32, 8, 6144, 2048, 16)
    assert L.pool_rows == 8 * 16 * 8
    assert L.recv_stride >= 33 and L.sf_stride_h >= 48 and L.sf_stride_i >= 16
    offs = [L.x_off, L.x_sf_off, L.topk_idx_off, L.topk_weights_off]
    assert offs == sorted(offs) and L.sym_bytes > offs[-1]
    assert all(o % 256 == 0 for o in offs)
    g = _lib.MxkGeom(8, 3, 32, 8, 6144, 2048, 16, 0)
    assert lib.mxk_sym_bytes(C.byref(g)) == L.sym_bytes
    assert lib.mxk_rwk_bytes(C.byref(g)) == L.rwk_bytes
    assert lib.mxk_unk_bytes(C.byref(g)) == L.unk_bytes
    # prefill-sized world still fits comfortably in one B200's memory
    P = _lib.compute_layout(8, 0, 32, 8, 7168, 2048, 4096)
    assert P.rwk_bytes + P.unk_bytes + P.sym_bytes < 8 << 30


def test_push_protocol_choice_by_geometry(lib):
    """push_eligible: the world's routing fits a CTA's shared memory; push_auto: in addition at most 2048
    routed pairs of capacity per rank on one GPU, 1024 in a world of several ranks (the tagged rows then
    cross NVLink with twice their bytes): the batch sizes where pushing beats the pull round trips."""
    d = _lib.compute_layout(8, 0, 32, 8, 6144, 2048, 16)        # baseline decode: 128 pairs per rank
    assert d.push_eligible == 1 and d.push_auto == 1 and d.xin_off > 0
    m = _lib.compute_layout(8, 0, 32, 8, 6144, 2048, 128)       # 1024 pairs per rank: the edge in a world of 8
    assert m.push_eligible == 1 and m.push_auto == 1
    m = _lib.compute_layout(8, 0, 32, 8, 6144, 2048, 256)       # 2048 pairs per rank, 16384 in the world: may push
    assert m.push_eligible == 1 and m.push_auto == 0
    s1 = _lib.compute_layout(1, 0, 32, 8, 6144, 2048, 256)      # one GPU: no NVLink to pay for
    assert s1.push_eligible == 1 and s1.push_auto == 1
    q = _lib.compute_layout(1, 0, 8, 8, 7168, 2048, 1024)       # one rank, 8192 pairs: may push, does not by default
    assert q.push_eligible == 1 and q.push_auto == 0
    p = _lib.compute_layout(8, 0, 32, 8, 7168, 2048, 4096)      # prefill-sized: pull only
    assert p.push_eligible == 0 and p.push_auto == 0


@pytest.mark.parametrize("geom", [
    (0, 0, 8, 8, 6144, 2048, 16, 0),      # no ranks
    (2, 2, 8, 8, 6144, 2048, 16, 0),      # rank out of range
    (1, 0, 8, 8, 6100, 2048, 16, 0),      # hidden not a multiple of 256
    (1, 0, 8, 8, 6144, 2000, 16, 0),      # intermediate not a multiple of 128
    (1, 0, 8, 0, 6144, 2048, 16, 0),      # topk
    (1, 0, 8, 8, 6144, 2048, 0, 0),       # max_tokens
])
def test_bad_geometry_is_rejected(lib, geom):
    g = _lib.MxkGeom(*geom)
    out = _lib.MxkLayout()
    assert lib.mxk_compute_layout(C.byref(g), C.byref(out)) == -1
    assert len(lib.mxk_last_error()) > 0


def test_launch_argument_validation_needs_no_gpu(lib):
    a = _lib.MxkLaunchArgs()
    a.R, a.rank, a.tokens = 1, 0, 4
    a.experts_per_rank, a.topk, a.hidden, a.intermediate, a.max_tokens = 8, 2, 512, 256, 32
    assert lib.mxk_launch_full(C.byref(a), None) == -1      # null buffers
    assert b"non-null" in lib.mxk_last_error()
    a.hidden = 500
    assert lib.mxk_launch_full(C.byref(a), None) == -1
    assert lib.mxk_launch_full(None, None) == -1
    assert lib.mxk_launch_empty(0, 32, 0, None) == -1


def test_select_win_matches_reference_golden(lib):
    import numpy as np
    g = np.load(os.path.join(ROOT, "tests", "golden", "sched.npz"))
    for ci in range(6):
        counts = np.ascontiguousarray(g[f"win_{ci}_counts"])
        got = [lib.mxk_select_win(counts.ctypes.data_as(C.POINTER(C.c_uint32)), 256, cap, wmin)
               for cap in (64, 96, 128) for wmin in (8, 32)]
        assert got == g[f"win_{ci}_out"].tolist()


def test_ctypes_mirrors_match_the_c_header(tmp_path):
    """Sizes and the offsets of the last fields of the three structs, as a C compiler lays out
    include/mxk_b200.h, against the ctypes mirrors in mini_mega_b200/_lib.py."""
    import subprocess
    src = tmp_path / "sizes.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "mxk_b200.h"\n'
        'int main(void) {\n'
        '  printf("%zu %zu %zu %zu\\n", sizeof(MxkLaunchArgs), offsetof(MxkLaunchArgs, weight_format),\n'
        '         offsetof(MxkLaunchArgs, w1_group), offsetof(MxkLaunchArgs, dispatch_mode));\n'
        '  printf("%zu %zu %zu\\n", sizeof(MxkLayout), offsetof(MxkLayout, push_auto), offsetof(MxkLayout, xin_off));\n'
        '  printf("%zu %zu %zu\\n", sizeof(MxkStatus), offsetof(MxkStatus, ticks), offsetof(MxkStatus, trace));\n'
        '  printf("%zu\\n", sizeof(MxkGeom));\n'
        '  return 0;\n}\n')
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split("\n")
    la, lay, st = _lib.MxkLaunchArgs, _lib.MxkLayout, _lib.MxkStatus
    assert [int(v) for v in out[0].split()] == [C.sizeof(la), la.weight_format.offset, la.w1_group.offset, la.dispatch_mode.offset]
    assert [int(v) for v in out[1].split()] == [C.sizeof(lay), lay.push_auto.offset, lay.xin_off.offset]
    assert [int(v) for v in out[2].split()] == [C.sizeof(st), st.ticks.offset, st.trace.offset]
    assert int(out[3]) == C.sizeof(_lib.MxkGeom)
