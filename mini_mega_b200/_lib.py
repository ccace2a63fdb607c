"""ctypes binding of libmxk_b200.so (the C ABI of include/mxk_b200.h).

The CUDA library is the product path: if it is missing this module raises, it
never falls back to a CPU implementation.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmxk_b200.so")
SRC_DIR = os.path.join(_HERE, "csrc")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile csrc/mxk_kernels.cu for sm_100a into libmxk_b200.so (in-tree)."""
    srcs = [os.path.join(SRC_DIR, f) for f in ("mxk_kernels.cu", "mxk_device.cuh", "mxk_phases.cuh", "mxk_gemm.cuh",
                                               "mxk_sched.cuh")]
    hdr = os.path.join(os.path.dirname(_HERE), "include", "mxk_b200.h")
    newest = max(os.path.getmtime(p) for p in srcs + [hdr])
    if not force and os.path.exists(LIB_PATH) and os.path.getmtime(LIB_PATH) >= newest:
        return LIB_PATH
    cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB_PATH, srcs[0]]
    subprocess.run(cmd, check=True)
    return LIB_PATH


class MxkGeom(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("R", "rank", "experts_per_rank", "topk", "hidden", "intermediate",
                                          "max_tokens", "slot_capacity")]


class MxkLayout(C.Structure):
    _fields_ = [
        ("sym_bytes", C.c_int64), ("x_off", C.c_int64), ("x_sf_off", C.c_int64), ("topk_idx_off", C.c_int64),
        ("topk_weights_off", C.c_int64),
        ("unk_bytes", C.c_int64), ("src_index_table_off", C.c_int64),
        ("expert_recv_counts_off", C.c_int64), ("combine_rows_off", C.c_int64), ("combine_cnt_off", C.c_int64),
        ("recv_stride", C.c_int32),
        ("rwk_bytes", C.c_int64), ("flags_off", C.c_int64), ("route_slot_counts_off", C.c_int64),
        ("pair_state_off", C.c_int64), ("prefix_tbl_off", C.c_int64), ("expert_row_base_off", C.c_int64),
        ("windows_off", C.c_int64), ("tasks_off", C.c_int64), ("l1_done_off", C.c_int64),
        ("row_meta_off", C.c_int64), ("pool_off", C.c_int64), ("pool_sf_off", C.c_int64), ("ffn_off", C.c_int64),
        ("ffn_sf_off", C.c_int64), ("pool_rows", C.c_int64),
        ("sf_stride_h", C.c_int32), ("sf_stride_i", C.c_int32), ("max_windows", C.c_int32), ("max_tasks", C.c_int32),
        ("pool_ready_off", C.c_int64), ("expert_first_win_off", C.c_int64),
        ("xin_off", C.c_int64), ("xin_src_words", C.c_int64), ("xin_row_words", C.c_int32),
        ("push_eligible", C.c_int32),
        ("route_scratch_off", C.c_int64), ("route_scratch_ctas", C.c_int32), ("push_auto", C.c_int32),
    ]


class MxkLaunchArgs(C.Structure):
    _fields_ = [
        ("R", C.c_int32), ("rank", C.c_int32), ("tokens", C.c_int32), ("slot_capacity", C.c_int32),
        ("win_cap", C.c_int32), ("grid", C.c_int32), ("threads", C.c_int32), ("smem", C.c_int64),
        ("rwk", C.c_void_p), ("unk", C.c_void_p), ("unk_peers", C.c_void_p), ("self", C.c_void_p),
        ("peer_bases", C.c_void_p), ("topk_idx", C.c_void_p), ("w1", C.c_void_p), ("w2", C.c_void_p),
        ("group_weights_ready", C.c_int32),
        ("topk_idx_off", C.c_int64), ("x_off", C.c_int64), ("weights_off", C.c_int64),
        ("in_bf16", C.c_int32), ("skip_combine", C.c_int32), ("y", C.c_void_p),
        ("max_spins", C.c_int32), ("skip_prologue", C.c_int32),
        ("experts_per_rank", C.c_int32), ("topk", C.c_int32), ("hidden", C.c_int32), ("intermediate", C.c_int32),
        ("max_tokens", C.c_int32),
        ("x_sf_off", C.c_int64), ("w1_sf", C.c_void_p), ("w2_sf", C.c_void_p), ("y_bf16", C.c_void_p),
        ("cta_pair", C.c_int32), ("dispatch_mode", C.c_int32),
        ("group_ranks", C.c_int32), ("group_skew_num", C.c_int32),
        ("w1_group", C.c_void_p), ("w2_group", C.c_void_p), ("w1_sf_group", C.c_void_p), ("w2_sf_group", C.c_void_p),
        ("weight_format", C.c_int32), ("group_hot_windows", C.c_int32),
    ]


class MxkStatus(C.Structure):
    _fields_ = [("launches", C.c_int64), ("status", C.c_int32), ("n_tasks", C.c_int32), ("n_l1_tasks", C.c_int32),
                ("n_windows", C.c_int32), ("total_rows", C.c_int32), ("helper_on", C.c_int32), ("dbg", C.c_int32 * 8),
                ("ticks", C.c_uint64 * 16), ("trace", C.c_uint64 * 64)]


# every symbol include/mxk_b200.h declares; tests check that the library exports them
EXPORTS = [
    "mxk_last_error", "mxk_version", "mxk_compute_layout", "mxk_sym_bytes", "mxk_rwk_bytes", "mxk_unk_bytes",
    "mxk_launch_prelude", "mxk_launch_compute", "mxk_launch_reduce", "mxk_launch_full", "mxk_launch_empty",
    "mxk_kernels_per_layer", "mxk_launch_phases", "mxk_launch_full_static",
    "mxk_static_scratch_bytes", "mxk_fill_weights", "mxk_fill_weights_e2m1", "mxk_e2m1_to_e4m3", "mxk_quantize_rows", "mxk_dump_kernel_resources", "mxk_read_status",
    "mxk_read_status_static", "mxk_rwk_ticks_off", "mxk_ticks_count", "mxk_set_ticks", "mxk_select_win",
    "mxk_group_ranks", "mxk_gs_schedule_member", "mxk_gs_schedule_member_hot", "mxk_gs_group_skewed", "mxk_lpt_assign", "mxk_gs_schedule_on_device",
    "mxk_symm_alloc", "mxk_symm_free", "mxk_ipc_export", "mxk_ipc_import", "mxk_ipc_close",
]

_LIB = None


class MxkError(RuntimeError):
    pass


def lib():
    """Load the CUDA library; raises if it has not been built."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        raise MxkError(f"{LIB_PATH} is missing: run mini_mega_b200._lib.build() (needs nvcc); "
                       "there is no CPU fallback")
    L = C.CDLL(LIB_PATH)
    L.mxk_last_error.restype = C.c_char_p
    L.mxk_compute_layout.argtypes = [C.POINTER(MxkGeom), C.POINTER(MxkLayout)]
    for n in ("mxk_sym_bytes", "mxk_rwk_bytes", "mxk_unk_bytes"):
        getattr(L, n).restype = C.c_int64
        getattr(L, n).argtypes = [C.POINTER(MxkGeom)]
    for n in ("mxk_launch_prelude", "mxk_launch_compute", "mxk_launch_reduce", "mxk_launch_full"):
        getattr(L, n).argtypes = [C.POINTER(MxkLaunchArgs), C.c_void_p]
    L.mxk_launch_full_static.argtypes = [C.POINTER(MxkLaunchArgs), C.c_void_p]
    L.mxk_static_scratch_bytes.restype = C.c_int64
    L.mxk_launch_phases.argtypes = [C.POINTER(MxkLaunchArgs), C.c_int, C.c_void_p]
    L.mxk_launch_empty.argtypes = [C.c_int, C.c_int, C.c_int64, C.c_void_p]
    L.mxk_fill_weights.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_uint32, C.c_void_p]
    L.mxk_fill_weights_e2m1.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_uint32, C.c_void_p]
    L.mxk_e2m1_to_e4m3.argtypes = [C.c_uint8]
    L.mxk_e2m1_to_e4m3.restype = C.c_uint8
    L.mxk_quantize_rows.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    L.mxk_read_status.argtypes = [C.c_void_p, C.POINTER(MxkStatus)]
    L.mxk_read_status_static.argtypes = [C.POINTER(MxkStatus)]
    L.mxk_rwk_ticks_off.restype = C.c_int64
    L.mxk_ticks_count.restype = C.c_int64
    L.mxk_set_ticks.argtypes = [C.c_int]
    i32p = C.POINTER(C.c_int32)
    L.mxk_gs_schedule_member.argtypes = [i32p, C.c_int, C.c_int, C.c_int, C.c_int, i32p, i32p, C.c_int]
    L.mxk_gs_group_skewed.argtypes = [i32p, C.c_int, C.c_int]
    L.mxk_lpt_assign.argtypes = [i32p, i32p, C.c_int, C.c_int, C.c_int, C.c_int, i32p, i32p, C.POINTER(C.c_int64), C.c_int]
    L.mxk_gs_schedule_member_hot.argtypes = [i32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, i32p, i32p, C.c_int]
    L.mxk_gs_schedule_on_device.argtypes = [i32p, C.c_int, C.c_int, C.c_int, C.c_int, i32p, i32p, i32p, C.c_int]
    L.mxk_select_win.argtypes = [C.POINTER(C.c_uint32), C.c_int, C.c_int, C.c_int]
    L.mxk_symm_alloc.argtypes = [C.POINTER(C.c_void_p), C.c_int64]
    L.mxk_symm_free.argtypes = [C.c_void_p]
    L.mxk_ipc_export.argtypes = [C.c_void_p, C.c_char_p]
    L.mxk_ipc_import.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    L.mxk_ipc_close.argtypes = [C.c_void_p]
    _LIB = L
    return L


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = lib().mxk_last_error().decode(errors="replace")
        raise MxkError(f"{what or 'mxk call'} failed (code {rc}): {msg}")


def compute_layout(R, rank, experts_per_rank, topk, hidden, intermediate, max_tokens, slot_capacity=0) -> MxkLayout:
    g = MxkGeom(R, rank, experts_per_rank, topk, hidden, intermediate, max_tokens, slot_capacity)
    out = MxkLayout()
    check(lib().mxk_compute_layout(C.byref(g), C.byref(out)), "mxk_compute_layout")
    return out
