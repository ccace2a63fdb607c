"""The drop-in C++ header include/megakernel.h, compiled and called like the reference's own
callers do (test/check.cu:171-172,204-205; test/mybench.cu:222-237): tests/cpp/consumer.cpp
fills fp8mega::MegaLaunchArgs and calls the fp8mega launchers; its static_asserts pin the
C++ struct to the C twin field by field.  CPU: it compiles, links libmxk_b200.so and reports
a bad-argument status for null buffers.  GPU: the toy layer through launch_full and through
launch_compute + launch_reduce equals the oracle / the ctypes path bit for bit."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from mini_mega_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "consumer.cpp")
OUT = os.path.join(ROOT, "tests", "cpp", "libconsumer.so")
CUDA_INC = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")


class ConsumerArgs(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("tokens", "experts", "topk", "hidden", "intermediate", "max_tokens")] + \
               [(n, C.c_void_p) for n in ("rwk", "unk", "unk_peers", "sym", "peer_bases", "w1", "w2", "w1_sf", "w2_sf",
                                          "y", "y_bf16")] + \
               [(n, C.c_int64) for n in ("topk_idx_off", "x_off", "weights_off", "x_sf_off")] + [("mode", C.c_int32)]


@pytest.fixture(scope="module")
def consumer():
    _lib.build()
    deps = [SRC, os.path.join(ROOT, "include", "megakernel.h"), os.path.join(ROOT, "include", "mxk_b200.h")]
    if not os.path.exists(OUT) or os.path.getmtime(OUT) < max(os.path.getmtime(p) for p in deps + [_lib.LIB_PATH]):
        libdir = os.path.dirname(_lib.LIB_PATH)
        subprocess.run(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                        "-I", CUDA_INC, SRC, "-o", OUT, "-L", libdir, "-l:libmxk_b200.so", f"-Wl,-rpath,{libdir}"],
                       check=True)
    lib = C.CDLL(OUT)
    lib.consumer_run.argtypes = [C.POINTER(ConsumerArgs), C.c_void_p]
    lib.consumer_wprobe.restype = C.c_uint8
    return lib


def test_header_compiles_and_reports_bad_arguments(consumer):
    assert consumer.consumer_null_buffers() == -1      # MXK_ERR_BAD_ARG through fp8mega::last_status()
    assert b"non-null" in _lib.lib().mxk_last_error()
    assert consumer.consumer_wprobe(17, 3, 5) == ((17 + 3 * 131 + 5 * 7) & 0x3F)


@pytest.mark.gpu
def test_cpp_caller_runs_the_toy_layer(consumer):
    import torch

    import mini_mega_b200 as mm
    from oracle import oracle as orc
    case = orc.gen_case(1, 8, 2, 512, 256, 32, seed=51, routing="logits", scaled=True)
    want = orc.layer_world(case)[0].y
    buf = mm.get_symm_buffer_for_mega_moe(None, 8, 32, 2, 512, 256)
    try:
        from gpu_world import dev_weights, load_inputs
        load_inputs(case, [buf])
        (w1, s1), (w2, s2) = dev_weights(case, 0)
        L = buf.layout
        y32 = torch.zeros((32, 512), dtype=torch.float32, device="cuda")
        y16 = torch.zeros((32, 512), dtype=torch.bfloat16, device="cuda")
        a = ConsumerArgs(32, 8, 2, 512, 256, 32, buf.rwk.data_ptr(), buf._unk_ptr, buf._unk_peers.data_ptr(), buf._sym_ptr,
                         buf._peer_bases.data_ptr(), w1.data_ptr(), w2.data_ptr(), s1.data_ptr(), s2.data_ptr(),
                         y32.data_ptr(), y16.data_ptr(), L.topk_idx_off, L.x_off, L.topk_weights_off, L.x_sf_off, 0)
        st = torch.cuda.current_stream().cuda_stream
        assert consumer.consumer_run(C.byref(a), st) == 0          # fp8mega::launch_full
        torch.cuda.synchronize()
        assert buf.status().status == 0
        full = y32.clone()
        assert orc.rel_l2(full.cpu().numpy(), want) <= 1e-2
        y32.zero_()
        a.mode = 1                                                  # launch_compute, then launch_reduce
        assert consumer.consumer_run(C.byref(a), st) == 0
        torch.cuda.synchronize()
        assert buf.status().status == 0 and buf.status().launches == 2
        assert torch.equal(y32, full)
        a.mode = 2                                                  # launch_prelude: tables only
        assert consumer.consumer_run(C.byref(a), st) == 0
        torch.cuda.synchronize()
        ref = orc.route_world(case)[0]
        assert np.array_equal(buf.table("prefix_tbl").cpu().numpy(), ref.prefix_tbl)
        a.mode = 3                                                  # launch_empty
        assert consumer.consumer_run(C.byref(a), st) == 0
        torch.cuda.synchronize()
    finally:
        buf.destroy()
