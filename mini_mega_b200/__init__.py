"""mini_mega_b200 — B200 (sm_100a) FP8xFP8 MoE layer behind the reference's host interface.

The package holds the CUDA library (``csrc/`` -> ``libmxk_b200.so``, C ABI in
``include/mxk_b200.h``) and a Python mirror of the reference's torch layer.
There is no CPU fallback: importing works anywhere, launching needs the built
library and a B200.
"""
from . import _lib, quant  # noqa: F401
from .mega import (  # noqa: F401
    SymmBuffer,
    bf16_fp8_mega_moe,
    bf16_mega_moe,
    fp8_fp4_mega_moe,
    fp8_mega_moe,
    fp8_mega_moe_compute,
    fp8_mega_moe_reduce,
    gather_group_weights,
    get_symm_buffer_for_mega_moe,
    get_symm_buffer_size_for_mega_moe,
    get_token_alignment_for_mega_moe,
    read_dbg_report,
    select_fp8_mega_moe_window,
    transform_weights_for_mega_moe,
)

__version__ = "0.1.0"
