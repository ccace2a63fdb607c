"""Host-side mirror of the reference's torch layer for the MoE hot path.

Same names and argument meaning as ``torch/mxmegakernel/mega/__init__.py`` of
the reference (``SymmBuffer`` :144-276, ``get_symm_buffer_for_mega_moe`` :478-490,
``transform_weights_for_mega_moe`` :553-573, ``fp8_mega_moe`` :610-655,
``fp8_mega_moe_compute`` / ``fp8_mega_moe_reduce`` :658-712), on top of the C ABI of
``include/mxk_b200.h``.  PyTorch supplies device memory, streams and the process
group used to exchange IPC handles; all compute is in ``libmxk_b200.so``.

Differences the B200 design makes visible:
  * geometry is a run-time property of the buffer (the reference freezes
    EPR=8 / topk=8 / H=6144 / I=2048, ``mega/__init__.py`` FROZEN_* constants);
  * UE8M0 block scales are supported: ``buffer.x_sf`` is a uint8 ``[cap, H/128]``
    view and the weights may be ``(fp8, scale)`` tuples;
  * weights stay in plain row-major ``[EPR, 2I, H]`` (gate rows, then up rows)
    and ``[EPR, H, I]``: TMA applies the shared-memory swizzle, so
    ``transform_weights_for_mega_moe`` only normalises dtypes;
  * ``y`` is written as bf16 by the reduce kernel itself.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple, Union

import torch
import torch.distributed as dist

from . import _lib
from ._lib import MxkLaunchArgs, MxkStatus, check, compute_layout

EXPERT_WINDOW_MIN = 8
EXPERT_WINDOW_MAX = 128
EXPERT_WINDOW_MULTIPLE = 8
_SUPPORTED_MMA_TYPES = ("fp8xfp8", "bf16xfp8", "fp8xfp4")   # fp8xfp4: the buffer of fp8xfp8, 4-bit weights at launch


class _DevMem:
    """Raw device allocation exposed to torch through __cuda_array_interface__."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _view(buf: torch.Tensor, dtype: torch.dtype, shape: Tuple[int, ...], offset_bytes: int) -> torch.Tensor:
    n = 1
    for s in shape:
        n *= int(s)
    itemsize = torch.empty((), dtype=dtype).element_size()
    return buf[offset_bytes: offset_bytes + n * itemsize].view(dtype).view(*shape)


def select_fp8_mega_moe_window(num_tokens: int, num_topk: int, num_ranks: int, num_experts: int,
                               mma_type: str = "fp8xfp8") -> int:
    """Rows per window (the UMMA M tile is 128, so 128 unless fewer rows can ever arrive)."""
    rows = max(1, num_tokens * num_ranks)  # a token picks an expert at most once
    win = min(EXPERT_WINDOW_MAX, (rows + 7) // 8 * 8)
    return max(EXPERT_WINDOW_MIN, win)


def get_token_alignment_for_mega_moe() -> int:
    return 1


def get_symm_buffer_size_for_mega_moe(num_ranks: int, num_experts: int, num_max_tokens_per_rank: int,
                                      num_topk: int, hidden: int, intermediate_hidden: int,
                                      num_shared_experts: int = 0, mma_type: str = "fp8xfp8",
                                      num_tokens: int = 0, expert_window: int = 0) -> int:
    L = compute_layout(num_ranks, 0, num_experts // num_ranks, num_topk, hidden, intermediate_hidden,
                       num_max_tokens_per_rank)
    return int(L.sym_bytes)


class SymmBuffer:
    """Symmetric buffers of one rank: ``sym`` (inputs, peers read), ``unk`` (peers write),
    ``rwk`` (private).  ``sym``/``unk`` come from ``mxk_symm_alloc`` so that they can be
    exported to the other ranks' processes; with ``group`` set, handles are exchanged with
    ``all_gather_object`` and the peers' blocks mapped (reference: ``mega/__init__.py``:224-243)."""

    def __init__(self, group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int, hidden: int,
                 intermediate_hidden: int, num_shared_experts: int = 0, mma_type: str = "fp8xfp8",
                 activation: str = "swiglu", grid_num_tokens: Optional[int] = None,
                 expert_window: Optional[int] = None, slot_capacity: int = 0, dispatch_mode: int = 0,
                 group_ranks: int = 0, group_skew_num: int = 0, group_hot_windows: int = 0,
                 _local_world: Optional[Tuple[int, int]] = None):
        if activation != "swiglu":
            raise ValueError(f"Only `swiglu` activation is supported, got `{activation}`")
        if mma_type not in _SUPPORTED_MMA_TYPES:
            raise NotImplementedError(f"only {_SUPPORTED_MMA_TYPES} is implemented, got mma_type={mma_type!r}")
        if num_shared_experts != 0:
            raise NotImplementedError("shared experts are not supported")
        if _local_world is not None:
            world_size, rank = _local_world  # several ranks inside one process, see local_world()
        elif group is None:
            world_size, rank = 1, 0
        else:
            world_size, rank = int(group.size()), int(group.rank())
        if num_experts % world_size:
            raise ValueError("num_experts must be divisible by the group size")
        cap = int(num_max_tokens_per_rank)
        if expert_window is None:
            expert_window = select_fp8_mega_moe_window(cap, num_topk, world_size, num_experts, mma_type)
        if (expert_window < EXPERT_WINDOW_MIN or expert_window > EXPERT_WINDOW_MAX
                or expert_window % EXPERT_WINDOW_MULTIPLE):
            raise ValueError(f"expert_window must be a multiple of 8 in [8,128], got {expert_window}")
        self.group, self.world_size, self.rank = group, world_size, rank
        self.num_experts = int(num_experts)
        self.num_experts_per_rank = self.num_experts // world_size
        self.num_max_tokens_per_rank = cap
        self.num_topk = int(num_topk)
        self.hidden, self.intermediate_hidden = int(hidden), int(intermediate_hidden)
        self.mma_type, self.activation = mma_type, activation
        self.expert_window = int(expert_window)
        self.slot_capacity = int(slot_capacity)
        self.dispatch_mode = int(dispatch_mode)
        # cross-rank helper scheduling for skewed routing (reference: MX_GROUP_SCHED): ranks per helper
        # group and the skew threshold; the group's weights are handed to the layer call
        self.group_ranks = int(group_ranks)
        self.group_skew_num = int(group_skew_num)
        # helper groups spread the windows of experts with at least this many windows (0 = 3; negative =
        # every window may move, the reference's schedule)
        self.group_hot_windows = int(group_hot_windows)
        if self.group_ranks > 1 and world_size % self.group_ranks:
            raise ValueError("group_ranks must divide the group size")
        self.launch_count = 0
        self.device = torch.cuda.current_device()
        self.layout = compute_layout(world_size, rank, self.num_experts_per_rank, self.num_topk, self.hidden,
                                     self.intermediate_hidden, cap, self.slot_capacity)
        L = self.layout
        lib = _lib.lib()
        self._owned, self._imported = [], []
        self._sym_ptr = self._alloc(int(L.sym_bytes))
        self._unk_ptr = self._alloc(int(L.unk_bytes))
        self.buffer = torch.as_tensor(_DevMem(self._sym_ptr, int(L.sym_bytes)), device=f"cuda:{self.device}")
        self.unk = torch.as_tensor(_DevMem(self._unk_ptr, int(L.unk_bytes)), device=f"cuda:{self.device}")
        self.rwk = torch.zeros(int(L.rwk_bytes), dtype=torch.uint8, device=f"cuda:{self.device}")

        sym_ptrs, unk_ptrs = [self._sym_ptr] * world_size, [self._unk_ptr] * world_size
        if world_size > 1 and _local_world is None:
            hs, hu = C.create_string_buffer(64), C.create_string_buffer(64)
            check(lib.mxk_ipc_export(self._sym_ptr, hs), "mxk_ipc_export(sym)")
            check(lib.mxk_ipc_export(self._unk_ptr, hu), "mxk_ipc_export(unk)")
            mine = (bytes(hs.raw), bytes(hu.raw))
            allh = [None] * world_size
            dist.all_gather_object(allh, mine, group=group)
            for r in range(world_size):
                if r == rank:
                    continue
                ps, pu = C.c_void_p(), C.c_void_p()
                check(lib.mxk_ipc_import(allh[r][0], C.byref(ps)), "mxk_ipc_import(sym)")
                check(lib.mxk_ipc_import(allh[r][1], C.byref(pu)), "mxk_ipc_import(unk)")
                self._imported += [ps.value, pu.value]
                sym_ptrs[r], unk_ptrs[r] = ps.value, pu.value
            dist.barrier(group=group)
        self._peer_bases = torch.tensor(sym_ptrs, dtype=torch.int64, device=f"cuda:{self.device}")
        self._unk_peers = torch.tensor(unk_ptrs, dtype=torch.int64, device=f"cuda:{self.device}")

        # fp8xfp8: `x` is the E4M3 region peers pull from.  bf16xfp8 (reference:
        # torch/mxmegakernel/mega/__init__.py:244-246): `x` is a private bf16 tensor the caller
        # fills; every layer call first quantises it into the E4M3 region `x_fp8` + `x_sf`
        # (one byte per element still crosses NVLink).
        self.x_fp8 = _view(self.buffer, torch.float8_e4m3fn, (cap, self.hidden), int(L.x_off))
        self.x_sf = _view(self.buffer, torch.uint8, (cap, self.hidden // 128), int(L.x_sf_off))
        if mma_type == "bf16xfp8":
            self.x = torch.zeros((cap, self.hidden), dtype=torch.bfloat16, device=f"cuda:{self.device}")
        else:
            self.x = self.x_fp8
        self.topk_idx = _view(self.buffer, torch.int64, (cap, self.num_topk), int(L.topk_idx_off))
        self.topk_weights = _view(self.buffer, torch.float32, (cap, self.num_topk), int(L.topk_weights_off))
        torch.cuda.synchronize()

    @classmethod
    def local_world(cls, world_size: int, num_experts: int, num_max_tokens_per_rank: int, num_topk: int,
                    hidden: int, intermediate_hidden: int, **kw):
        """All ranks of a world inside ONE process on the current device (no IPC): the
        peer tables simply point at each other's blocks.  Because kernels of different
        ranks wait on each other, such a world must be driven phase by phase with
        ``mxk_launch_phases`` (every rank's ROUTE, then every rank's SETUP, ...)."""
        bufs = [cls(None, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
                    _local_world=(world_size, r), **kw) for r in range(world_size)]
        dev = f"cuda:{bufs[0].device}"
        sym = torch.tensor([b._sym_ptr for b in bufs], dtype=torch.int64, device=dev)
        unk = torch.tensor([b._unk_ptr for b in bufs], dtype=torch.int64, device=dev)
        for b in bufs:
            b._peer_bases, b._unk_peers = sym, unk
        torch.cuda.synchronize()
        return bufs

    def _alloc(self, nbytes: int) -> int:
        p = C.c_void_p()
        check(_lib.lib().mxk_symm_alloc(C.byref(p), nbytes), "mxk_symm_alloc")
        self._owned.append(p.value)
        return p.value

    # -- table views for tests / diagnostics (reference harness reads the same tables:
    #    test/mega_common.cuh:321-334, test/check.cu:183-195)
    def table(self, name: str) -> torch.Tensor:
        L, R, EPR = self.layout, self.world_size, self.num_experts_per_rank
        cap, topk, H, I = self.num_max_tokens_per_rank, self.num_topk, self.hidden, self.intermediate_hidden
        slot = self.slot_capacity or cap
        rows = int(L.pool_rows)
        spec = {
            "route_slot_counts": (self.rwk, torch.int32, (R * EPR,), L.route_slot_counts_off),
            "pair_state": (self.rwk, torch.uint8, (cap * topk,), L.pair_state_off),
            "prefix_tbl": (self.rwk, torch.int32, (EPR, R + 1), L.prefix_tbl_off),
            "expert_row_base": (self.rwk, torch.int32, (EPR + 1,), L.expert_row_base_off),
            "windows": (self.rwk, torch.int32, (L.max_windows, 4), L.windows_off),
            "tasks": (self.rwk, torch.int32, (L.max_tasks, 4), L.tasks_off),
            "row_meta": (self.rwk, torch.int32, (rows, 4), L.row_meta_off),
            "pool": (self.rwk, torch.uint8, (rows + 128, H), L.pool_off),
            "pool_sf": (self.rwk, torch.uint8, (rows, L.sf_stride_h), L.pool_sf_off),
            "ffn": (self.rwk, torch.uint8, (rows + 128, I), L.ffn_off),
            "ffn_sf": (self.rwk, torch.uint8, (rows, L.sf_stride_i), L.ffn_sf_off),
            # epoch-tagged 64-bit words: [..., 0] = payload, [..., 1] = launch epoch
            "src_index_table_raw": (self.unk, torch.int32, (2, EPR, R, slot, 2), L.src_index_table_off),
            "expert_recv_counts_raw": (self.unk, torch.int32, (2, R, L.recv_stride, 2), L.expert_recv_counts_off),
            "combine_rows": (self.unk, torch.int16, (topk, cap, H), L.combine_rows_off),
            "combine_cnt": (self.unk, torch.int32, (topk, cap), L.combine_cnt_off),
        }
        if name in ("src_index_table", "expert_recv_counts"):      # payload words only
            return self.table(name + "_raw")[..., 0]
        if name in ("src_index_table_tags", "expert_recv_counts_tags"):
            return self.table(name[:-5] + "_raw")[..., 1]
        spec = spec[name]
        return _view(spec[0], spec[1], spec[2], int(spec[3]))

    def packed_layout(self, num_tokens: int):
        """Offsets of a PACKED input image for `num_tokens` tokens: x, x_sf, topk_idx and
        topk_weights back to back (each region 256-byte aligned) from the start of the symmetric
        block, so that a host can bring a step's inputs over with ONE copy instead of four.
        Returns (x_off, x_sf_off, topk_idx_off, topk_weights_off, total_bytes).  Peers that pull
        rows address them with their own launch's offsets: either every rank packs for the same
        token count, or the buffer runs the push-mode prologue (which never reads a peer's block)."""
        T, H, topk = int(num_tokens), self.hidden, self.num_topk
        a256 = lambda v: (v + 255) // 256 * 256   # noqa: E731
        x_off = 0
        x_sf_off = a256(x_off + T * H)
        idx_off = a256(x_sf_off + T * (H // 128))
        w_off = a256(idx_off + T * topk * 8)
        return x_off, x_sf_off, idx_off, w_off, w_off + T * topk * 4

    def status(self) -> MxkStatus:
        st = MxkStatus()
        check(_lib.lib().mxk_read_status(self.rwk.data_ptr(), C.byref(st)), "mxk_read_status")
        return st

    def launch_args(self, num_tokens: int, l1=None, l2=None, y_bf16: Optional[torch.Tensor] = None,
                    y_f32: Optional[torch.Tensor] = None, expert_window: Optional[int] = None,
                    max_spins: int = 0, grid: int = 0, skip_combine: int = 0,
                    cta_pair: Optional[int] = None, dispatch_mode: Optional[int] = None,
                    packed: bool = False, group_weights=None, weight_format: int = 0) -> MxkLaunchArgs:
        L = self.layout
        a = MxkLaunchArgs()
        a.R, a.rank, a.tokens = self.world_size, self.rank, int(num_tokens)
        a.slot_capacity = self.slot_capacity
        a.win_cap = int(expert_window or self.expert_window)
        a.grid, a.threads, a.smem = grid, 0, 0
        a.rwk, a.unk = self.rwk.data_ptr(), self._unk_ptr
        a.unk_peers, a.self, a.peer_bases = self._unk_peers.data_ptr(), self._sym_ptr, self._peer_bases.data_ptr()
        a.topk_idx = None
        a.topk_idx_off, a.x_off, a.weights_off = L.topk_idx_off, L.x_off, L.topk_weights_off
        a.x_sf_off = L.x_sf_off
        if packed:   # inputs were copied in as one packed image, see packed_layout()
            a.x_off, a.x_sf_off, a.topk_idx_off, a.weights_off, _ = self.packed_layout(num_tokens)
        a.experts_per_rank, a.topk = self.num_experts_per_rank, self.num_topk
        a.hidden, a.intermediate, a.max_tokens = self.hidden, self.intermediate_hidden, self.num_max_tokens_per_rank
        a.max_spins, a.skip_combine = int(max_spins), int(skip_combine)
        for name, w in (("w1", l1), ("w2", l2)):
            if w is None:
                continue
            data, sf = w if isinstance(w, tuple) else (w, None)
            setattr(a, name, data.data_ptr())
            setattr(a, name + "_sf", None if sf is None else sf.data_ptr())
        a.y = None if y_f32 is None else y_f32.data_ptr()
        a.y_bf16 = None if y_bf16 is None else y_bf16.data_ptr()
        a.cta_pair = int(getattr(self, "cta_pair", 0) if cta_pair is None else cta_pair)
        # prologue protocol (0 automatic, 1 pull, 2 push): a property of the buffer because every
        # rank of a launch must use the same one
        a.dispatch_mode = int(self.dispatch_mode if dispatch_mode is None else dispatch_mode)
        if group_weights is not None and self.group_ranks > 1:
            for name, w in (("w1", group_weights[0]), ("w2", group_weights[1])):
                data, sf = w if isinstance(w, tuple) else (w, None)
                setattr(a, name + "_group", data.data_ptr())
                setattr(a, name + "_sf_group", None if sf is None else sf.data_ptr())
            a.group_ranks, a.group_skew_num, a.group_weights_ready = self.group_ranks, self.group_skew_num, 1
            a.group_hot_windows = self.group_hot_windows
        a.weight_format = int(weight_format)   # 0 = E4M3 bytes, 1 = packed e2m1 codes (every weight tensor of the launch)
        return a

    def group_members(self):
        """Ranks of this rank's helper group in member order (interleaved groups: group =
        rank % n_groups, member = rank // n_groups; reference src/group_sched.cuh:61-80)."""
        if self.group_ranks <= 1:
            return [self.rank]
        n_groups = self.world_size // self.group_ranks
        return [self.rank % n_groups + m * n_groups for m in range(self.group_ranks)]

    def destroy(self):
        lib = _lib.lib()
        torch.cuda.synchronize()
        for p in self._imported:
            lib.mxk_ipc_close(p)
        self._imported = []
        self.x = self.x_sf = self.topk_idx = self.topk_weights = None
        self.buffer = self.unk = None
        for p in self._owned:
            lib.mxk_symm_free(p)
        self._owned = []
        self.rwk = None


def get_symm_buffer_for_mega_moe(group, num_experts: int, num_max_tokens_per_rank: int, num_topk: int,
                                 hidden: int, intermediate_hidden: int, num_shared_experts: int = 0,
                                 use_fp8_dispatch: Optional[bool] = None, mma_type: str = "fp8xfp8",
                                 activation: str = "swiglu", num_tokens: Optional[int] = None,
                                 expert_window: Optional[int] = None, slot_capacity: int = 0,
                                 dispatch_mode: int = 0, group_ranks: int = 0, group_skew_num: int = 0,
                                 group_hot_windows: int = 0) -> SymmBuffer:
    if use_fp8_dispatch is not None:
        assert use_fp8_dispatch == (mma_type.split("x")[0] == "fp8")
    return SymmBuffer(group, num_experts, num_max_tokens_per_rank, num_topk, hidden, intermediate_hidden,
                      num_shared_experts, mma_type=mma_type, activation=activation, grid_num_tokens=num_tokens,
                      expert_window=expert_window, slot_capacity=slot_capacity, dispatch_mode=dispatch_mode,
                      group_ranks=group_ranks, group_skew_num=group_skew_num, group_hot_windows=group_hot_windows)


WeightArg = Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]


def _norm_weight(name: str, w: WeightArg, fp4: bool = False):
    data, sf = w if isinstance(w, tuple) else (w, None)
    ok = (torch.uint8, torch.int8) if fp4 else (torch.float8_e4m3fn, torch.uint8)
    if not isinstance(data, torch.Tensor) or data.dtype not in ok:
        raise TypeError(f"{name} must be a " + ("packed e2m1 (uint8 / int8) tensor" if fp4 else "float8_e4m3fn (or raw uint8) tensor"))
    if data.dim() != 3:
        raise ValueError(f"{name} must be [experts, rows, k]" + (" with k / 2 bytes per row" if fp4 else ""))
    data = data.contiguous().view(torch.uint8)
    if fp4 and data.data_ptr() % 32:
        data = data.clone()      # the 4-bit tensor map wants a 32-byte aligned base; fresh allocations are 256-byte aligned
    if sf is None:
        return data
    if sf.dtype == torch.float32:  # power-of-two floats as the reference quantisers return them
        bits = sf.contiguous().view(torch.int32)
        if bool(((bits & 0x7FFFFF) != 0).any()) or bool((bits < 0).any()):
            raise ValueError(f"{name} scales must be positive powers of two (UE8M0)")
        sf = (bits >> 23).to(torch.uint8)
    elif sf.dtype != torch.uint8:
        raise TypeError(f"{name} scales must be float32 powers of two or uint8 exponents")
    e, rows, k = data.shape
    k = 2 * k if fp4 else k
    if tuple(sf.shape) != (e, rows // 128, k // 128):
        raise ValueError(f"{name} scales must be [experts, rows/128, k/128], got {tuple(sf.shape)}")
    return data, sf.contiguous()


def transform_weights_for_mega_moe(l1_weights: WeightArg, l2_weights: WeightArg, activation: str = "swiglu",
                                   weight_format: str = "e4m3"):
    """Offline weight preparation.  ``l1`` is ``[EPR, 2I, H]`` with gate rows first, ``l2`` is
    ``[EPR, H, I]``; each may come with 128x128 UE8M0 block scales.  The B200 kernels read
    plain row-major bytes through TMA, so this only validates, makes contiguous and turns
    scale planes into exponent bytes (the reference re-tiles into MetaX lane order here).
    ``weight_format="e2m1"``: the tensors hold packed 4-bit codes, ``[EPR, rows, k / 2]`` bytes with the
    element of even k in the low nibble (``quant.per_block_cast_to_fp4``), for ``fp8_fp4_mega_moe``."""
    assert activation == "swiglu", f"Only `swiglu` supported, got `{activation}`"
    if weight_format not in ("e4m3", "e2m1"):
        raise ValueError(f"weight_format must be 'e4m3' or 'e2m1', got {weight_format!r}")
    fp4 = weight_format == "e2m1"
    l1, l2 = _norm_weight("l1_weights", l1_weights, fp4), _norm_weight("l2_weights", l2_weights, fp4)
    if isinstance(l1, tuple) != isinstance(l2, tuple):
        raise ValueError("l1 and l2 must both carry scales or both be raw")
    return l1, l2


def gather_group_weights(sym_buffer: SymmBuffer, l1_weights, l2_weights):
    """The weights of every expert of this rank's helper group, in group order (member m's
    experts at [m * EPR, (m + 1) * EPR)), collected from the members with broadcasts over the
    buffer's process group (reference: the chunked all_gather into rwk->ld.w1g / w2g,
    torch/mxmegakernel/mega/__init__.py:370-385).  Every rank of the group must call it; the
    result is what ``fp8_mega_moe(..., group_weights=...)`` takes.  Memory: group_ranks times this
    rank's own weights."""
    G, R = sym_buffer.group_ranks, sym_buffer.world_size
    if G <= 1:
        return None
    members = sym_buffer.group_members()
    scaled = isinstance(l1_weights, tuple)
    own = [t for w in (l1_weights, l2_weights) for t in (w if scaled else (w,))]
    parts = [[None] * G for _ in own]
    scratch = [torch.empty_like(t) for t in own]
    for r in range(R):
        mine = r in members
        for i, t in enumerate(own):
            buf = t if r == sym_buffer.rank else (torch.empty_like(t) if mine else scratch[i])
            dist.broadcast(buf, src=dist.get_global_rank(sym_buffer.group, r) if sym_buffer.group is not None else r,
                           group=sym_buffer.group)
            if mine:
                parts[i][members.index(r)] = buf
    cat = [torch.cat(p, dim=0).contiguous() for p in parts]
    return ((cat[0], cat[1]), (cat[2], cat[3])) if scaled else (cat[0], cat[1])


def _quantize_input(sym_buffer: "SymmBuffer", num_tokens: int, scaled: bool) -> None:
    """bf16xfp8 buffers: quantise `x` (bf16) into the region peers pull from, on the launch stream."""
    if sym_buffer.mma_type != "bf16xfp8" or num_tokens == 0:
        return
    check(_lib.lib().mxk_quantize_rows(sym_buffer.x.data_ptr(), int(num_tokens), sym_buffer.hidden,
                                       sym_buffer.x_fp8.data_ptr(),
                                       sym_buffer.x_sf.data_ptr() if scaled else None, _stream_ptr()),
          "mxk_quantize_rows")


def _check_buffer(sym_buffer: SymmBuffer, fn: str):
    # like the reference (torch/mxmegakernel/mega/__init__.py:615-618) the fp8 entry points take
    # both buffer kinds; a bf16xfp8 buffer gets its input quantised first
    if sym_buffer.mma_type not in _SUPPORTED_MMA_TYPES:
        raise ValueError(f"{fn} requires an fp8xfp8 / bf16xfp8 / fp8xfp4 SymmBuffer, got {sym_buffer.mma_type!r}")


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check_weights(sym_buffer: SymmBuffer, l1, l2, weight_format: int = 0):
    d1 = l1[0] if isinstance(l1, tuple) else l1
    d2 = l2[0] if isinstance(l2, tuple) else l2
    EPR, H, I = sym_buffer.num_experts_per_rank, sym_buffer.hidden, sym_buffer.intermediate_hidden
    if weight_format not in (0, 1):
        raise ValueError(f"weight_format must be 0 (E4M3) or 1 (packed e2m1), got {weight_format!r}")
    div = 2 if weight_format == 1 else 1     # bytes per row: k, or k / 2 for packed 4-bit codes
    if tuple(d1.shape) != (EPR, 2 * I, H // div) or tuple(d2.shape) != (EPR, H, I // div):
        raise ValueError(f"weights must be [{EPR},{2 * I},{H // div}] and [{EPR},{H},{I // div}], got {tuple(d1.shape)} "
                         f"and {tuple(d2.shape)}")
    if weight_format == 1 and (d1.data_ptr() % 32 or d2.data_ptr() % 32):
        raise ValueError("packed e2m1 weights must be 32-byte aligned (see transform_weights_for_mega_moe)")


def fp8_mega_moe(y: torch.Tensor, l1_weights, l2_weights, sym_buffer: SymmBuffer,
                 cumulative_local_expert_recv_stats=None, activation: str = "swiglu", activation_clamp=None,
                 expert_window: Optional[int] = None, max_spins: int = 0, cta_pair: Optional[int] = None,
                 packed_inputs: bool = False, group_weights=None, weight_format: int = 0) -> None:
    """One MoE layer: ``y[t] = sum_k w_k * W2_e SwiGLU(W1_e x_t)`` for this rank's
    ``y.shape[0]`` tokens, inputs taken from ``sym_buffer.x / x_sf / topk_idx / topk_weights``
    (or, with ``packed_inputs``, from the packed image described by ``SymmBuffer.packed_layout``).
    ``group_weights`` (from ``gather_group_weights``) on a buffer created with ``group_ranks`` > 1
    switches the cross-rank helper scheduling on: launches whose group load is skewed spread the
    group's (expert, window) units over its members.
    Every rank of the group must call it the same number of times (a rank with zero
    tokens still launches so that it joins the barrier and serves its experts)."""
    _check_buffer(sym_buffer, "fp8_mega_moe")
    if activation != "swiglu":
        raise ValueError(f"fp8xfp8 requires activation='swiglu', got {activation!r}")
    num_tokens = int(y.shape[0])
    if num_tokens > sym_buffer.num_max_tokens_per_rank:
        raise ValueError(f"num_tokens={num_tokens} exceeds capacity {sym_buffer.num_max_tokens_per_rank}")
    if y.dtype != torch.bfloat16 or (num_tokens and (y.shape[1] != sym_buffer.hidden or not y.is_contiguous())):
        raise ValueError("y must be a contiguous bf16 [tokens, hidden] tensor")
    _check_weights(sym_buffer, l1_weights, l2_weights, weight_format)
    lib = _lib.lib()
    _quantize_input(sym_buffer, num_tokens, isinstance(l1_weights, tuple) and l1_weights[1] is not None)
    a = sym_buffer.launch_args(num_tokens, l1_weights, l2_weights, y_bf16=y, expert_window=expert_window,
                               max_spins=max_spins, cta_pair=cta_pair, packed=packed_inputs, group_weights=group_weights,
                               weight_format=weight_format)
    if num_tokens == 0:  # nothing to reduce, but the rank still serves its experts
        check(lib.mxk_launch_compute(C.byref(a), _stream_ptr()), "mxk_launch_compute")
    else:
        check(lib.mxk_launch_full(C.byref(a), _stream_ptr()), "mxk_launch_full")
    sym_buffer.launch_count += 1


def fp8_mega_moe_compute(l1_weights, l2_weights, sym_buffer: SymmBuffer, num_tokens: int,
                         activation: str = "swiglu", activation_clamp=None,
                         expert_window: Optional[int] = None, max_spins: int = 0) -> None:
    """Compute segment only: prologue, dispatch, L1, L2 and combine push (no ``y``)."""
    _check_buffer(sym_buffer, "fp8_mega_moe_compute")
    num_tokens = int(num_tokens)
    if num_tokens < 0 or num_tokens > sym_buffer.num_max_tokens_per_rank:
        raise ValueError(f"num_tokens={num_tokens} exceeds capacity {sym_buffer.num_max_tokens_per_rank}")
    _check_weights(sym_buffer, l1_weights, l2_weights)
    _quantize_input(sym_buffer, num_tokens, isinstance(l1_weights, tuple) and l1_weights[1] is not None)
    a = sym_buffer.launch_args(num_tokens, l1_weights, l2_weights, expert_window=expert_window,
                               max_spins=max_spins)
    check(_lib.lib().mxk_launch_compute(C.byref(a), _stream_ptr()), "mxk_launch_compute")
    sym_buffer.launch_count += 1


def fp8_mega_moe_reduce(y: torch.Tensor, sym_buffer: SymmBuffer, num_tokens: Optional[int] = None,
                        max_spins: int = 0) -> None:
    """Reduce segment only; must follow ``fp8_mega_moe_compute`` on the same rank."""
    _check_buffer(sym_buffer, "fp8_mega_moe_reduce")
    nt = int(num_tokens) if num_tokens is not None else int(y.shape[0])
    if nt <= 0 or nt > sym_buffer.num_max_tokens_per_rank:
        raise ValueError(f"num_tokens={nt} out of range (capacity {sym_buffer.num_max_tokens_per_rank})")
    a = sym_buffer.launch_args(nt, y_bf16=y, max_spins=max_spins)
    check(_lib.lib().mxk_launch_reduce(C.byref(a), _stream_ptr()), "mxk_launch_reduce")


def bf16_mega_moe(*args, **kwargs):
    raise NotImplementedError("only fp8xfp8 and bf16xfp8 are implemented")


def bf16_fp8_mega_moe(y: torch.Tensor, l1_weights, l2_weights, sym_buffer: SymmBuffer, **kwargs) -> None:
    """bf16 activations + FP8 weights (reference: torch/mxmegakernel/mega/__init__.py:719-757): the
    caller fills ``sym_buffer.x`` (bf16); the rows are quantised on the device to E4M3 with 1x128
    UE8M0 scales (plain cast when the weights carry no scale planes) and peers pull the bytes."""
    if sym_buffer.mma_type != "bf16xfp8":
        raise ValueError(f"bf16_fp8_mega_moe requires a bf16xfp8 SymmBuffer, got {sym_buffer.mma_type!r}")
    fp8_mega_moe(y, l1_weights, l2_weights, sym_buffer, **kwargs)


def fp8_fp4_mega_moe(y: torch.Tensor, l1_weights, l2_weights, sym_buffer: SymmBuffer, **kwargs) -> None:
    """FP8 activations x 4-bit (e2m1) weights (reference: the MX_FP4_W build of the kernel,
    src/common.cuh:99-134; its Python layer leaves this entry point unimplemented).  The weights are
    packed codes ``[EPR, 2I, H/2]`` / ``[EPR, H, I/2]`` (``quant.per_block_cast_to_fp4``,
    ``transform_weights_for_mega_moe(..., weight_format="e2m1")``) with the usual 128x128 scale
    planes; everything else is ``fp8_mega_moe``.  The result equals the 8-bit layer run on the
    expanded weights (``quant.e2m1_to_e4m3``); the layer reads half the weight bytes."""
    fp8_mega_moe(y, l1_weights, l2_weights, sym_buffer, weight_format=1, **kwargs)


def read_dbg_report(sym_buffer: SymmBuffer, hidden: int = 0, intermediate_hidden: int = 0):
    st = sym_buffer.status()
    return {"status": st.status, "dbg": list(st.dbg), "launches": st.launches, "n_tasks": st.n_tasks,
            "n_windows": st.n_windows, "total_rows": st.total_rows}
