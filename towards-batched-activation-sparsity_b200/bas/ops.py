"""Torch-facing host layer over the C ABI: packed-weight cache, per-stream workspaces, launches.

torch is used for device memory and streams only.  Every function here launches libbas kernels on
``torch.cuda.current_stream()``; none synchronises, and after one warm-up call (which creates the
per-stream workspace and the packed weight) none allocates, so calls can be captured in a CUDA
graph the way the reference's benchmark captures its wrappers
(scripts/bench_perstep_actual_kernel_speedup.py:60-77).
"""

from __future__ import annotations

import weakref
from typing import Optional

import torch

from . import abi as _abi
from .abi import (BLOCK_K, GEMM_BF16, IDS_STABLE, X_STABLE, NEXT_INDEPENDENT, MAX_BATCH, SCORE_BF16, SCORE_INPUTS_STABLE, SCORE_ENERGY, SCORE_NORM, TP_HANDLE_BYTES,
                  check, lib)

_PACKED: dict[tuple, torch.Tensor] = {}
_PACK_STATS = {"hits": 0, "misses": 0}
_GEMM_WS: dict[tuple, torch.Tensor] = {}
_SELECT_WS: dict[tuple, torch.Tensor] = {}
_SELECT_OUT: dict[tuple, tuple] = {}


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _require_cuda_fp16(t: torch.Tensor, name: str) -> None:
    """CUDA tensor of one of the two 16-bit float types the kernels take (the reference's kernels
    accept both, kernels/shared_mask_batched_triton_min_runtime.py:21)."""
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (libbas has no CPU path)")
    if t.dtype not in (torch.float16, torch.bfloat16):
        raise TypeError(f"{name} must be float16 or bfloat16, got {t.dtype}")


def n_keep_from_density(density: float, nb: int, min_keep: int = 1) -> int:
    """The reference's rule: max(min_keep, min(nb, int(round(density * nb))))
    (scripts/bench_roundrobin_e2e_decode.py:102)."""
    return max(int(min_keep), min(int(nb), int(round(float(density) * int(nb)))))


# ---------------------------------------------------------------------------------------------
# packed weights
# ---------------------------------------------------------------------------------------------

def pack_weight(weight: torch.Tensor) -> torch.Tensor:
    """Repack an nn.Linear weight [N, K] into libbas's tile-major layout (uint8 tensor, opaque)."""
    _require_cuda_fp16(weight, "weight")
    if weight.dim() != 2 or weight.stride(1) != 1:
        raise ValueError("weight must be [N, K] with unit stride along K")
    n, k = weight.shape
    packed = torch.empty(lib.bas_packed_weight_bytes(n, k), dtype=torch.uint8, device=weight.device)
    with torch.cuda.device(weight.device):
        check(lib.bas_pack_weight(weight.data_ptr(), n, k, weight.stride(0), packed.data_ptr(), _stream_ptr()),
              "bas_pack_weight")
    return packed


def get_packed_weight(weight: torch.Tensor, block_k: int = BLOCK_K, cache_prefix: str = "gemm") -> torch.Tensor:
    """Cached :func:`pack_weight`, keyed like the reference's cache
    (kernels/shared_mask_batched_triton_min_runtime.py:3136-3146).  Unlike the reference's, an
    entry dies with its weight tensor, so a recycled address can never alias a stale pack."""
    if int(block_k) != BLOCK_K:
        raise ValueError(f"block_k must be {BLOCK_K}")
    key = (cache_prefix, weight.data_ptr(), str(weight.device), str(weight.dtype), tuple(weight.shape),
           tuple(weight.stride()), int(block_k))
    packed = _PACKED.get(key)
    if packed is not None:
        _PACK_STATS["hits"] += 1
        return packed
    _PACK_STATS["misses"] += 1
    packed = pack_weight(weight)
    _PACKED[key] = packed
    weakref.finalize(weight, _PACKED.pop, key, None)
    return packed


def clear_caches() -> None:
    _PACKED.clear()
    _GEMM_WS.clear()
    _SELECT_WS.clear()
    _SELECT_OUT.clear()


# ---------------------------------------------------------------------------------------------
# workspaces (one per device and stream; calls on one stream never overlap)
# ---------------------------------------------------------------------------------------------

def gemm_workspace(device: torch.device) -> torch.Tensor:
    key = (device.index, _stream_ptr())
    ws = _GEMM_WS.get(key)
    if ws is None:
        nbytes = lib.bas_gemm_workspace_bytes(MAX_BATCH, 1)
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        check(lib.bas_workspace_init(ws.data_ptr(), nbytes, _stream_ptr()), "bas_workspace_init")
        _GEMM_WS[key] = ws
    return ws


def select_workspace(device: torch.device, k: int) -> torch.Tensor:
    key = (device.index, _stream_ptr(), int(k))
    ws = _SELECT_WS.get(key)
    if ws is None:
        nbytes = lib.bas_select_workspace_bytes(int(k))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=device)
        check(lib.bas_workspace_init(ws.data_ptr(), nbytes, _stream_ptr()), "bas_workspace_init")
        _SELECT_WS[key] = ws
    return ws


def read_status(device: Optional[torch.device] = None) -> int:
    """Synchronously read and clear the status word of the current stream's workspace."""
    import ctypes

    device = device or torch.device("cuda", torch.cuda.current_device())
    ws = gemm_workspace(device)
    flags = ctypes.c_uint(0)
    check(lib.bas_read_device_status(ws.data_ptr(), ctypes.byref(flags), _stream_ptr()), "bas_read_device_status")
    return int(flags.value)


# ---------------------------------------------------------------------------------------------
# launches
# ---------------------------------------------------------------------------------------------

def gemm(x2d: torch.Tensor, packed: torch.Tensor, out2d: torch.Tensor, *, ids: Optional[torch.Tensor] = None,
         count: Optional[torch.Tensor] = None, k_host: Optional[int] = None,
         bitmap: Optional[torch.Tensor] = None, family: int = 0, ids_stable: bool = False,
         x_stable: bool = False, next_independent: bool = False, cluster: int = 0, pairs: int = 0, tp=None, max_ctas: int = 0) -> None:
    """out2d[B, N] = x2d[B, K] restricted to the active blocks, times W^T.

    ``ids`` int32 device list (``count``: optional int32[1] device-side length, ``k_host`` an upper
    bound) or ``bitmap`` uint8[K/64] (``k_host`` then optionally tells how many blocks to expect).  ``family``: 0 by batch size, 1 CUDA-core, 2 tcgen05.
    ``ids_stable``: promise that ``ids`` is not written by the kernel launched just before this
    call on the stream; the kernel then streams weights while that kernel is still finishing.
    ``x_stable`` (with ``ids_stable``): the same promise for ``x2d`` - it was complete before the kernel
    launched just before this call started (a resident input, or the x that call already read); the
    kernel then waits for its predecessor only before it stores ``out2d``.
    ``next_independent`` (with both promises): a hint that the call after this one will be launched
    with ``x_stable`` too (a chain of independent calls); wide outputs then take an even smaller grid.
    ``cluster``: 0 lets the library choose; 1, 2 or 4 forces the tcgen05 kernel's cluster size.
    ``pairs``: 0 lets the library choose; 2, 3 or 4 forces its number of copy/MMA warp pairs.
    ``max_ctas``: 0 lets the library choose; else an upper bound (up to 255) on the kernel's CTAs.
    x, out (and the weight that was packed) are all float16 or all bfloat16.
    ``tp``: an :class:`ExchangeGroup`; x and packed are then this rank's K-shard and out receives
    the sum over the group's ranks, formed inside the kernel (every rank must make the same call).
    Batches above 64 rows are run in slices of 64."""
    _require_cuda_fp16(x2d, "x")
    _require_cuda_fp16(out2d, "out")
    if x2d.dtype != out2d.dtype:
        raise TypeError("x and out must have the same dtype (the packed weight must hold that type too)")
    bf16 = GEMM_BF16 if x2d.dtype == torch.bfloat16 else 0
    if x2d.dim() != 2 or out2d.dim() != 2 or x2d.stride(1) != 1 or out2d.stride(1) != 1:
        raise ValueError("x and out must be 2-D with unit inner stride")
    bt, k = x2d.shape
    n = out2d.shape[1]
    if out2d.shape[0] != bt:
        raise ValueError("x and out disagree on the batch")
    if bitmap is None:
        if ids is None:
            raise ValueError("either ids or bitmap is required")
        if ids.dtype != torch.int32 or not ids.is_contiguous():
            raise TypeError("ids must be a contiguous int32 tensor")
        if k_host is None:
            k_host = int(ids.numel())
    else:
        if bitmap.dtype != torch.uint8 or not bitmap.is_contiguous():
            raise TypeError("bitmap must be a contiguous uint8 tensor")
        k_host = int(k_host) if k_host is not None else 0      # with a byte map: a hint, 0 = unknown
    if x2d.data_ptr() % 16 or x2d.stride(0) % 8 or k % 8:
        raise ValueError("x rows must be 16-byte aligned and K a multiple of 8")
    with torch.cuda.device(x2d.device):
        ws = gemm_workspace(x2d.device)
        stream = _stream_ptr()
        for b0 in range(0, bt, MAX_BATCH):
            bsz = min(MAX_BATCH, bt - b0)
            xs, ys = x2d[b0:b0 + bsz], out2d[b0:b0 + bsz]
            fn = lib.bas_gemm_ex if tp is None else (lambda *a: lib.bas_gemm_allreduce(tp.handle, *a))
            check(fn(
                xs.data_ptr(), xs.stride(0), packed.data_ptr(),
                ids.data_ptr() if ids is not None and bitmap is None else None,
                count.data_ptr() if count is not None else None, int(k_host),
                bitmap.data_ptr() if bitmap is not None else None,
                bsz, k, n, ys.data_ptr(), ys.stride(0), ws.data_ptr(), ws.numel(),
                int(family) | (IDS_STABLE if ids_stable else 0) | (X_STABLE if ids_stable and x_stable else 0) | (NEXT_INDEPENDENT if next_independent else 0) | bf16 | (int(cluster) << 8) | (int(pairs) << 12) | (int(max_ctas) << 16), stream),
                "bas_gemm")


class GemmList:
    """A fixed sequence of :func:`gemm` calls run as ONE persistent kernel (``bas_list_*``): the
    decode step's chain of linears (the reference runs 224 patched forwards per token,
    scripts/bench_roundrobin_e2e_decode.py:331-503) without a kernel boundary between them.

    ``calls``: dicts with ``x`` [B, K], ``packed``, ``out`` [B, N], one of ``ids`` / ``bitmap``
    (``count``, ``k_host`` as for :func:`gemm`) and ``depends_on``: index of the earlier call that
    must be complete before ``x`` is read (normally the call that writes it), or -1.  Masks must be
    complete before :meth:`run`; they may change between runs.

    Selection inside the launch: an entry ``{"select": x, "n_keep": n, "score_kind": SCORE_NORM,
    "depends_on": d}`` scores the blocks of ``x`` as :func:`select_topk` does (same bits) once call ``d``
    is complete; a call with ``"mask_from": index_of_that_entry`` instead of ``ids`` / ``bitmap`` then runs
    with the top-``n`` blocks (``"mask_block0"``: the block of the mask that is its block 0, for a K-shard;
    ``"ids_out"``: an int32 tensor that receives the kept ids of the whole mask, ascending).  Indices in
    ``depends_on`` / ``mask_from`` count entries of both kinds.  With ``tp``, an entry may be given
    ``"sharded": (first_block, blocks_of_the_whole_input)``: its ``x`` is this rank's K-shard, the ranks exchange
    their block scores inside the launch and ``n_keep`` blocks of the WHOLE input are kept; the row-parallel
    calls over that shard then run with their part of the mask (``mask_block0 = first_block``).

    Output-block sparsity and compact operands (the reference's 2-D kernels): ``"n_ids"``, an int32 tensor of
    64-column output blocks, makes a call compute only those blocks - into their own columns of ``out``
    (the others are left alone) or, with ``"out_compact": True``, side by side into an ``out`` that is
    ``len(n_ids) * 64`` wide (``"n"``: the real output width, needed then).  ``"x_compact": True``: ``x`` holds
    only the active input blocks, in the order of ``ids`` (``"k"``: the weight's K, needed then).  All tensors
    are kept alive by the list.  :meth:`run` launches on the current stream, allocates nothing and can be captured in a
    CUDA graph; runs of one list must not overlap."""

    def __init__(self, calls, *, cluster: int = 0, pairs: int = 0, max_ctas: int = 0, min_units: int = 0, tp=None):
        """``tp``: an :class:`ExchangeGroup`; calls with ``row_parallel=True`` then hold this rank's K-shard
        and their outputs are summed over the group's ranks inside the kernel (every rank builds and runs
        the same list; such a call must depend on the row-parallel call before it)."""
        import ctypes

        calls = list(calls)
        if not calls:
            raise ValueError("a list needs at least one call")
        arr = (_abi.ListCall * len(calls))()
        self._keep = []
        first = calls[0]["select"] if "select" in calls[0] else calls[0]["x"]
        dtype = first.dtype
        self.device = first.device
        for i, c in enumerate(calls):
            a = arr[i]
            if "select" in c:
                x = c["select"]
                _require_cuda_fp16(x, "select")
                if x.dtype != dtype or x.dim() != 2 or x.stride(1) != 1:
                    raise ValueError("a selection entry's x must be 2-D with unit inner stride and the list's dtype")
                a.op, a.x_dev, a.ldx = _abi.LIST_SELECT, x.data_ptr(), x.stride(0)
                a.batch, a.k, a.k_host = x.shape[0], x.shape[1], int(c["n_keep"])
                a.score_kind = int(c.get("score_kind", _abi.SCORE_NORM))
                a.depends_on = int(c.get("depends_on", -1))
                if c.get("sharded") is not None:          # (first block of this rank's shard, blocks of the whole input)
                    a.mask_block0, a.n_host = (int(v) for v in c["sharded"])
                    a.shape_flags = _abi.LIST_SELECT_SHARDED
                self._keep.append((x,))
                continue
            x, out, packed = c["x"], c["out"], c["packed"]
            _require_cuda_fp16(x, "x")
            _require_cuda_fp16(out, "out")
            if x.dtype != dtype or out.dtype != dtype:
                raise TypeError("all x and out of a list must have one dtype")
            n_ids = c.get("n_ids")
            if n_ids is not None and (n_ids.dtype != torch.int32 or not n_ids.is_contiguous() or n_ids.numel() == 0):
                raise TypeError("n_ids must be a contiguous, non-empty int32 tensor")
            if x.dim() != 2 or out.dim() != 2 or x.stride(1) != 1 or out.stride(1) != 1 or x.shape[0] != out.shape[0]:
                raise ValueError("x and out must be 2-D with unit inner stride and the same batch")
            if x.shape[0] > MAX_BATCH:
                raise ValueError(f"a call of a list takes at most {MAX_BATCH} rows")
            ids, bitmap, count = c.get("ids"), c.get("bitmap"), c.get("count")
            k_host = c.get("k_host")
            mask_from, ids_out = c.get("mask_from"), c.get("ids_out")
            if mask_from is not None:
                if ids is not None or bitmap is not None or count is not None:
                    raise ValueError("a call with mask_from takes no ids, bitmap or count")
                if ids_out is not None and (ids_out.dtype != torch.int32 or not ids_out.is_contiguous()):
                    raise TypeError("ids_out must be a contiguous int32 tensor")
                k_host = 0
            elif bitmap is None:
                if ids is None:
                    raise ValueError("either ids or bitmap is required")
                if ids.dtype != torch.int32 or not ids.is_contiguous():
                    raise TypeError("ids must be a contiguous int32 tensor")
                k_host = int(ids.numel()) if k_host is None else int(k_host)
            else:
                if bitmap.dtype != torch.uint8 or not bitmap.is_contiguous():
                    raise TypeError("bitmap must be a contiguous uint8 tensor")
                k_host = int(k_host) if k_host is not None else 0
            a.x_dev, a.ldx, a.packed_dev = x.data_ptr(), x.stride(0), packed.data_ptr()
            a.ids_dev = ids.data_ptr() if ids is not None and bitmap is None and ids.numel() else None
            a.count_dev = count.data_ptr() if count is not None else None
            a.bitmap_dev = bitmap.data_ptr() if bitmap is not None else None
            a.y_dev, a.ldy = out.data_ptr(), out.stride(0)
            a.k_host, a.batch, a.k, a.n = k_host, x.shape[0], int(c.get("k", x.shape[1])), int(c.get("n", out.shape[1]))
            if n_ids is not None:
                a.n_ids_dev, a.n_host = n_ids.data_ptr(), int(n_ids.numel())
            a.shape_flags = (_abi.LIST_OUT_COMPACT if c.get("out_compact") else 0) | (_abi.LIST_X_COMPACT if c.get("x_compact") else 0)
            if c.get("x_compact") and x.shape[1] < k_host * BLOCK_K:
                raise ValueError("a compact x holds one 64-channel block per id")
            if c.get("out_compact") and n_ids is not None and out.shape[1] < n_ids.numel() * 64:
                raise ValueError("a compact out holds one 64-column block per entry of n_ids")
            a.depends_on = int(c.get("depends_on", -1))
            a.row_parallel = 1 if c.get("row_parallel") else 0
            if mask_from is not None:
                a.mask_entry, a.mask_block0 = int(mask_from) + 1, int(c.get("mask_block0", 0))
                a.ids_out_dev = ids_out.data_ptr() if ids_out is not None else None
            self._keep.append((x, out, packed, ids, bitmap, count, ids_out, n_ids))
        self.n_calls = len(calls)
        self.handle = ctypes.c_void_p()
        flags = (GEMM_BF16 if dtype == torch.bfloat16 else 0) | (int(cluster) << 8) | (int(pairs) << 12) | (int(max_ctas) << 16) | (int(min_units) << 24)
        self.tp = tp
        with torch.cuda.device(self.device):
            if tp is not None:
                check(lib.bas_list_create_tp(ctypes.byref(self.handle), arr, len(calls), flags, tp.handle), "bas_list_create_tp")
            else:
                check(lib.bas_list_create(ctypes.byref(self.handle), arr, len(calls), flags), "bas_list_create")

    def run(self) -> None:
        with torch.cuda.device(self.device):
            check(lib.bas_list_run(self.handle, _stream_ptr()), "bas_list_run")

    def read_status(self) -> int:
        """Synchronously read and clear the list's device status word."""
        import ctypes

        flags = ctypes.c_uint(0)
        with torch.cuda.device(self.device):
            check(lib.bas_list_read_status(self.handle, ctypes.byref(flags), _stream_ptr()), "bas_list_read_status")
        return int(flags.value)

    def reset(self) -> None:
        """After a run that reported an expired wait: synchronise and zero the completion counters."""
        with torch.cuda.device(self.device):
            check(lib.bas_list_reset(self.handle), "bas_list_reset")

    def set_wait(self, wait_ms: float, never_ready_call: int = -1) -> None:
        """Bound of the kernel's waits; ``never_ready_call`` (tests of the expiry path) names a call
        whose dependency is never seen complete."""
        check(lib.bas_list_set_wait(self.handle, float(wait_ms), int(never_ready_call)), "bas_list_set_wait")

    def info(self) -> dict:
        import ctypes

        v = [ctypes.c_int(0) for _ in range(4)]
        check(lib.bas_list_info(self.handle, *[ctypes.byref(t) for t in v]), "bas_list_info")
        return dict(zip(("ctas", "cluster", "slots", "pairs"), (int(t.value) for t in v)))

    def close(self) -> None:
        if self.handle:
            with torch.cuda.device(self.device):
                torch.cuda.synchronize()
                lib.bas_list_destroy(self.handle)
            self.handle = None
            self._keep = []

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class ExchangeGroup:
    """This rank's exchange area for row-parallel contractions summed inside the kernel, connected
    to the areas of the other ranks of ``group`` (one process per GPU, all on one box).  The handles
    travel through ``torch.distributed``; construction is collective and ends with a barrier."""

    def __init__(self, device, max_batch: int, n: int, group=None):
        import ctypes

        import torch.distributed as dist

        self.device = torch.device(device)
        multi = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.group = group
        self.world = dist.get_world_size(group) if multi else 1
        self.rank = dist.get_rank(group) if multi else 0
        self.handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            check(lib.bas_tp_create(ctypes.byref(self.handle), self.rank, self.world, int(max_batch), int(n)),
                  "bas_tp_create")
            mine = (ctypes.c_ubyte * TP_HANDLE_BYTES)()
            check(lib.bas_tp_handle(self.handle, mine), "bas_tp_handle")
            if multi:
                local = torch.tensor(list(mine), dtype=torch.uint8, device=self.device)
                gathered = [torch.empty_like(local) for _ in range(self.world)]
                dist.all_gather(gathered, local, group=group)
                blob = bytes(torch.cat(gathered).cpu().tolist())
            else:
                blob = bytes(mine)
            buf = (ctypes.c_ubyte * len(blob)).from_buffer_copy(blob)
            check(lib.bas_tp_connect(self.handle, buf), "bas_tp_connect")
            if multi:
                dist.barrier(group=group)      # nobody publishes into an area that is not mapped yet

    def close(self) -> None:
        """Collective: every rank unmaps its peers, all meet, then each frees its own area."""
        import torch.distributed as dist

        if not self.handle:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            if self.world > 1:
                dist.barrier(group=self.group)
            lib.bas_tp_disconnect(self.handle)
            if self.world > 1:
                dist.barrier(group=self.group)
            lib.bas_tp_destroy(self.handle)
        self.handle = None

    def __del__(self):
        # not collective: a group that was never closed is left to process exit when it has peers
        try:
            if self.handle and self.world == 1:
                self.close()
        except Exception:
            pass


def build_bitmap(ids: torch.Tensor, nb: int, device=None, count: Optional[torch.Tensor] = None) -> torch.Tensor:
    """uint8[nb] with 1 at the active ids; one kernel, no host synchronisation."""
    device = torch.device(device) if device is not None else ids.device
    if device.type != "cuda":
        raise ValueError("bitmap must live on a CUDA device (libbas has no CPU path)")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    ids = ids.to(device=device, dtype=torch.int32).contiguous()
    bm = torch.empty(int(nb), dtype=torch.uint8, device=device)
    with torch.cuda.device(device):
        check(lib.bas_build_bitmap(ids.data_ptr() if ids.numel() else None,
                                   count.data_ptr() if count is not None else None,
                                   int(ids.numel()), int(nb), bm.data_ptr(), _stream_ptr()), "bas_build_bitmap")
    return bm


def _select_buffers(device: torch.device, nb: int):
    key = (device.index, _stream_ptr(), nb)
    bufs = _SELECT_OUT.get(key)
    if bufs is None:
        bufs = (torch.empty(nb, dtype=torch.int32, device=device),
                torch.empty(1, dtype=torch.int32, device=device))
        _SELECT_OUT[key] = bufs
    return bufs


_LISTS_2D: "dict[tuple, GemmList]" = {}
_LISTS_2D_MAX = 32


def gemm_2d(x2d: torch.Tensor, packed: torch.Tensor, out2d: torch.Tensor, *, ids: torch.Tensor,
            n_ids: Optional[torch.Tensor] = None, out_compact: bool = False, x_compact: bool = False,
            k: Optional[int] = None, n: Optional[int] = None) -> None:
    """One masked contraction with output-block sparsity and / or compact operands (the reference's 2-D wrappers,
    kernels/shared_mask_batched_triton_min_runtime.py:3411-3467, 3498-3850): the arguments of a
    :class:`GemmList` call.  It runs as a list launch of one call; the list is kept (the 32 most recent argument
    sets, by addresses and shapes, tensors included), so that a caller who passes the same buffers again - a
    benchmark loop, a decode step with persistent buffers - pays for its creation once."""
    key = (x2d.data_ptr(), tuple(x2d.shape), x2d.stride(0), packed.data_ptr(), out2d.data_ptr(), tuple(out2d.shape),
           out2d.stride(0), ids.data_ptr(), int(ids.numel()), None if n_ids is None else (n_ids.data_ptr(), int(n_ids.numel())),
           bool(out_compact), bool(x_compact), k, n, x2d.dtype, str(x2d.device))
    lst = _LISTS_2D.pop(key, None)
    if lst is None:
        call = {"x": x2d, "packed": packed, "out": out2d, "ids": ids, "out_compact": out_compact, "x_compact": x_compact}
        if n_ids is not None:
            call["n_ids"] = n_ids
        if k is not None:
            call["k"] = int(k)
        if n is not None:
            call["n"] = int(n)
        lst = GemmList([call])
        while len(_LISTS_2D) >= _LISTS_2D_MAX:
            _LISTS_2D.pop(next(iter(_LISTS_2D))).close()
    _LISTS_2D[key] = lst          # most recent last
    lst.run()


def select_topk(x2d: torch.Tensor, n_keep: int, score_kind: int = SCORE_NORM, *,
                ids_out: Optional[torch.Tensor] = None, count_out: Optional[torch.Tensor] = None,
                bitmap_out: Optional[torch.Tensor] = None, scores_out: Optional[torch.Tensor] = None,
                chan_scale: Optional[torch.Tensor] = None, block_mult: Optional[torch.Tensor] = None,
                inputs_stable: bool = False):
    """Device-side batch-shared top-k selection.  Returns (ids[:n_keep] int32 ascending, count int32[1]);
    both stay on the device.  Without explicit outputs, per-stream buffers are reused.

    ``chan_scale`` (float32 [>= 64 * (K // 64)]) and ``block_mult`` (float32 [K // 64]) are the
    reference's optional score modifiers (scripts/bench_roundrobin_e2e_decode.py:104-112): weighted
    squares per channel, and a factor per block (see :func:`prior_multiplier`).

    ``inputs_stable``: promise that no kernel still running when this call starts writes ``x2d`` or
    touches the outputs (pass explicit ``ids_out`` / ``count_out`` that alternate between steps) or
    the selection workspace; the scoring then overlaps the kernel launched before this call."""
    return _select(x2d, 0, int(n_keep), int(score_kind) | (SCORE_INPUTS_STABLE if inputs_stable else 0), 0.0,
                   ids_out, count_out, bitmap_out, scores_out, chan_scale, block_mult)


def prior_multiplier(block_prior: torch.Tensor, prior_alpha: float = 1.0, prior_eps: float = 0.1) -> torch.Tensor:
    """float32 ``clamp(prior + eps, min=1e-6) ** alpha``, the factor the reference applies to the block
    scores (scripts/bench_roundrobin_e2e_decode.py:109-112).  A prior is fixed per projection:
    evaluate this once and pass the result as ``block_mult``."""
    p = block_prior.to(dtype=torch.float32)
    return torch.clamp(p + float(prior_eps), min=1e-6).pow(float(prior_alpha)).contiguous()


def select_budget(x2d: torch.Tensor, energy_keep: float, min_keep: int = 1, *,
                  ids_out: Optional[torch.Tensor] = None, count_out: Optional[torch.Tensor] = None,
                  bitmap_out: Optional[torch.Tensor] = None, scores_out: Optional[torch.Tensor] = None,
                  full_above: Optional[int] = None):
    """Device-side energy-budget selection (variable count).  Returns (ids buffer [nb], count int32[1]);
    only the first ``count`` ids are meaningful, and reading ``count`` on the host synchronises.
    ``full_above``: a budget that keeps more blocks than this keeps them all (the reference's dense
    fallback, scripts/bench_alpaca_energy_budget_e2e.py:104-109, decided on the device)."""
    return _select(x2d, 1, int(min_keep), SCORE_ENERGY, float(energy_keep), ids_out, count_out, bitmap_out, scores_out,
                   full_above=full_above)


def _select(x2d, mode, n_keep, score_kind, energy_keep, ids_out, count_out, bitmap_out, scores_out,
            chan_scale=None, block_mult=None, full_above=None):
    _require_cuda_fp16(x2d, "x")
    for name, t, need in (("chan_scale", chan_scale, (x2d.shape[1] // BLOCK_K) * BLOCK_K),
                          ("block_mult", block_mult, x2d.shape[1] // BLOCK_K)):
        if t is None:
            continue
        if mode != 0:
            raise ValueError(f"{name} applies to the top-k selection only")
        if not t.is_cuda or t.device != x2d.device or t.dtype != torch.float32 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous float32 tensor on x's device")
        if t.numel() < need:
            raise ValueError(f"{name} needs at least {need} elements")
    if x2d.dim() != 2 or x2d.stride(1) != 1:
        raise ValueError("x must be 2-D with unit inner stride")
    bt, k = x2d.shape
    nb = k // BLOCK_K
    if nb < 1:
        raise ValueError("K must be at least 64")
    if ids_out is None or count_out is None:
        ids_buf, cnt_buf = _select_buffers(x2d.device, nb)
        ids_out = ids_out if ids_out is not None else ids_buf
        count_out = count_out if count_out is not None else cnt_buf
    if scores_out is not None and scores_out.dtype != torch.float64:
        raise TypeError("scores_out must be float64")
    with torch.cuda.device(x2d.device):
        ws = select_workspace(x2d.device, k)
        args = (ids_out.data_ptr(), count_out.data_ptr(),
                bitmap_out.data_ptr() if bitmap_out is not None else None,
                scores_out.data_ptr() if scores_out is not None else None,
                ws.data_ptr(), ws.numel(), _stream_ptr())
        bf16 = SCORE_BF16 if x2d.dtype == torch.bfloat16 else 0
        if mode == 0 and (chan_scale is not None or block_mult is not None):
            check(lib.bas_select_topk_weighted(x2d.data_ptr(), x2d.stride(0), bt, k, n_keep, int(score_kind) | bf16,
                                               chan_scale.data_ptr() if chan_scale is not None else None,
                                               block_mult.data_ptr() if block_mult is not None else None, *args),
                  "bas_select_topk_weighted")
            return ids_out[:n_keep], count_out
        if mode == 0:
            check(lib.bas_select_topk(x2d.data_ptr(), x2d.stride(0), bt, k, n_keep, int(score_kind) | bf16, *args),
                  "bas_select_topk")
            return ids_out[:n_keep], count_out
        if full_above is not None:
            check(lib.bas_select_budget_capped(x2d.data_ptr(), x2d.stride(0), bt, k, energy_keep, n_keep, int(full_above),
                                               bf16, *args), "bas_select_budget_capped")
            return ids_out, count_out
        check(lib.bas_select_budget_ex(x2d.data_ptr(), x2d.stride(0), bt, k, energy_keep, n_keep, bf16, *args),
              "bas_select_budget_ex")
        return ids_out, count_out


def select_gemm(x2d: torch.Tensor, packed: torch.Tensor, out2d: torch.Tensor, n_keep: int,
                score_kind: int = SCORE_NORM, *, energy_keep: Optional[float] = None,
                ids_out: Optional[torch.Tensor] = None, count_out: Optional[torch.Tensor] = None,
                bitmap_out: Optional[torch.Tensor] = None, scores_out: Optional[torch.Tensor] = None,
                cluster: int = 0, max_ctas: int = 0):
    """Batch-shared mask selection and the masked contraction in one call (one launch where the
    contraction runs in clusters, else the two-launch chain; same ids and sums).  ``energy_keep``
    switches from top-k of ``n_keep`` to the energy budget with at least ``n_keep`` blocks.
    Returns (ids buffer, count int32[1]); the first ``count`` ids are the kept blocks, ascending."""
    _require_cuda_fp16(x2d, "x")
    _require_cuda_fp16(out2d, "out")
    if x2d.dtype != out2d.dtype:
        raise TypeError("x and out must have the same dtype")
    if x2d.dim() != 2 or out2d.dim() != 2 or x2d.stride(1) != 1 or out2d.stride(1) != 1:
        raise ValueError("x and out must be 2-D with unit inner stride")
    bt, k = x2d.shape
    n = out2d.shape[1]
    if bt > MAX_BATCH or out2d.shape[0] != bt:
        raise ValueError(f"batch must agree and be at most {MAX_BATCH}")
    nb = k // BLOCK_K
    if nb < 1:
        raise ValueError("K must be at least 64")
    if ids_out is None or count_out is None:
        ids_buf, cnt_buf = _select_buffers(x2d.device, nb)
        ids_out = ids_out if ids_out is not None else ids_buf
        count_out = count_out if count_out is not None else cnt_buf
    if scores_out is not None and scores_out.dtype != torch.float64:
        raise TypeError("scores_out must be float64")
    bf16 = x2d.dtype == torch.bfloat16
    with torch.cuda.device(x2d.device):
        gws, sws = gemm_workspace(x2d.device), select_workspace(x2d.device, k)
        check(lib.bas_select_gemm(
            x2d.data_ptr(), x2d.stride(0), packed.data_ptr(), bt, k, n, int(n_keep),
            int(score_kind) | (SCORE_BF16 if bf16 else 0), float(energy_keep) if energy_keep is not None else -1.0,
            out2d.data_ptr(), out2d.stride(0), ids_out.data_ptr(), count_out.data_ptr(),
            bitmap_out.data_ptr() if bitmap_out is not None else None,
            scores_out.data_ptr() if scores_out is not None else None,
            gws.data_ptr(), gws.numel(), sws.data_ptr(), sws.numel(),
            (GEMM_BF16 if bf16 else 0) | (int(cluster) << 8) | (int(max_ctas) << 16), _stream_ptr()), "bas_select_gemm")
    return ids_out, count_out


def sparse_linear(x: torch.Tensor, weight: torch.Tensor, density: float, *, score_kind: int = SCORE_NORM,
                  cache_prefix: str = "sparse_linear", out: Optional[torch.Tensor] = None,
                  fixed_active_blocks: Optional[torch.Tensor] = None, energy_keep: Optional[float] = None,
                  min_keep: int = 1, block_mult: Optional[torch.Tensor] = None,
                  block_score_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The decode-time operator of the reference's ``_sparse_linear``
    (scripts/bench_roundrobin_e2e_decode.py:179-284) through :func:`select_gemm`: selection and
    contraction in one launch where the shape allows, else chained, never a host round trip.  x is [B, K] or [B, 1, K].

    * More than one position per sequence (prefill) or ``density >= 1`` runs the dense
      ``F.linear``, as the reference does (:200-201).
    * ``fixed_active_blocks``: skip the selection and use these ids (mask reuse, :209-210).
    * ``energy_keep``: keep the shortest descending-energy prefix of blocks that reaches this
      fraction of the total energy, at least ``min_keep`` blocks - the variable-count mode of
      scripts/bench_alpaca_energy_budget_e2e.py:49-56, without its host synchronisation: the count
      stays on the device and the contraction reads it there.
    * ``block_score_scale`` / ``block_mult``: the reference's channel weights and block prior
      (:104-112; ``block_mult = prior_multiplier(prior, alpha, eps)``, and like the reference a
      factor whose length is not the block count is ignored); top-k mode only, two launches.
    """
    x3 = x.reshape(x.shape[0], 1, x.shape[1]) if x.dim() == 2 else x
    if x3.shape[1] != 1 or (energy_keep is None and fixed_active_blocks is None and float(density) >= 1.0):
        return torch.nn.functional.linear(x, weight)
    bt, k = x3.shape[0], x3.shape[2]
    n = weight.shape[0]
    x2d = x3.reshape(bt, k)
    packed = get_packed_weight(weight, BLOCK_K, cache_prefix)
    if out is None:
        out = torch.empty(bt, 1, n, device=x.device, dtype=x.dtype)
    out2d = out.view(bt, n)
    nb = k // BLOCK_K
    if block_mult is not None and block_mult.numel() != nb:
        block_mult = None
    weighted = energy_keep is None and (block_mult is not None or block_score_scale is not None)
    if fixed_active_blocks is not None:
        ids = fixed_active_blocks.to(device=x.device, dtype=torch.int32).contiguous()
        gemm(x2d, packed, out2d, ids=ids)
    elif weighted:
        n_keep = n_keep_from_density(density, nb, min_keep)
        ids, count = select_topk(x2d, n_keep, score_kind, chan_scale=block_score_scale, block_mult=block_mult)
        gemm(x2d, packed, out2d, ids=ids, count=count, k_host=n_keep)
    elif bt > MAX_BATCH:
        if energy_keep is not None:
            ids, count = select_budget(x2d, float(energy_keep), int(min_keep))
            gemm(x2d, packed, out2d, ids=ids, count=count, k_host=nb)
        else:
            n_keep = n_keep_from_density(density, nb, min_keep)
            ids, count = select_topk(x2d, n_keep, score_kind)
            gemm(x2d, packed, out2d, ids=ids, count=count, k_host=n_keep)
    elif energy_keep is not None:
        select_gemm(x2d, packed, out2d, int(min_keep), SCORE_ENERGY, energy_keep=float(energy_keep))
    else:
        select_gemm(x2d, packed, out2d, n_keep_from_density(density, nb, min_keep), score_kind)
    return out.reshape(bt, n) if x.dim() == 2 else out
