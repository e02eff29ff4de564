"""Drop-in for the reference module ``kernels/shared_mask_batched_triton_min_runtime.py``.

Same names, argument meaning and error behaviour as the reference's host wrappers, so that
``scripts/bench_perstep_actual_kernel_speedup.py``, ``scripts/profile_kernel_configs.py`` and the
end-to-end decode scripts run against it unchanged; the work is done by libbas (hand-written
sm_100a CUDA) instead of Triton kernels.  Differences a caller can observe:

* ``num_split_k`` and the ``tile_*`` arguments are accepted and ignored: the split of the active
  blocks over the GPU is chosen inside the library (column ranges per CTA or per cluster), and
  the result does not depend on it beyond fp32 rounding.
* The tensor returned by ``_get_prepacked_weight_block_major`` is an opaque uint8 buffer in
  libbas's tile-major layout, not the reference's ``[K/64, 64, N]`` view.  No caller reads it.
* float16 or bfloat16 (x, weight and out alike).  There is no CPU path: CPU tensors raise
  ``ValueError``.
* The 2-D wrappers (output blocks, compact output, compact input) take the output width from the
  weight.  The reference's compact wrapper lets its kernel take it from the compact tensor, which masks
  the output blocks that lie past that width (zeros); here they hold the products.
"""

from __future__ import annotations

from types import SimpleNamespace
from typing import Optional

import torch

from bas import ops as _ops
from bas.abi import BLOCK_K as _BLOCK_K

# kernels/shared_mask_batched_triton_min_runtime.py:17 — the reference reads an environment
# override; the block size of this implementation is fixed.
INDEX_BLOCK_META_SIZE = _BLOCK_K

# The tuner (scripts/profile_kernel_configs.py:70-83, 135-146) enumerates tile configurations and
# reads ``.best_config`` of the autotuned bitmap kernel.  There is one configuration here.
_PREPACK_AUTOTUNE_CONFIGS = [SimpleNamespace(kwargs={"BLOCK_B": 16, "BLOCK_N": 128}, num_warps=4, num_stages=3)]
prepacked_block_sparse_gemm_bitmap_preload_batched_kernel = SimpleNamespace(best_config=_PREPACK_AUTOTUNE_CONFIGS[0])


def _build_active_k_bitmap(active_blocks: torch.Tensor, total_k_blocks: int, device) -> torch.Tensor:
    """uint8 [total_k_blocks], 1 at the active ids (reference :1056-1061)."""
    return _ops.build_bitmap(active_blocks, int(total_k_blocks), device)


def _get_prepacked_weight_block_major(weight: torch.Tensor, block_k: int, cache_prefix: str = "gemm") -> torch.Tensor:
    """Warm (or hit) the packed-weight cache (reference :3133-3163)."""
    return _ops.get_packed_weight(weight, int(block_k), cache_prefix)


def _views(x: torch.Tensor, out: torch.Tensor):
    bsz, seqlen, m_dim = x.shape
    n_dim = out.shape[-1]
    bt = bsz * seqlen
    x2d = x.view(bt, m_dim)
    y2d = out.view(bt, n_dim)
    if not x2d.is_contiguous():
        x2d = x2d.contiguous()
    if y2d.stride(-1) != 1:
        raise ValueError("out must have unit stride along its last dimension")
    return x2d, y2d


def _ids32(active_blocks: torch.Tensor) -> torch.Tensor:
    if active_blocks.dtype != torch.int32:
        active_blocks = active_blocks.to(dtype=torch.int32)
    if not active_blocks.is_contiguous():
        active_blocks = active_blocks.contiguous()
    return active_blocks


def _prepacked_block_sparse_gemm_from_active_blocks_splitk(
    x: torch.Tensor,
    weight: torch.Tensor,
    active_blocks: torch.Tensor,
    out: torch.Tensor,
    cache_prefix: str = "gemm_1d_sk",
    num_split_k: Optional[int] = None,
    tile_b: Optional[int] = None,
    tile_n: Optional[int] = None,
    tile_warps: Optional[int] = None,
    tile_stages: Optional[int] = None,
) -> None:
    """Index-list family (reference :1350-1454): out = x[:, active blocks] . W[:, active blocks]^T."""
    if int(active_blocks.numel()) <= 0:
        out.zero_()
        return
    packed = _ops.get_packed_weight(weight, _BLOCK_K, cache_prefix)
    x2d, y2d = _views(x, out)
    _ops.gemm(x2d, packed, y2d, ids=_ids32(active_blocks))


def _prepacked_block_sparse_gemm_from_active_blocks_bitmap_preload(
    x: torch.Tensor,
    weight: torch.Tensor,
    active_blocks: torch.Tensor,
    out: torch.Tensor,
    cache_prefix: str = "gemm_bpl",
    total_k_blocks: Optional[int] = None,
    prebuilt_bitmap: Optional[torch.Tensor] = None,
) -> None:
    """Bitmap family (reference :1064-1138).  As in the reference, when a bitmap is passed it, not
    the id list, decides which blocks are summed (:847); the id list only answers "is it empty"."""
    if int(active_blocks.numel()) <= 0:
        out.zero_()
        return
    packed = _ops.get_packed_weight(weight, _BLOCK_K, cache_prefix)
    x2d, y2d = _views(x, out)
    if prebuilt_bitmap is not None:
        nb = (x.shape[-1] + _BLOCK_K - 1) // _BLOCK_K
        if total_k_blocks is not None and int(total_k_blocks) != nb:
            raise ValueError(f"total_k_blocks={total_k_blocks} does not match K={x.shape[-1]}")
        if int(prebuilt_bitmap.numel()) != nb:
            raise ValueError(f"bitmap has {prebuilt_bitmap.numel()} entries, expected {nb}")
        # the id list and the byte map agree in every caller: its length sizes the launch
        _ops.gemm(x2d, packed, y2d, bitmap=prebuilt_bitmap, k_host=min(int(active_blocks.numel()), nb))
    else:
        _ops.gemm(x2d, packed, y2d, ids=_ids32(active_blocks))


def _prepacked_block_sparse_gemm_from_active_blocks_bitmap_preload_splitk(
    x: torch.Tensor,
    weight: torch.Tensor,
    active_blocks: torch.Tensor,
    out: torch.Tensor,
    cache_prefix: str = "gemm_bpl_sk",
    total_k_blocks: Optional[int] = None,
    prebuilt_bitmap: Optional[torch.Tensor] = None,
    num_split_k: Optional[int] = None,
    tile_b: Optional[int] = None,
    tile_n: Optional[int] = None,
    tile_warps: Optional[int] = None,
    tile_stages: Optional[int] = None,
) -> None:
    """Bitmap family with split-K (reference :1235-1347); same computation as the call above."""
    _prepacked_block_sparse_gemm_from_active_blocks_bitmap_preload(
        x, weight, active_blocks, out, cache_prefix=cache_prefix,
        total_k_blocks=total_k_blocks, prebuilt_bitmap=prebuilt_bitmap)


def _prepacked_block_sparse_gemm_from_active_blocks(
    x: torch.Tensor,
    weight: torch.Tensor,
    active_blocks: torch.Tensor,
    out: torch.Tensor,
    cache_prefix: str = "gemm",
    proj_tag: str = "",
    sort_active_blocks: bool = True,
    use_run_compressed: bool = True,
    active_blocks_limit: Optional[int] = None,
) -> None:
    """Generic 1-D entry of the decode scripts (reference :3166-3344).  Sorting and run compression
    only reorder the same sum, so they are accepted and ignored; ``active_blocks_limit`` keeps the
    first entries of the list (:3178, :3190-3191)."""
    num_blocks = int(active_blocks.numel()) if active_blocks_limit is None else int(active_blocks_limit)
    if num_blocks <= 0:
        out.zero_()
        return
    ids = _ids32(active_blocks)
    if int(ids.numel()) > num_blocks:
        ids = ids[:num_blocks].contiguous()
    packed = _ops.get_packed_weight(weight, _BLOCK_K, cache_prefix)
    x2d, y2d = _views(x, out)
    _ops.gemm(x2d, packed, y2d, ids=ids)


# ---------------------------------------------------------------------------------------------
# Output-block ("2-D") sparsity and compact operands (reference :2289-2894, 3411-3495, 3498-4009).
# Explored by the reference, unused by its published numbers; here they are one more form of the
# same list launch (bas_list_call.n_ids_dev / shape_flags), through ops.gemm_2d.
# ---------------------------------------------------------------------------------------------
INDEX_BLOCK_OUT_META_SIZE = 64      # reference :19 reads an environment override; fixed here

_TEMP_BUFFERS: dict = {}


def _get_temp_tensor_buffer(prefix: str, shape, dtype, device, zero_fill: bool = False) -> torch.Tensor:
    """A scratch tensor that keeps its address from call to call (reference :3112-3130)."""
    key = (prefix, tuple(int(v) for v in shape), dtype, str(device))
    buf = _TEMP_BUFFERS.get(key)
    if buf is None:
        buf = torch.empty(key[1], dtype=dtype, device=device)
        _TEMP_BUFFERS[key] = buf
    if zero_fill:
        buf.zero_()
    return buf


def _sort_active_blocks_asc(active_blocks: torch.Tensor) -> torch.Tensor:
    return torch.sort(active_blocks).values if int(active_blocks.numel()) > 1 else active_blocks


def _prepacked_block_sparse_gemm_from_compact_input_blocks(
    x_compact: torch.Tensor,
    weight: torch.Tensor,
    active_blocks: torch.Tensor,
    out: torch.Tensor,
    cache_prefix: str = "gemm_compactin",
    sort_active_blocks: bool = True,
) -> None:
    """``x_compact`` [B, S, len(active_blocks) * 64] holds the active input blocks in ascending block
    order (reference :3411-3467)."""
    num_blocks = int(active_blocks.numel())
    if num_blocks <= 0:
        out.zero_()
        return
    ids = _ids32(active_blocks)
    if sort_active_blocks:
        ids = _sort_active_blocks_asc(ids)
    packed = _ops.get_packed_weight(weight, _BLOCK_K, cache_prefix)
    x2d, y2d = _views(x_compact, out)
    _ops.gemm_2d(x2d, packed, y2d, ids=ids, x_compact=True, k=int(weight.shape[1]))


def _scatter_compact_to_dense_output(compact_out: torch.Tensor, active_n_blocks: torch.Tensor, block_n: int,
                                     out_dense: torch.Tensor) -> None:
    """Columns ``i * block_n ..`` of the compact tensor go to block ``active_n_blocks[i]`` of the dense one
    (reference :3470-3495; there a host loop over ``.tolist()``, here one indexed copy on the device)."""
    if int(active_n_blocks.numel()) <= 0:
        return
    blk = int(block_n)
    n_dense = int(out_dense.shape[-1])
    comp2d = compact_out.reshape(-1, compact_out.shape[-1])
    out2d = out_dense.view(-1, n_dense)
    cols = (active_n_blocks.to(torch.int64)[:, None] * blk + torch.arange(blk, device=out_dense.device)[None, :]).reshape(-1)
    cols = cols[: comp2d.shape[1]]
    keep = cols < n_dense
    out2d[:, cols[keep]] = comp2d[:, : cols.numel()][:, keep]


def _prepacked_block_sparse_gemm_2d_from_active_blocks(
    x: torch.Tensor,
    weight: torch.Tensor,
    active_k_blocks: torch.Tensor,
    active_n_blocks: Optional[torch.Tensor],
    out: torch.Tensor,
    cache_prefix: str = "gemm2d",
    proj_tag: str = "",
    sort_active_k_blocks: bool = True,
    sort_active_n_blocks: bool = True,
    zero_fill_out: bool = False,
    compact_output: bool = False,
    scatter_compact_to_dense: bool = False,
    active_n_mask_u8: Optional[torch.Tensor] = None,
    active_k_blocks_limit: Optional[int] = None,
    active_n_blocks_limit: Optional[int] = None,
):
    """Only the output blocks in ``active_n_blocks`` (64 columns each) are computed (reference :3498-3850).
    Dense form: they land in their own columns of ``out``, the others keep what they held (zeros with
    ``zero_fill_out``); returns ``(None, ids)``.  ``compact_output``: they land side by side in a scratch tensor
    [B, S, len(ids) * 64] that is returned with the ids (and scattered into ``out`` on request).  The output
    width is the weight's, also where the reference passes a compact ``out``."""
    bsz, seqlen, _ = x.shape
    num_k = int(active_k_blocks.numel()) if active_k_blocks_limit is None else int(active_k_blocks_limit)
    if num_k <= 0:
        out.zero_()
        return None, torch.empty((0,), device=out.device, dtype=torch.int32)
    k_ids = _ids32(active_k_blocks)
    if int(k_ids.numel()) > num_k:
        k_ids = k_ids[:num_k].contiguous()
    if sort_active_k_blocks:
        k_ids = _sort_active_blocks_asc(k_ids)
    n_real = int(weight.shape[0])
    if active_n_blocks is None and active_n_mask_u8 is not None:
        # blocks with any active column (the reference keeps a cache of these per mask; this reads the mask)
        m = active_n_mask_u8.reshape(-1)
        pad = (-int(m.numel())) % INDEX_BLOCK_OUT_META_SIZE
        if pad:
            m = torch.cat([m, m.new_zeros(pad)])
        active_n_blocks = torch.nonzero(m.view(-1, INDEX_BLOCK_OUT_META_SIZE).any(dim=1)).reshape(-1).to(torch.int32)
    if active_n_blocks is None:
        active_n_blocks = torch.arange((n_real + 63) // 64, device=out.device, dtype=torch.int32)
    n_ids = _ids32(active_n_blocks)
    if sort_active_n_blocks:
        n_ids = _sort_active_blocks_asc(n_ids)
    num_n = int(n_ids.numel()) if active_n_blocks_limit is None else min(int(active_n_blocks_limit), int(n_ids.numel()))
    if num_n <= 0:
        out.zero_()
        return None, n_ids
    n_ids = n_ids[:num_n].contiguous()
    packed = _ops.get_packed_weight(weight, _BLOCK_K, cache_prefix)
    x2d = x.view(bsz * seqlen, x.shape[-1])
    if not x2d.is_contiguous():
        x2d = x2d.contiguous()
    if compact_output:
        comp = _get_temp_tensor_buffer(f"{cache_prefix}_compact2d_out", (bsz * seqlen, num_n * 64), out.dtype, out.device)
        _ops.gemm_2d(x2d, packed, comp, ids=k_ids, n_ids=n_ids, out_compact=True, n=n_real)
        comp3d = comp.view(bsz, seqlen, num_n * 64)
        if scatter_compact_to_dense:
            if zero_fill_out:
                out.zero_()
            _scatter_compact_to_dense_output(comp3d, n_ids, 64, out)
        return comp3d, n_ids
    if zero_fill_out:
        out.zero_()
    _, y2d = _views(x, out)
    _ops.gemm_2d(x2d, packed, y2d, ids=k_ids, n_ids=n_ids, n=n_real)
    return None, n_ids


def _prepacked_block_sparse_gemm_2d_bitmap_from_active_blocks(
    x: torch.Tensor,
    weight: torch.Tensor,
    active_k_blocks: torch.Tensor,
    active_n_blocks: Optional[torch.Tensor],
    out: torch.Tensor,
    cache_prefix: str = "gemm2d_bmp",
    sort_active_n_blocks: bool = True,
    zero_fill_out: bool = False,
    active_n_blocks_limit: Optional[int] = None,
):
    """The reference's sequential-bitmap form of the same contraction (:3853-3966): another way to walk the
    same blocks, so the same call here."""
    return _prepacked_block_sparse_gemm_2d_from_active_blocks(
        x, weight, active_k_blocks, active_n_blocks, out, cache_prefix=cache_prefix,
        sort_active_n_blocks=sort_active_n_blocks, zero_fill_out=zero_fill_out, active_n_blocks_limit=active_n_blocks_limit)


def _prepacked_block_sparse_gemm_2d_compact_from_active_blocks(
    x: torch.Tensor,
    weight: torch.Tensor,
    active_k_blocks: torch.Tensor,
    active_n_blocks: Optional[torch.Tensor],
    cache_prefix: str = "gemm2d_compact",
    proj_tag: str = "",
    sort_active_k_blocks: bool = True,
    sort_active_n_blocks: bool = True,
):
    """Compact output + the output block ids (reference :3969-4009)."""
    bsz, seqlen, _ = x.shape
    num_n = int(active_n_blocks.numel()) if active_n_blocks is not None else 0
    if num_n <= 0:
        return (torch.empty((bsz, seqlen, 0), device=x.device, dtype=x.dtype),
                torch.empty((0,), device=x.device, dtype=torch.int32))
    dummy = torch.empty((bsz, seqlen, 0), device=x.device, dtype=x.dtype)     # the dense output is not used
    comp, ids = _prepacked_block_sparse_gemm_2d_from_active_blocks(
        x, weight, active_k_blocks, active_n_blocks, dummy, cache_prefix=cache_prefix, proj_tag=proj_tag,
        sort_active_k_blocks=sort_active_k_blocks, sort_active_n_blocks=sort_active_n_blocks, compact_output=True)
    if comp is None:                       # no active input block: the product is zero
        comp = torch.zeros((bsz, seqlen, num_n * 64), device=x.device, dtype=x.dtype)
        ids = _sort_active_blocks_asc(_ids32(active_n_blocks)) if sort_active_n_blocks else _ids32(active_n_blocks)
    return comp, ids
