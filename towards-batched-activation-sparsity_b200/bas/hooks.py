"""Model hook layer: replaces ``forward`` of a model's linear projections by the masked decode
operator, with the semantics of the reference's patchers

* ``_patch_roundrobin_sparse`` / ``_restore`` (scripts/bench_roundrobin_e2e_decode.py:287-512): one
  density per (layer, projection) from an allocation table, optional per-step density schedules,
  block priors, weight-aware scores and mask reuse; prefill (more than one position) and
  density >= 1 stay dense;
* ``_patch_adaptive`` (scripts/bench_alpaca_energy_budget_e2e.py:65-123): energy-budget or uniform
  top-k selection on the block energies, with a dense fallback where too little would be skipped.

Differences a caller can observe: selection and contraction run on the device without a host
round trip (the reference's budget mode and dense fallback read the count on the host), so the
statistics that need that count are accumulated on the device and read by :func:`read_stats`; the
kernel-choice fields of a lookup table (``best_kern`` / ``mask``, ``best_K`` / ``K``, tiles) are
accepted in either schema and ignored, there being one kernel.  The reference's energy-gate
fallbacks (:371-468), a calibration experiment that reads a ratio on the host per call, are not
part of this layer.
"""

from __future__ import annotations

from typing import Callable, Optional

import torch

from . import ops
from .abi import BLOCK_K, SCORE_ENERGY, SCORE_NORM

PROJS = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
PROJ_TO_SHAPE = {"q_proj": "qkvo", "k_proj": "qkvo", "v_proj": "qkvo", "o_proj": "qkvo",
                 "gate_proj": "gate_up", "up_proj": "gate_up", "down_proj": "down"}


def get_module(model, layer_idx: int, proj: str):
    """``model.model.layers[i].self_attn.<proj>`` / ``.mlp.<proj>`` (reference :82-86)."""
    layer = model.model.layers[layer_idx]
    if proj in {"q_proj", "k_proj", "v_proj", "o_proj"}:
        return getattr(layer.self_attn, proj)
    return getattr(layer.mlp, proj)


def nearest_cfg(sweep: Optional[dict], shape: str, density: float) -> dict:
    """The lookup-table row nearest to ``density`` (reference :74-79), tolerant of both schemas the
    reference's scripts write and of a missing table."""
    if not sweep or shape not in sweep or not sweep[shape]:
        return {"best_kern": "bas", "best_K": 1, "best_tile": None, "density_key": None}
    rows = sweep[shape]
    key = min(rows.keys(), key=lambda k: abs(float(k) - float(density)))
    cfg = dict(rows[key])
    cfg.setdefault("best_kern", {"bitmap": "bpl"}.get(str(cfg.get("mask", "naive")), str(cfg.get("mask", "naive"))))
    cfg.setdefault("best_K", cfg.get("K", 1))
    cfg.setdefault("best_tile", cfg.get("tile"))
    cfg["density_key"] = key
    return cfg


def _num_layers(model) -> int:
    return len(model.model.layers)


def patch_sparse(model, alloc: dict, sweep: Optional[dict] = None, *, block_priors: Optional[dict] = None,
                 prior_alpha: float = 1.0, prior_eps: float = 0.1, reuse_masks: bool = False,
                 weight_aware_score: bool = False, step_density_alloc: Optional[dict] = None,
                 score_kind: int = SCORE_NORM, module_of: Callable = get_module, projs=PROJS):
    """Patch every projection of every layer; returns ``(originals, stats)`` for :func:`restore`.

    ``alloc[str(layer)][proj]`` is the kept density of that cell; ``step_density_alloc[(layer, proj)]``
    optionally a list of densities per decode step (index 0 belongs to the dense prefill pass: decode
    calls start at index 1 and wrap, reference :345-360); ``block_priors[(layer, proj)]`` a float
    tensor per block; ``weight_aware_score`` weights the squares by the squared column norms of the
    weight (:319-320); ``reuse_masks`` keeps the first decode call's mask of a cell for all later ones."""
    block_k = BLOCK_K
    stats = {"calls": 0, "sparse_calls": 0, "dense_calls": 0}
    mask_cache: dict = {}
    decode_calls: dict = {}
    originals = []
    for li in range(_num_layers(model)):
        for proj in projs:
            mod = module_of(model, li, proj)
            density = float(alloc[str(li)][proj])
            schedule = (step_density_alloc or {}).get((li, proj))
            scale = None
            if weight_aware_score and density < 1.0:
                scale = mod.weight.detach().float().pow(2).sum(dim=0).contiguous()
            cfg = nearest_cfg(sweep, PROJ_TO_SHAPE.get(proj, proj), density)
            prefix = f"bas_hook_l{li}_{proj}"
            ops.get_packed_weight(mod.weight, block_k, prefix)          # warm the pack cache (:321)
            prior = (block_priors or {}).get((li, proj))
            mult = None
            if prior is not None and int(prior.numel()) == int(mod.weight.shape[1]) // block_k:
                mult = ops.prior_multiplier(prior.to(mod.weight.device), prior_alpha, prior_eps)
            orig_forward = mod.forward

            def forward(x, _mod=mod, _density=density, _prefix=prefix, _mult=mult, _key=(li, proj), _orig=orig_forward,
                        _scale=scale, _schedule=schedule, _cfg=cfg):
                stats["calls"] += 1
                x3 = x.reshape(x.shape[0], 1, x.shape[-1]) if x.dim() == 2 else x
                active_density = _density
                if _schedule is not None and x3.shape[1] == 1:
                    raw = int(decode_calls.get(_key, 0))
                    decode_calls[_key] = raw + 1
                    idx = (raw % (len(_schedule) - 1)) + 1 if len(_schedule) > 1 else 0
                    active_density = float(_schedule[idx] if idx < len(_schedule) else _schedule[-1])
                if x3.shape[1] != 1 or active_density >= 1.0:              # prefill and dense cells (:200-201)
                    stats["dense_calls"] += 1
                    return _orig(x)
                stats["sparse_calls"] += 1
                bias = getattr(_mod, "bias", None)
                if reuse_masks and _key in mask_cache:
                    y = ops.sparse_linear(x, _mod.weight, active_density, cache_prefix=_prefix,
                                          fixed_active_blocks=mask_cache[_key])
                else:
                    y = ops.sparse_linear(x, _mod.weight, active_density, score_kind=score_kind, cache_prefix=_prefix,
                                          block_mult=_mult, block_score_scale=_scale)
                    if reuse_masks:
                        nb = x3.shape[2] // block_k
                        n_keep = ops.n_keep_from_density(active_density, nb)
                        ids, _ = ops.select_topk(x3.reshape(x3.shape[0], x3.shape[2]), n_keep, score_kind,
                                                 chan_scale=_scale, block_mult=_mult)
                        mask_cache[_key] = ids.clone()
                return y if bias is None else y + bias

            mod.forward = forward
            originals.append((mod, orig_forward))
    stats["mask_cache"] = mask_cache
    return originals, stats


def patch_adaptive(model, sweep: Optional[dict], mode: str, value: float, *, min_sparse_sparsity: float = 0.0,
                   module_of: Callable = get_module, projs=PROJS):
    """``mode='energy'``: keep the shortest descending-energy prefix of blocks reaching ``value`` of the
    total energy; ``mode='uniform'``: keep ``1 - value`` of the blocks by energy.  Where the kept
    share would skip less than ``min_sparse_sparsity`` of the blocks the call is dense
    (scripts/bench_alpaca_energy_budget_e2e.py:104-109): here the selection kernel then keeps every
    block, on the device, and the same contraction kernel runs them all.  Returns
    ``(originals, stats)``; ``stats['cells'][(layer, proj)]`` holds a device tensor
    ``[kept, total, dense_fallbacks]`` that every decode call adds to (:func:`read_stats`)."""
    if mode not in ("energy", "uniform"):
        raise ValueError("mode must be 'energy' or 'uniform'")
    block_k = BLOCK_K
    stats = {"calls": 0, "cells": {}}
    originals = []
    for li in range(_num_layers(model)):
        for proj in projs:
            mod = module_of(model, li, proj)
            nb = int(mod.weight.shape[1]) // block_k
            prefix = f"bas_hook_eb_l{li}_{proj}"
            ops.get_packed_weight(mod.weight, block_k, prefix)
            nearest_cfg(sweep, PROJ_TO_SHAPE.get(proj, proj), 1.0)      # lookup tables are tolerated, not needed
            # largest kept count that still counts as sparse, by the reference's own float test
            full_above = nb
            for kk in range(nb + 1):
                if (1.0 - float(kk) / float(nb)) < float(min_sparse_sparsity):
                    full_above = kk - 1
                    break
            cell = torch.zeros(3, dtype=torch.int64, device=mod.weight.device)
            stats["cells"][(li, proj)] = cell
            ids_buf = torch.empty(nb, dtype=torch.int32, device=mod.weight.device)
            cnt_buf = torch.zeros(1, dtype=torch.int32, device=mod.weight.device)
            orig_forward = mod.forward

            def forward(x, _mod=mod, _orig=orig_forward, _prefix=prefix, _nb=nb, _full=full_above, _cell=cell,
                        _ids=ids_buf, _cnt=cnt_buf):
                stats["calls"] += 1
                x3 = x.reshape(x.shape[0], 1, x.shape[-1]) if x.dim() == 2 else x
                if x3.shape[1] != 1:                                     # prefill stays dense (:87-88)
                    return _orig(x)
                bt, k = x3.shape[0], x3.shape[2]
                x2d = x3.reshape(bt, k)
                packed = ops.get_packed_weight(_mod.weight, block_k, _prefix)
                out = torch.empty(bt, 1, _mod.weight.shape[0], device=x.device, dtype=x.dtype)
                if mode == "energy":
                    ops.select_budget(x2d, float(value), 1, ids_out=_ids, count_out=_cnt, full_above=_full)
                else:
                    n_keep = ops.n_keep_from_density(1.0 - float(value), _nb)
                    if n_keep > _full:
                        n_keep = _nb
                    ops.select_topk(x2d, n_keep, SCORE_ENERGY, ids_out=_ids, count_out=_cnt)
                ops.gemm(x2d, packed, out.view(bt, -1), ids=_ids, count=_cnt, k_host=_nb)
                # statistics without a host round trip: kept, total, calls that ran every block
                _cell[0] += _cnt[0]
                _cell[1] += _nb
                _cell[2] += (_cnt[0] > _full).to(torch.int64)
                bias = getattr(_mod, "bias", None)
                y = out.reshape(bt, -1) if x.dim() == 2 else out
                return y if bias is None else y + bias

            mod.forward = forward
            originals.append((mod, orig_forward))
    return originals, stats


def read_stats(stats: dict) -> dict:
    """Host copy of the per-cell counters of :func:`patch_adaptive` (synchronises)."""
    out = {}
    for key, cell in stats.get("cells", {}).items():
        kept, total, dense = (int(v) for v in cell.cpu().tolist())
        out[key] = {"kept": kept, "total_k": total, "dense_fallback_calls": dense}
    return out


def restore(originals) -> None:
    """Undo :func:`patch_sparse` / :func:`patch_adaptive` (reference :510-512)."""
    for mod, orig in originals:
        mod.forward = orig
