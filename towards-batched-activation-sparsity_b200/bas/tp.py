"""Tensor-parallel layout of a decode-step linear stack over the GPUs of one box.

The reference is single-GPU (it has no distributed code); this module is the sharding the
benchmark specification asks for on top of the same kernels:

* q, k, v, gate, up are column-parallel: rank r owns output columns [n0, n1) and produces that
  slice of Y; nothing is exchanged.
* o, down are row-parallel: rank r owns the 64-channel blocks [b0, b1) of the input, multiplies
  its slice of X with its slice of W, and the partial outputs are summed with one NCCL
  all-reduce.
* The batch-shared block mask is replicated: every rank holds the same byte map over all
  blocks; a row-parallel rank simply passes the slice [b0, b1) of it to the kernel (a view: no
  copy, no host synchronisation).

Pure layout arithmetic lives in :func:`shard_bounds` and is testable without a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

BLOCK_K = 64


def shard_bounds(total_units: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, near-equal split of ``total_units`` over ``world`` ranks: [begin, end) of ``rank``.
    172 blocks over 8 ranks gives 22/21-block shards (172 = 8 * 21 + 4)."""
    if not (0 <= rank < world) or total_units < 0:
        raise ValueError("bad rank / world / size")
    return rank * total_units // world, (rank + 1) * total_units // world


def column_shard(n: int, world: int, rank: int, align: int = BLOCK_K) -> tuple[int, int]:
    """Output-column range of a column-parallel linear, in whole groups of ``align`` columns so that
    the gate/up shard of a rank is exactly the input shard of its down projection."""
    units = (n + align - 1) // align
    u0, u1 = shard_bounds(units, world, rank)
    return min(u0 * align, n), min(u1 * align, n)


def row_shard_blocks(k: int, world: int, rank: int) -> tuple[int, int]:
    """Input-block range [b0, b1) of a row-parallel linear."""
    return shard_bounds((k + BLOCK_K - 1) // BLOCK_K, world, rank)


@dataclass
class LinearSpec:
    name: str
    n: int            # output features
    k: int            # input features
    parallel: str     # "column" or "row"
    dist: str         # activation distribution of its input: "normal" or "laplace"


# One Llama-2-7B decoder layer's projections (scripts/bench_perstep_actual_kernel_speedup.py:37-53).
LLAMA2_7B_LAYER = (
    LinearSpec("q_proj", 4096, 4096, "column", "normal"),
    LinearSpec("k_proj", 4096, 4096, "column", "normal"),
    LinearSpec("v_proj", 4096, 4096, "column", "normal"),
    LinearSpec("o_proj", 4096, 4096, "row", "normal"),
    LinearSpec("gate_proj", 11008, 4096, "column", "normal"),
    LinearSpec("up_proj", 11008, 4096, "column", "normal"),
    LinearSpec("down_proj", 4096, 11008, "row", "laplace"),
)


# Projections that read the same activation through the same mask can run as one masked GEMM over
# their concatenated output columns (the reference's own CLI assumes this for q/k/v,
# kernels/shared_mask_batched_triton_min_runtime.py:4645): q+k+v and gate+up.
SHARES_PREVIOUS_INPUT = ("k_proj", "v_proj", "up_proj")
FUSED_GROUPS = (("qkv_proj", ("q_proj", "k_proj", "v_proj")), ("gate_up_proj", ("gate_proj", "up_proj")))


class ShardedLinear:
    """One rank's shard of a masked linear: packed weight slice plus the views it needs per call.
    ``weight_full`` may be a list of [n_i, k] matrices of column-parallel projections sharing one
    input: the rank's column shard of each is taken and they are stacked into one packed weight."""

    def __init__(self, spec: LinearSpec, weight_full, world: int, rank: int):
        import torch

        from . import ops

        self.spec, self.world, self.rank = spec, world, rank
        parts = list(weight_full) if isinstance(weight_full, (list, tuple)) else [weight_full]
        if spec.parallel == "column":
            self.part_bounds = [column_shard(w.shape[0], world, rank) for w in parts]
            self.n0, self.n1 = self.part_bounds[0] if len(parts) == 1 else (0, sum(b - a for a, b in self.part_bounds))
            self.b0, self.b1 = 0, (spec.k + BLOCK_K - 1) // BLOCK_K
            shard = torch.cat([w[a:b] for w, (a, b) in zip(parts, self.part_bounds)]) if len(parts) > 1 \
                else parts[0][self.n0:self.n1]
        else:
            if len(parts) != 1:
                raise ValueError("only column-parallel projections can be stacked")
            self.n0, self.n1 = 0, spec.n
            self.b0, self.b1 = row_shard_blocks(spec.k, world, rank)
            shard = parts[0][:, self.b0 * BLOCK_K: min(self.b1 * BLOCK_K, spec.k)]
        self.k_local = shard.shape[1]
        self.n_local = shard.shape[0]
        self.packed = ops.pack_weight(shard.contiguous()) if self.n_local and self.k_local else None

    def forward(self, x2d, bitmap, out2d, ids_stable: bool = True, exchange=None, n_keep: int = 0,
                x_stable: bool = False, next_independent: bool = False):
        """x2d is the replicated [B, K] activation, bitmap the replicated uint8[K/64] mask.  Writes
        this rank's output slice (column-parallel) or partial sum (row-parallel) into out2d; with an
        ``exchange`` group a row-parallel linear writes the sum over all ranks instead (formed inside
        the contraction kernel), and no collective has to follow."""
        from . import ops

        if self.packed is None:
            if exchange is not None:
                raise ValueError("a rank without a K-shard cannot take part in the in-kernel sum")
            out2d.zero_()
            return
        row = self.spec.parallel == "row"
        xs = x2d[:, self.b0 * BLOCK_K: self.b0 * BLOCK_K + self.k_local] if row else x2d
        # n_keep: active blocks of the whole mask; a K-shard expects its share of them
        nb_all = bitmap.numel()
        hint = max(1, (int(n_keep) * (self.b1 - self.b0) + nb_all - 1) // nb_all) if n_keep else 0
        ops.gemm(xs, self.packed, out2d, bitmap=bitmap[self.b0:self.b1], k_host=hint, ids_stable=ids_stable,
                 x_stable=x_stable, next_independent=next_independent, tp=exchange if row else None)


class DecodeLinearStack:
    """``layers`` x the seven projections, random-init N(0, 0.02^2), sharded over the process group.

    ``step()`` runs every linear once on its replicated synthetic input with its fixed mask and
    all-reduces the row-parallel outputs; it is what the benchmark times as one decode step of the
    linear stack.  Inputs are generated per linear, identically on every rank.

    ``fuse_shared_inputs``: q/k/v and gate/up read one activation through one mask (as they do in
    the model) and run as one masked GEMM each: four launches per layer instead of seven.
    ``allreduce``: how the row-parallel partial outputs are summed over the ranks."""

    def __init__(self, layers: int, batch: int, sparsity: float, device, world: int = 1, rank: int = 0,
                 seed: int = 0, group=None, fuse_shared_inputs: bool = False, allreduce: str = "nccl",
                 specs=LLAMA2_7B_LAYER):
        import torch

        from . import ops
        from .abi import SCORE_NORM

        if allreduce not in ("nccl", "in_kernel"):
            raise ValueError("allreduce must be 'nccl' or 'in_kernel'")
        self.world, self.rank, self.group, self.batch = world, rank, group, batch
        # "in_kernel": o and down add their partial outputs over the ranks inside the contraction
        # kernel (peer stores over NVLink, each rank polls its own area); "nccl": one all-reduce call after each of them
        self.specs = tuple(specs)    # the projections of one layer, by the seven names of LLAMA2_7B_LAYER
        self.exchange = ops.ExchangeGroup(device, batch, max(s.n for s in self.specs if s.parallel == "row"),
                                          group) if allreduce == "in_kernel" else None
        # True: every call declares its input stable, which the stack's pre-generated inputs literally
        # are (a throughput probe over the seven shapes; a model's o, down, q and gate depend on the
        # kernel before them and could not)
        self.independent_calls = False
        self.items = []
        self.item_meta = []      # per item: (layer, [index of each stacked projection in LLAMA2_7B_LAYER])
        self.seed = seed
        self._shared = {}
        gen = torch.Generator(device=device)
        self.active_bytes = 0
        fused_of = {m: name for name, members in FUSED_GROUPS for m in members} if fuse_shared_inputs else {}

        def shared_input(spec):
            if spec.name not in self._shared:     # inputs and masks are per projection type, shared by the layers
                if spec.dist == "normal":
                    x = torch.randn(batch, spec.k, generator=gen, device=device, dtype=torch.float32).half()
                else:
                    u = torch.rand(batch, spec.k, generator=gen, device=device, dtype=torch.float32) - 0.5
                    x = (-torch.sign(u) * torch.log1p(-2.0 * u.abs())).half()
                nb = spec.k // BLOCK_K
                n_keep = ops.n_keep_from_density(1.0 - sparsity, nb)
                bitmap = torch.empty(nb, dtype=torch.uint8, device=device)
                ops.select_topk(x, n_keep, SCORE_NORM, bitmap_out=bitmap)
                self._shared[spec.name] = (x, bitmap, n_keep)
            return self._shared[spec.name]

        for li in range(layers):
            pending = {}     # fused group name -> [spec, weights]
            pending_si = {}
            for si, spec in enumerate(self.specs):
                gen.manual_seed(seed * 1_000_003 + li * 16 + si)
                w = (torch.randn(spec.n, spec.k, generator=gen, device=device, dtype=torch.float32) * 0.02).half()
                group_name = fused_of.get(spec.name)
                if group_name is not None:
                    members = dict(FUSED_GROUPS)[group_name]
                    entry = pending.setdefault(group_name, [spec, []])
                    entry[1].append(w)
                    pending_si.setdefault(group_name, []).append(si)
                    if len(entry[1]) < len(members):
                        continue
                    first, ws = entry
                    spec = LinearSpec(group_name, sum(t.shape[0] for t in ws), first.k, "column", first.dist)
                    x, bitmap, n_keep = shared_input(first)
                    lin = ShardedLinear(spec, ws, world, rank)
                    self.item_meta.append((li, list(pending_si[group_name])))
                    del ws, entry[1][:]
                else:
                    x, bitmap, n_keep = shared_input(spec)
                    lin = ShardedLinear(spec, w, world, rank)
                    self.item_meta.append((li, [si]))
                del w
                out = torch.zeros(batch, lin.n_local, dtype=torch.float16, device=device)
                self.items.append((lin, x, bitmap, out, n_keep))
                self.active_bytes += n_keep * BLOCK_K * spec.n * 2
        torch.cuda.synchronize(device)
        if world > 1:
            # the ranks have generated and packed their weights at their own pace: meet before the first
            # step, whose exchange kernels wait (bounded) for one another inside the kernel
            import torch.distributed as dist
            dist.barrier(group=group)

    def close(self) -> None:
        """Collective when the stack sums inside the kernel: releases the exchange areas."""
        if self.exchange is not None:
            self.exchange.close()
            self.exchange = None

    def parity_check(self, layers: int = 1) -> dict:
        """Run one step and compare this rank's outputs of the first ``layers`` layers with the
        unsharded product, computed here in fp32 from the regenerated full weights (the single-GPU
        result is the oracle of the sharded one): a column-parallel output against its column range, a
        row-parallel output - after the sum over ranks - against the whole product.  Also checks that
        every rank holds the same masks (a hash of every byte map, gathered over the group).
        Returns ``{"checked", "max_err", "ids_equal"}`` with the maximum taken over the ranks; collective."""
        self.step()
        return self.parity_check_outputs(layers)

    def parity_check_outputs(self, layers: int = 1) -> dict:
        """The comparison of :meth:`parity_check` on whatever the output buffers hold now."""
        import torch
        import torch.distributed as dist

        torch.cuda.synchronize()
        dev = self.items[0][1].device
        gen = torch.Generator(device=dev)
        max_err, checked = 0.0, 0
        for (lin, x, bitmap, out, _), (li, sis) in zip(self.items, self.item_meta):
            if li >= layers:
                continue
            mask = bitmap.to(torch.float32).repeat_interleave(BLOCK_K)[: x.shape[1]]
            xm = x.float() * mask
            parts = []
            for si, (a, b) in zip(sis, lin.part_bounds if lin.spec.parallel == "column" else [(0, lin.spec.n)]):
                spec = self.specs[si]
                gen.manual_seed(self.seed * 1_000_003 + li * 16 + si)
                w = (torch.randn(spec.n, spec.k, generator=gen, device=dev, dtype=torch.float32) * 0.02).half()
                parts.append((xm @ w.float().t())[:, a:b])
                del w
            ref = torch.cat(parts, dim=1)
            err = float((out.float() - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
            max_err = max(max_err, err)
            checked += 1
        # same masks everywhere: position-weighted sum and population of every byte map
        sig = []
        for name in sorted(self._shared):
            bm = self._shared[name][1].to(torch.int64)
            sig += [int((bm * torch.arange(1, bm.numel() + 1, device=bm.device)).sum()), int(bm.sum())]
        ids_equal = True
        if self.world > 1:
            mine = torch.tensor(sig, dtype=torch.int64, device=dev)
            gathered = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(gathered, mine, group=self.group)
            ids_equal = all(bool(torch.equal(g, gathered[0])) for g in gathered)
            t = torch.tensor([max_err], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
            max_err = float(t.item())
        return {"checked": checked, "max_err": max_err, "ids_equal": bool(ids_equal)}

    # what each projection's input is the output of, in the model (attention itself is not part of
    # the stack: o reads what follows v)
    MODEL_DEPENDENCY = {"q_proj": "down_proj", "k_proj": "down_proj", "v_proj": "down_proj", "qkv_proj": "down_proj",
                        "o_proj": ("v_proj", "qkv_proj"), "gate_proj": "o_proj", "up_proj": "o_proj",
                        "gate_up_proj": "o_proj", "down_proj": ("up_proj", "gate_up_proj")}

    def make_list(self, dependencies: bool = True, select: bool = False, sharded_select: bool = False, **tuning):
        """The whole step as one persistent launch per rank (``ops.GemmList``).  With ``dependencies``
        every call waits for the call whose output its input is in the model; without, no call waits
        for any other (a probe of the kernel's streaming rate; single GPU only).  On several ranks the
        stack must have been built with ``allreduce="in_kernel"``: the row-parallel calls then add their
        outputs over the ranks inside the list kernel, through the stack's exchange group.

        ``select``: the masks are not taken from the stack's byte maps but computed inside the launch, as a
        decode step has to: one selection entry per distinct input, scored once that input is complete, ranked
        by the calls that use it.  A row-parallel call ranks
        the whole (replicated) input's scores and keeps the blocks of its own K-shard - or, ``sharded_select``,
        every rank scores only its own K-shard of a row-parallel call's input, as if that were all it held (what a
        chained forward leaves it with), and the ranks exchange the scores inside the launch."""
        from . import ops
        from .abi import SCORE_NORM

        if self.world != 1 and (self.exchange is None or not dependencies):
            raise ValueError("on several ranks the one-launch step needs allreduce='in_kernel' and the dependencies")
        last = {}
        calls = []
        entry_of = {}     # (layer, input name) -> index of its selection entry
        for (lin, x, bitmap, out, n_keep), (li, _) in zip(self.items, self.item_meta):
            dep = -1
            if dependencies:
                want = self.MODEL_DEPENDENCY[lin.spec.name]
                for name in (want if isinstance(want, tuple) else (want,)):
                    dep = max(dep, last.get(name, -1))
            row = lin.spec.parallel == "row"
            xs = x[:, lin.b0 * BLOCK_K: lin.b0 * BLOCK_K + lin.k_local] if row else x
            call = {"x": xs, "packed": lin.packed, "out": out, "depends_on": dep, "row_parallel": row and self.world > 1}
            if select:
                # one entry per distinct input of a layer (this stack generates an input per projection type, so
                # only the stacked q+k+v and gate+up share one: four entries per layer then, as in the model)
                sharded = sharded_select and row and self.world > 1
                key = (li, x.data_ptr(), dep, sharded)
                if key not in entry_of:
                    entry_of[key] = len(calls)
                    entry = {"select": xs if sharded else x, "n_keep": int(n_keep), "score_kind": SCORE_NORM, "depends_on": dep}
                    if sharded:
                        entry["sharded"] = (lin.b0, bitmap.numel())
                    calls.append(entry)
                call["mask_from"] = entry_of[key]
                call["mask_block0"] = lin.b0 if row else 0
            else:
                nb_all = bitmap.numel()
                call["bitmap"] = bitmap[lin.b0:lin.b1]
                call["k_host"] = max(1, (int(n_keep) * (lin.b1 - lin.b0) + nb_all - 1) // nb_all)
            last[lin.spec.name] = len(calls)
            calls.append(call)
        return ops.GemmList(calls, tp=self.exchange if self.world > 1 else None, **tuning)

    def step(self) -> None:
        import torch.distributed as dist

        for lin, x, bitmap, out, n_keep in self.items:
            # k, v and up read, in the model, the activation the call before them (q, gate) has already
            # read: only these declare their input stable
            lin.forward(x, bitmap, out, exchange=self.exchange, n_keep=n_keep,
                        x_stable=self.independent_calls or lin.spec.name in SHARES_PREVIOUS_INPUT,
                        next_independent=self.independent_calls)
            if lin.spec.parallel == "row" and self.world > 1 and self.exchange is None:
                dist.all_reduce(out, group=self.group)
