"""One rank of the multi-GPU test of the row-parallel sum formed inside the contraction kernel
(started by tests/test_tp_gpu.py through torch.distributed.run, one process per GPU).  Not a test
module itself."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "towards-batched-activation-sparsity_b200"))

from bas import ops, tp          # noqa: E402
from oracle import bas_oracle as O   # noqa: E402

TOL = 2e-3


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    group = ops.ExchangeGroup(dev, 64, 4104)
    failures = []
    call = 0
    for b, k, n, n_keep in [(16, 11008, 4096, 62), (64, 11008, 4096, 83), (2, 4096, 4096, 13), (33, 1088, 4104, 9),
                            (16, 11008, 4096, 3), (16, 11008, 4096, 62)]:
        nb = (k + 63) // 64
        x_h = O.make_activations(b, k, seed=100 + call, dist="laplace")
        w_h = O.make_weight(n, k, seed=200 + call)
        ids_h = O.random_active_blocks(nb, n_keep, seed=300 + call)
        b0, b1 = tp.row_shard_blocks(k, world, rank)
        k0, k1 = b0 * 64, min(b1 * 64, k)
        x = torch.from_numpy(x_h).to(dev)
        packed = ops.pack_weight(torch.from_numpy(np.ascontiguousarray(w_h[:, k0:k1])).to(dev))
        bitmap = torch.from_numpy(O.build_bitmap(ids_h, nb)).to(dev)
        out = torch.full((b, n), float("nan"), dtype=torch.float16, device=dev)
        for rep in range(3):
            out.fill_(float("nan"))
            ops.gemm(x[:, k0:k1], packed, out, bitmap=bitmap[b0:b1], tp=group, ids_stable=bool(rep & 1))
            call += 1
        torch.cuda.synchronize()
        status = ops.read_status(dev)
        err = O.max_err_ratio(out.float().cpu().numpy(), O.masked_gemm(x_h, w_h, ids_h))
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        same = all(torch.equal(g, gathered[0]) for g in gathered)
        if status != 0 or not err <= TOL or not same:
            failures.append((b, k, n, n_keep, status, err, same))
    # ranks that split the work differently (another grid size, another cluster shape, an id list of
    # another length): elements are exchanged by (row, column), so the sums must not care
    for b, k, n, n_keep in [(16, 11008, 4096, 62), (64, 4096, 4096, 23), (5, 2048, 4104, 9)]:
        nb = (k + 63) // 64
        x_h = O.make_activations(b, k, seed=500 + call, dist="laplace")
        w_h = O.make_weight(n, k, seed=600 + call)
        ids_h = O.random_active_blocks(nb, n_keep, seed=700 + call)
        b0, b1 = tp.row_shard_blocks(k, world, rank)
        k0, k1 = b0 * 64, min(b1 * 64, k)
        local = ids_h[(ids_h >= b0) & (ids_h < b1)] - b0
        x = torch.from_numpy(x_h).to(dev)
        packed = ops.pack_weight(torch.from_numpy(np.ascontiguousarray(w_h[:, k0:k1])).to(dev))
        out = torch.full((b, n), float("nan"), dtype=torch.float16, device=dev)
        ops.gemm(x[:, k0:k1], packed, out, ids=torch.from_numpy(np.ascontiguousarray(local, dtype=np.int32)).to(dev),
                 tp=group, cluster=(1, 2, 4, 0)[rank % 4], max_ctas=(40, 96, 0, 148)[rank % 4])
        call += 1
        torch.cuda.synchronize()
        status = ops.read_status(dev)
        err = O.max_err_ratio(out.float().cpu().numpy(), O.masked_gemm(x_h, w_h, ids_h))
        gathered = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(gathered, out)
        same = all(torch.equal(g, gathered[0]) for g in gathered)
        if status != 0 or not err <= TOL or not same:
            failures.append(("mixed grids", b, k, n, n_keep, status, err, same))
    # the layer stack: in-kernel sums against NCCL all-reduces of fp16 partials
    outs = {}
    for mode in ("nccl", "in_kernel"):
        stack = tp.DecodeLinearStack(1, 16, 0.638, dev, world, rank, seed=3, allreduce=mode)
        stack.step()
        stack.step()
        torch.cuda.synchronize()
        outs[mode] = [o.float().clone() for lin, _, _, o, _ in stack.items if lin.spec.parallel == "row"]
        if ops.read_status(dev) != 0:
            failures.append(("stack status", mode))
        stack.close()
        del stack
    for a, c in zip(outs["nccl"], outs["in_kernel"]):
        d = float((a - c).abs().max() / c.abs().max())
        if not d <= 4e-3:       # the NCCL path rounds every rank's partial to fp16 first
            failures.append(("stack", d))
    group.close()
    # The same sums inside a list launch: column-parallel -> row-parallel -> column-parallel -> row-parallel,
    # every call reading the output of the call before it; the row-parallel outputs (summed over the ranks
    # inside the kernel: partials to the tile's owner, results back) against the oracle and across ranks.
    lgroup = ops.ExchangeGroup(dev, 64, 4096)
    for b, kk, cluster_ok in [(16, 2048, True), (64, 4096, True), (5, 1024, True)]:
        nmid = 4096
        x_h = O.make_activations(b, kk, seed=800 + b)
        wa_h, wb_h = O.make_weight(nmid, kk, seed=801 + b, std=0.03), O.make_weight(4096, nmid, seed=802 + b, std=0.03)
        wc_h, wd_h = O.make_weight(nmid, 4096, seed=803 + b, std=0.03), O.make_weight(1000, nmid, seed=804 + b, std=0.03)
        ia, ib = O.random_active_blocks(kk // 64, max(1, kk // 128), seed=805), O.random_active_blocks(nmid // 64, 23, seed=806)
        ic, idd = O.random_active_blocks(64, 30, seed=807), O.random_active_blocks(nmid // 64, 40, seed=808)
        n0, n1 = tp.column_shard(nmid, world, rank)                   # this rank's columns of the column-parallel calls
        b0, b1 = n0 // 64, n1 // 64                                   # = its input blocks of the row-parallel calls
        def pk(w):
            return ops.pack_weight(torch.from_numpy(np.ascontiguousarray(w)).to(dev))
        def local_ids(ids):
            return torch.from_numpy(np.ascontiguousarray(ids[(ids >= b0) & (ids < b1)] - b0, dtype=np.int32)).to(dev)
        x = torch.from_numpy(x_h).to(dev)
        ya = torch.full((b, n1 - n0), float("nan"), dtype=torch.float16, device=dev)
        yb = torch.full((b, 4096), float("nan"), dtype=torch.float16, device=dev)
        yc = torch.full((b, n1 - n0), float("nan"), dtype=torch.float16, device=dev)
        yd = torch.full((b, 1000), float("nan"), dtype=torch.float16, device=dev)
        lst = ops.GemmList([
            {"x": x, "packed": pk(wa_h[n0:n1]), "out": ya, "ids": torch.from_numpy(ia).to(dev)},
            {"x": ya, "packed": pk(wb_h[:, n0:n1]), "out": yb, "ids": local_ids(ib), "depends_on": 0, "row_parallel": True},
            {"x": yb, "packed": pk(wc_h[n0:n1]), "out": yc, "ids": torch.from_numpy(ic).to(dev), "depends_on": 1},
            {"x": yc, "packed": pk(wd_h[:, n0:n1]), "out": yd, "ids": local_ids(idd), "depends_on": 2, "row_parallel": True},
        ], tp=lgroup)
        for rep in range(3):
            lst.run()
        torch.cuda.synchronize()
        status = lst.read_status()
        # the oracle, stage by stage on the device's own (gathered) inputs
        def gathered_cols(t):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t.contiguous())
            return torch.cat(parts, dim=1).float().cpu().numpy()
        ya_full = gathered_cols(ya)
        yc_full = gathered_cols(yc)
        errs = [O.max_err_ratio(ya_full, O.masked_gemm(x_h, wa_h, ia)),
                O.max_err_ratio(yb.float().cpu().numpy(), O.masked_gemm(ya_full.astype(np.float16), wb_h, ib)),
                O.max_err_ratio(yc_full, O.masked_gemm(yb.cpu().numpy(), wc_h, ic)),
                O.max_err_ratio(yd.float().cpu().numpy(), O.masked_gemm(yc_full.astype(np.float16), wd_h, idd))]
        same = True
        for t in (yb, yd):
            parts = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(parts, t)
            same = same and all(torch.equal(g, parts[0]) for g in parts)
        if status != 0 or not all(e <= TOL for e in errs) or not same:
            failures.append(("list exchange", b, kk, status, errs, same))
        lst.close()
    # the layer stack as one launch per rank against the per-call in-kernel sums
    stack = tp.DecodeLinearStack(2, 16, 0.638, dev, world, rank, seed=5, allreduce="in_kernel")
    par = stack.parity_check(layers=2)
    lst = stack.make_list()
    for o in [it[3] for it in stack.items]:
        o.fill_(float("nan"))
    lst.run()
    lst.run()
    torch.cuda.synchronize()
    par_list = stack.parity_check_outputs(layers=2)
    if lst.read_status() != 0 or not par["max_err"] <= TOL or not par_list["max_err"] <= TOL or not par_list["ids_equal"]:
        failures.append(("stack as a list", par, par_list))
    lst.close()
    # ... and with the masks computed inside the launch (a row-parallel call keeps its K-shard's part of the mask
    # that every rank ranks from the same scores)
    lst = stack.make_list(select=True)
    for o in [it[3] for it in stack.items]:
        o.fill_(float("nan"))
    lst.run()
    lst.run()
    torch.cuda.synchronize()
    par_sel = stack.parity_check_outputs(layers=2)
    status = lst.read_status()
    if status != 0 or not par_sel["max_err"] <= TOL:
        failures.append(("stack as a list with selection", hex(status), par_sel))
    lst.close()
    # ... and with every rank scoring only its own K-shard of a row-parallel call's input: the ranks exchange the
    # block scores inside the launch and keep their part of ONE global top-k - the same mask as before
    lst = stack.make_list(select=True, sharded_select=True)
    for o in [it[3] for it in stack.items]:
        o.fill_(float("nan"))
    for _ in range(3):
        lst.run()
    torch.cuda.synchronize()
    par_sh = stack.parity_check_outputs(layers=2)
    status = lst.read_status()
    if status != 0 or not par_sh["max_err"] <= TOL:
        failures.append(("stack as a list with sharded selection", hex(status), par_sh))
    lst.close()
    stack.close()
    # the same on shards of unequal size (43 blocks over two ranks: 21 / 22)
    small = tuple(tp.LinearSpec(s.name, {4096: 1024, 11008: 2752}[s.n], {4096: 1024, 11008: 2752}[s.k], s.parallel, s.dist)
                  for s in tp.LLAMA2_7B_LAYER)
    stack = tp.DecodeLinearStack(3, 16, 0.638, dev, world, rank, seed=11, allreduce="in_kernel", specs=small, fuse_shared_inputs=True)
    par = stack.parity_check(layers=3)
    lst = stack.make_list(select=True, sharded_select=True)
    for o in [it[3] for it in stack.items]:
        o.fill_(float("nan"))
    for _ in range(2):
        lst.run()
    torch.cuda.synchronize()
    par_sh = stack.parity_check_outputs(layers=3)
    status = lst.read_status()
    if status != 0 or not par["max_err"] <= TOL or not par_sh["max_err"] <= TOL:
        failures.append(("uneven shards, sharded selection", hex(status), par, par_sh))
    lst.close()
    stack.close()
    # Shards of unequal size, as eight ranks get them from the 7B shapes (43 column groups and 43 blocks
    # over two ranks: 21 / 22), and a rank whose K-shard of o_proj holds no active block at all: it
    # still has to send its zeros for every tile.
    small = tuple(tp.LinearSpec(s.name, {4096: 1024, 11008: 2752}[s.n], {4096: 1024, 11008: 2752}[s.k], s.parallel, s.dist)
                  for s in tp.LLAMA2_7B_LAYER)
    stack = tp.DecodeLinearStack(2, 16, 0.638, dev, world, rank, seed=7, allreduce="in_kernel", specs=small)
    bm_o = stack._shared["o_proj"][1]
    keep = int(bm_o.sum())
    bm_o.zero_()
    bm_o[:keep] = 1                       # all active blocks in the first ranks' shards
    par = stack.parity_check(layers=2)
    lst = stack.make_list()
    for o in [it[3] for it in stack.items]:
        o.fill_(float("nan"))
    for _ in range(3):
        lst.run()
    torch.cuda.synchronize()
    par_list = stack.parity_check_outputs(layers=2)
    status = lst.read_status()            # reading clears it
    if status != 0 or not par["max_err"] <= TOL or not par_list["max_err"] <= TOL or not par_list["ids_equal"]:
        failures.append(("uneven shards as a list", hex(status), par, par_list))
        print(f"rank {rank}: uneven shards as a list: status {status:#x}", flush=True)
    lst.close()
    stack.close()
    lgroup.close()
    # A rank that stays away: every rank but rank 0 leaves out one call (between steps, nothing of its
    # own in flight).  Rank 0's kernel sends its words, polls for the others' with a bound of a few
    # milliseconds, gives up, reports BAS_DEV_WAIT_EXPIRED through the status word and returns: an error
    # code, not a hang.  The group's call counters are out of step afterwards, so it is destroyed.
    from bas import abi
    late = ops.ExchangeGroup(dev, 16, 4096)
    x_h, w_h = O.make_activations(16, 1024, seed=900), O.make_weight(4096, 1024, seed=901)
    b0, b1 = tp.row_shard_blocks(1024, world, rank)
    x = torch.from_numpy(x_h).to(dev)[:, b0 * 64:b1 * 64]
    packed = ops.pack_weight(torch.from_numpy(np.ascontiguousarray(w_h[:, b0 * 64:b1 * 64])).to(dev))
    ids = torch.arange(b1 - b0, dtype=torch.int32, device=dev)
    out = torch.full((16, 4096), float("nan"), dtype=torch.float16, device=dev)
    ops.gemm(x, packed, out, ids=ids, tp=late)                    # everybody: a complete call
    torch.cuda.synchronize()
    err = O.max_err_ratio(out.float().cpu().numpy(), O.masked_gemm(x_h, w_h, np.arange(16, dtype=np.int32)))
    if ops.read_status(dev) != 0 or not err <= TOL:
        failures.append(("late group, first call", err))
    dist.barrier()
    if rank == 0:
        abi.check(abi.lib.bas_set_wait_ms(5.0), "bas_set_wait_ms")
        out.fill_(float("nan"))
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        ops.gemm(x, packed, out, ids=ids, tp=late)                # the others never make this call
        t1.record()
        torch.cuda.synchronize()
        status = ops.read_status(dev)
        abi.check(abi.lib.bas_set_wait_ms(1000.0), "bas_set_wait_ms")
        if not (status & abi.DEV_WAIT_EXPIRED) or t0.elapsed_time(t1) > 2000.0 or not bool(torch.isnan(out).all()):
            failures.append(("expiry", status, t0.elapsed_time(t1), int(torch.isnan(out).sum())))
    dist.barrier()
    late.close()
    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    if rank == 0:
        print("TP_IN_KERNEL_SUM", "OK" if int(flag.item()) == 0 else f"FAILED {failures}", flush=True)
    dist.destroy_process_group()
    sys.exit(0 if int(flag.item()) == 0 else 1)


if __name__ == "__main__":
    main()
