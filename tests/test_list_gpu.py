"""GPU parity of the list kernel (bas_list_*): a sequence of masked contractions run as one
persistent launch, through the C ABI, against the CPU oracle - chains whose activations are the
previous call's output, the Llama layer's seven shapes with the model's dependencies, ragged
and narrow shapes, every form of the active set, repeated runs and CUDA-graph replays, and the
expiry path of its bounded waits (made to run out by a dependency that is never reported)."""

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import bas_oracle as O  # noqa: E402

TOL = 2e-3   # max|y - ref| / max|ref|, the parity rule of the benchmark specification


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)


def _ops():
    from bas import ops
    return ops


def _chain(dev, batch, dims, keeps, seed, cluster=0, pairs=0, max_ctas=0, runs=1, form="ids", dtype=None):
    """x0 [batch, dims[0]] -> W0 -> y0 = x1 -> W1 -> ...: every call reads the output of the call before
    it.  Each stage is checked against the oracle applied to the DEVICE's own input of that stage, so
    the tolerance is the single-call one."""
    ops = _ops()
    x0 = O.make_activations(batch, dims[0], seed=seed)
    ws = [O.make_weight(dims[i + 1], dims[i], seed=seed + 10 + i, std=1.0 / np.sqrt(dims[i] * keeps[i] / ((dims[i] + 63) // 64)))
          for i in range(len(dims) - 1)]
    idl = [O.random_active_blocks((dims[i] + 63) // 64, keeps[i], seed=seed + 20 + i) for i in range(len(dims) - 1)]
    tdt = torch.float16 if dtype is None else dtype
    bufs = [torch.from_numpy(x0).to(dev).to(tdt)]
    for i in range(len(dims) - 1):
        # row stride padded to a multiple of 8 elements so that the buffer can be the next call's input
        ld = (dims[i + 1] + 7) // 8 * 8
        bufs.append(torch.full((batch, ld), float("nan"), dtype=tdt, device=dev)[:, :dims[i + 1]])
    calls = []
    for i in range(len(dims) - 1):
        wt = torch.from_numpy(ws[i]).to(dev).to(tdt)
        ws[i] = wt.float().cpu().numpy()          # the weights as the device holds them
        c = {"x": bufs[i], "packed": ops.pack_weight(wt), "out": bufs[i + 1], "depends_on": i - 1}
        nb = (dims[i] + 63) // 64
        if form == "bitmap":
            bm = np.zeros(nb, np.uint8)
            bm[idl[i]] = 1
            c["bitmap"] = torch.from_numpy(bm).to(dev)
            c["k_host"] = len(idl[i])
        elif form == "count":
            padded = np.concatenate([idl[i], np.full(3, nb - 1, np.int32)]).astype(np.int32)
            c["ids"] = torch.from_numpy(padded).to(dev)
            c["count"] = torch.tensor([len(idl[i])], dtype=torch.int32, device=dev)
            c["k_host"] = len(padded)
        else:
            c["ids"] = torch.from_numpy(np.ascontiguousarray(idl[i], dtype=np.int32)).to(dev)
        calls.append(c)
    lst = ops.GemmList(calls, cluster=cluster, pairs=pairs, max_ctas=max_ctas)
    outs = []
    for _ in range(runs):
        for b in bufs[1:]:
            b.fill_(float("nan"))
        lst.run()
        torch.cuda.synchronize()
        assert lst.read_status() == 0
        outs.append([b.float().cpu().numpy() for b in bufs])
    info = lst.info()
    lst.close()
    for got in outs:
        for i in range(len(dims) - 1):
            x_in = got[i].astype(np.float32)
            mask = np.zeros(((dims[i] + 63) // 64) * 64, np.float32)
            for j in idl[i]:
                mask[j * 64:(j + 1) * 64] = 1
            ref = (x_in * mask[:dims[i]]) @ ws[i].astype(np.float32).T
            assert np.isfinite(got[i + 1]).all(), f"stage {i}: non-finite output"
            err = O.max_err_ratio(got[i + 1], ref)
            tol = TOL if dtype is None else 2.0 ** -7
            assert err <= tol, f"stage {i} ({dims[i]}->{dims[i + 1]}, batch {batch}, {info}): err ratio {err:.3e}"
    for got in outs[1:]:
        for a, b in zip(got, outs[0]):
            assert np.array_equal(a, b), "a repeated run changed the result"
    return info


@pytest.mark.parametrize("batch", [1, 2, 16, 17, 33, 64])
def test_dependent_chain_matches_oracle(dev, batch):
    _chain(dev, batch, [1024, 4096, 512, 2048, 1024], [9, 30, 5, 20], seed=batch, runs=3)


@pytest.mark.parametrize("cluster", [1, 2, 4])
@pytest.mark.parametrize("batch", [16, 64])
def test_chain_with_every_cluster_size(dev, batch, cluster):
    info = _chain(dev, batch, [2048, 4096, 11008, 4096], [17, 23, 62], seed=7 + cluster, cluster=cluster, runs=2)
    assert info["cluster"] == cluster


@pytest.mark.parametrize("pairs", [2, 3, 4])
def test_chain_with_every_pair_count(dev, pairs):
    _chain(dev, 16, [4096, 4096, 11008, 4096], [23, 23, 62], seed=40 + pairs, pairs=pairs, runs=2)


@pytest.mark.parametrize("form", ["bitmap", "count"])
def test_chain_with_byte_maps_and_device_counts(dev, form):
    _chain(dev, 16, [2048, 1024, 4096, 1024], [11, 7, 30], seed=60, form=form, runs=2)


def test_chain_with_ragged_and_narrow_shapes(dev):
    # K not a multiple of 64 (the last block is partial), N not a multiple of 8, outputs narrower than
    # one cluster's usual share
    _chain(dev, 5, [1000, 200, 520, 72, 264, 136], [9, 3, 6, 2, 4], seed=70, runs=2)
    _chain(dev, 20, [520, 96, 4104, 40], [5, 2, 33], seed=71, runs=2)


def test_chain_with_capped_grid(dev):
    _chain(dev, 16, [4096, 4096, 2048], [23, 40], seed=80, max_ctas=24, runs=2)


def test_chain_bf16(dev):
    _chain(dev, 16, [2048, 4096, 1024], [17, 40], seed=90, runs=2, dtype=torch.bfloat16)


def test_llama_layer_with_model_dependencies(dev):
    """q, k, v <- x; o <- v; gate, up <- o; down <- up; two layers, q of the second <- down of the
    first.  Every output against the oracle and against the single-call entry point."""
    ops = _ops()
    b = 16
    shapes = [("q", 4096, 4096), ("k", 4096, 4096), ("v", 4096, 4096), ("o", 4096, 4096), ("gate", 11008, 4096),
              ("up", 11008, 4096), ("down", 4096, 11008)]
    deps = {"q": "down", "k": "down", "v": "down", "o": "v", "gate": "o", "up": "o", "down": "up"}
    calls, meta, index = [], [], {}
    for layer in range(2):
        for name, n, k in shapes:
            seed = layer * 100 + len(calls)
            x = O.make_activations(b, k, seed=seed, dist="laplace" if name == "down" else "normal")
            w = O.make_weight(n, k, seed=seed + 1)
            nb = k // 64
            ids = O.random_active_blocks(nb, O.n_keep_from_density(0.362, nb), seed=seed + 2)
            tx, tw = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
            out = torch.full((b, n), float("nan"), dtype=torch.float16, device=dev)
            dep = index.get((layer, deps[name]), index.get((layer - 1, deps[name]), -1))
            index[(layer, name)] = len(calls)
            calls.append({"x": tx, "packed": ops.pack_weight(tw), "out": out, "depends_on": dep,
                          "ids": torch.from_numpy(ids).to(dev)})
            meta.append((x, w, ids))
    lst = ops.GemmList(calls)
    g = torch.cuda.CUDAGraph()
    lst.run()
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    with torch.cuda.graph(g, stream=s):
        lst.run()
    for c in calls:
        c["out"].fill_(float("nan"))
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert lst.read_status() == 0
    for c, (x, w, ids) in zip(calls, meta):
        ref = O.masked_gemm(x, w, ids)
        y = c["out"].cpu().numpy()
        assert O.max_err_ratio(y, ref) <= TOL
        single = torch.empty_like(c["out"])
        ops.gemm(c["x"], c["packed"], single, ids=c["ids"])
        torch.cuda.synchronize()
        assert O.max_err_ratio(y, single.float().cpu().numpy()) <= 1e-3
    lst.close()


def test_empty_sets_and_bad_ids(dev):
    ops = _ops()
    b, k, n = 16, 1024, 512
    x = torch.from_numpy(O.make_activations(b, k, seed=1)).to(dev)
    w = O.make_weight(n, k, seed=2)
    packed = ops.pack_weight(torch.from_numpy(w).to(dev))
    out_empty = torch.full((b, n), float("nan"), dtype=torch.float16, device=dev)
    out_bad = torch.full((b, n), float("nan"), dtype=torch.float16, device=dev)
    zero_map = torch.zeros(k // 64, dtype=torch.uint8, device=dev)
    ids_bad = torch.tensor([3, 99, 5, -2], dtype=torch.int32, device=dev)
    lst = ops.GemmList([{"x": x, "packed": packed, "out": out_empty, "bitmap": zero_map},
                        {"x": x, "packed": packed, "out": out_bad, "ids": ids_bad}])
    lst.run()
    torch.cuda.synchronize()
    from bas import abi
    assert lst.read_status() == abi.DEV_BAD_BLOCK_ID
    assert float(out_empty.float().abs().max()) == 0.0
    ref = O.masked_gemm(x.cpu().numpy(), w, np.array([3, 5], np.int32))
    assert O.max_err_ratio(out_bad.cpu().numpy(), ref) <= TOL
    lst.close()


def test_argument_checks(dev):
    ops = _ops()
    from bas import BasError
    x = torch.zeros(4, 128, dtype=torch.float16, device=dev)
    packed = ops.pack_weight(torch.zeros(64, 128, dtype=torch.float16, device=dev))
    out = torch.zeros(4, 64, dtype=torch.float16, device=dev)
    ids = torch.zeros(1, dtype=torch.int32, device=dev)
    with pytest.raises(BasError):      # a call may only depend on an earlier one
        ops.GemmList([{"x": x, "packed": packed, "out": out, "ids": ids, "depends_on": 0}])
    with pytest.raises(BasError):      # more ids than blocks
        ops.GemmList([{"x": x, "packed": packed, "out": out, "ids": torch.zeros(5, dtype=torch.int32, device=dev)}])
    with pytest.raises(ValueError):
        ops.GemmList([])


def test_wait_that_runs_out_is_reported_and_the_list_recovers(dev):
    """The second call's dependency is never reported complete (a switch of the list, for this test):
    its activation copies wait, the bound (a few milliseconds here) runs out, the kernel returns with
    BAS_DEV_WAIT_EXPIRED in the status word - nothing traps or spins for ever - and after a reset the
    same list computes the right result."""
    ops = _ops()
    from bas import abi
    b = 16
    x0 = O.make_activations(b, 1024, seed=5)
    w0, w1 = O.make_weight(2048, 1024, seed=6, std=0.05), O.make_weight(512, 2048, seed=7, std=0.05)
    i0, i1 = O.random_active_blocks(16, 9, seed=8), O.random_active_blocks(32, 20, seed=9)
    tx = torch.from_numpy(x0).to(dev)
    mid = torch.zeros(b, 2048, dtype=torch.float16, device=dev)
    out = torch.zeros(b, 512, dtype=torch.float16, device=dev)
    lst = ops.GemmList([
        {"x": tx, "packed": ops.pack_weight(torch.from_numpy(w0).to(dev)), "out": mid, "ids": torch.from_numpy(i0).to(dev)},
        {"x": mid, "packed": ops.pack_weight(torch.from_numpy(w1).to(dev)), "out": out, "ids": torch.from_numpy(i1).to(dev),
         "depends_on": 0}])
    lst.set_wait(5.0, never_ready_call=1)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    lst.run()
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 2000.0           # bounded: a handful of 5 ms waits, not a hang
    assert lst.read_status() & abi.DEV_WAIT_EXPIRED
    lst.reset()
    lst.set_wait(1000.0, never_ready_call=-1)
    for _ in range(2):
        lst.run()
    torch.cuda.synchronize()
    assert lst.read_status() == 0
    ref_mid = O.masked_gemm(x0, w0, i0)
    assert O.max_err_ratio(mid.cpu().numpy(), ref_mid) <= TOL
    ref = O.masked_gemm(mid.cpu().numpy(), w1, i1)
    assert O.max_err_ratio(out.cpu().numpy(), ref) <= TOL
    lst.close()
