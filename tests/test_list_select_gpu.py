"""GPU parity of selection inside the list kernel: entries that score the blocks of an activation as
part of the launch, and contractions that rank those scores at their call boundary and run with the
kept blocks.  The ids must equal the oracle's top-k (score descending, id ascending; NaN first) bit for
bit - the rule of scripts/bench_roundrobin_e2e_decode.py:90-113 - and bas_select_topk's own; the outputs
must equal the oracle's masked product of the device's own input."""

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import bas_oracle as O  # noqa: E402

TOL = 2e-3   # max|y - ref| / max|ref|
TOL_BF16 = 2.0 ** -7   # an output rounded to 8 significant bits


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)


def _ops():
    from bas import ops
    return ops


def _masked_ref(x, w, ids):
    mask = np.zeros(x.shape[1], np.float32)
    for j in ids:
        mask[j * 64:(j + 1) * 64] = 1
    return (x.astype(np.float32) * mask) @ w.astype(np.float32).T


def _select_and_multiply(dev, x_h, n, n_keep, score_kind, seed, dtype=torch.float16, runs=1, consumers=1):
    """[select(x), gemm(x, mask_from=0) x consumers] as one launch; returns the ids per run."""
    ops = _ops()
    batch, k = x_h.shape
    x = torch.from_numpy(x_h).to(dev).to(dtype)
    calls = [{"select": x, "n_keep": n_keep, "score_kind": score_kind}]
    ws, outs, idbufs = [], [], []
    for q in range(consumers):
        w = torch.from_numpy(O.make_weight(n, k, seed=seed + q)).to(dev).to(dtype)
        ws.append(w)
        outs.append(torch.full((batch, n), float("nan"), dtype=dtype, device=dev))
        idbufs.append(torch.full((max(n_keep, 1),), -1, dtype=torch.int32, device=dev))
        calls.append({"x": x, "packed": ops.pack_weight(w), "out": outs[-1], "mask_from": 0, "ids_out": idbufs[-1]})
    lst = ops.GemmList(calls)
    got = []
    for _ in range(runs):
        for o in outs:
            o.fill_(float("nan"))
        lst.run()
        torch.cuda.synchronize()
        assert lst.read_status() == 0
        ids = idbufs[0].cpu().numpy()[:n_keep]
        for ib in idbufs[1:]:
            assert np.array_equal(ib.cpu().numpy()[:n_keep], ids)
        x_dev = x.float().cpu().numpy()
        for w, o in zip(ws, outs):
            ref = _masked_ref(x_dev, w.float().cpu().numpy(), ids)
            if n_keep == 0:
                assert not np.any(o.float().cpu().numpy())
            elif np.isfinite(ref).all():     # inputs with NaN / inf are checked on the ids alone
                assert O.max_err_ratio(o.float().cpu().numpy(), ref) <= (TOL_BF16 if dtype == torch.bfloat16 else TOL)
        got.append(ids)
    lst.close()
    return got


@pytest.mark.parametrize("batch,k,n,n_keep,kind", [
    (16, 11008, 4096, 62, "norm"), (2, 11008, 4096, 34, "norm"), (64, 11008, 4096, 83, "energy"),
    (1, 4096, 4096, 23, "norm"), (16, 4096, 11008, 23, "energy"), (7, 704, 200, 5, "norm"),
    (16, 64, 64, 1, "norm"), (33, 2752, 1024, 43, "norm"), (16, 4096, 512, 0, "norm"), (16, 21952, 256, 100, "energy")])
def test_ids_equal_the_oracle_and_the_selection_kernel(dev, batch, k, n, n_keep, kind):
    ops = _ops()
    from bas import abi
    sk = abi.SCORE_NORM if kind == "norm" else abi.SCORE_ENERGY
    x_h = O.make_activations(batch, k, seed=batch * 1000 + k, dist="laplace")
    got = _select_and_multiply(dev, x_h, n, n_keep, sk, seed=5, runs=2)
    want = O.topk_ids(O.block_scores(x_h, sk), n_keep)
    ids_k, _ = ops.select_topk(torch.from_numpy(x_h).to(dev), n_keep, sk)
    for ids in got:
        assert np.array_equal(ids, np.asarray(want, dtype=np.int32))
        assert np.array_equal(ids, ids_k.cpu().numpy()[:n_keep])


def test_ties_go_to_the_lower_id(dev):
    # blocks 3, 40 and 41 are copies of block 7: equal scores to the last bit; with 7 the boundary of the
    # top-k, the kept set has to take the lower ids first
    from bas import abi
    x_h = O.make_activations(16, 4096, seed=77) * 0.01
    x_h[:, 7 * 64:8 * 64] = O.make_activations(16, 64, seed=78)
    for j in (3, 40, 41):
        x_h[:, j * 64:(j + 1) * 64] = x_h[:, 7 * 64:8 * 64]
    scores = O.block_scores(x_h, O.SCORE_NORM)
    assert scores[3] == scores[7] == scores[40] == scores[41]
    for n_keep in (1, 2, 3, 4, 5):
        got = _select_and_multiply(dev, x_h, 256, n_keep, abi.SCORE_NORM, seed=9)[0]
        assert np.array_equal(got, np.asarray(O.topk_ids(scores, n_keep), dtype=np.int32))
        assert set([3, 7, 40, 41][:min(n_keep, 4)]) <= set(int(v) for v in got)


def test_all_equal_scores_keep_the_first_blocks(dev):
    from bas import abi
    x_h = np.ones((16, 11008), np.float16)
    got = _select_and_multiply(dev, x_h, 128, 62, abi.SCORE_ENERGY, seed=3)[0]
    assert np.array_equal(got, np.arange(62, dtype=np.int32))


def test_non_finite_activations_rank_like_torch_topk(dev):
    from bas import abi
    x_h = O.make_activations(16, 4096, seed=31)
    x_h[3, 5 * 64 + 2] = np.nan
    x_h[0, 17 * 64] = np.inf
    x_h[1, 60 * 64 + 63] = np.nan
    got = _select_and_multiply(dev, x_h, 128, 4, abi.SCORE_NORM, seed=3)[0]
    with np.errstate(all="ignore"):
        want = O.topk_ids(O.block_scores(x_h, O.SCORE_NORM), 4)
    assert np.array_equal(got, np.asarray(want, dtype=np.int32))
    assert {5, 17, 60} <= set(int(v) for v in got)


def test_bf16_and_shared_masks(dev):
    # three contractions (q, k, v) run with one entry's mask
    from bas import abi
    x_h = O.make_activations(16, 4096, seed=41)
    got = _select_and_multiply(dev, x_h, 1024, 23, abi.SCORE_NORM, seed=50, dtype=torch.bfloat16, consumers=3)[0]
    x_b = torch.from_numpy(x_h).to(torch.bfloat16).float().numpy()
    assert np.array_equal(got, np.asarray(O.topk_ids(O.block_scores(x_b, O.SCORE_NORM), 23), dtype=np.int32))


def test_golden_selections_of_the_reference(dev, golden):
    # the selections recorded from the reference's own Python (inputs regenerated from their seeds)
    from bas import abi
    data, meta = golden
    checked = 0
    for ci, c in enumerate(meta["select"]):
        if c["k"] % 64:
            continue
        x_h = O.make_activations(c["batch"], c["k"], c["seed"], c["dist"])
        n_keep = O.n_keep_from_density(c["density"], c["k"] // 64)
        for sk, name in ((abi.SCORE_NORM, "norm"), (abi.SCORE_ENERGY, "energy")):
            got = _select_and_multiply(dev, x_h, 128, n_keep, sk, seed=1)[0]
            assert np.array_equal(got, data[f"select{ci}_{name}_ids"]), f"case {ci} {name}"
            checked += 1
    assert checked >= 22


@pytest.mark.parametrize("max_ctas,pairs", [(0, 0), (3, 0), (8, 2), (50, 3)])
def test_chain_with_fresh_masks(dev, max_ctas, pairs):
    """x0 -> [select, W0] -> x1 -> [select, W1] -> x2 -> [select, W2]: every mask is computed inside the launch
    from an activation that the launch itself produced.  Also on grids far smaller than the GPU (every CTA then
    scores many blocks and walks many column ranges) and with fewer copy warps."""
    ops = _ops()
    from bas import abi
    batch, dims, keeps = 16, [4096, 2752, 1024, 4096], [23, 16, 6]
    x0 = O.make_activations(batch, dims[0], seed=90)
    bufs = [torch.from_numpy(x0).to(dev)]
    calls, ws, idbufs = [], [], []
    for i in range(3):
        w = torch.from_numpy(O.make_weight(dims[i + 1], dims[i], seed=91 + i, std=1.0 / np.sqrt(64 * keeps[i]))).to(dev)
        ws.append(w)
        bufs.append(torch.full((batch, dims[i + 1]), float("nan"), dtype=torch.float16, device=dev))
        idbufs.append(torch.full((keeps[i],), -1, dtype=torch.int32, device=dev))
        dep = 2 * i - 1            # the contraction of the stage before (entries alternate select, contraction)
        calls.append({"select": bufs[i], "n_keep": keeps[i], "score_kind": abi.SCORE_NORM, "depends_on": dep})
        calls.append({"x": bufs[i], "packed": ops.pack_weight(w), "out": bufs[i + 1], "mask_from": 2 * i,
                      "ids_out": idbufs[i], "depends_on": dep})
    lst = ops.GemmList(calls, max_ctas=max_ctas, pairs=pairs)
    g = None
    for run in range(4):
        for b in bufs[1:]:
            b.fill_(float("nan"))
        if run < 2:
            lst.run()
        else:                       # replays of a captured launch
            if g is None:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    lst.run()
            g.replay()
        torch.cuda.synchronize()
        assert lst.read_status() == 0
        for i in range(3):
            x_in = bufs[i].float().cpu().numpy()
            want = O.topk_ids(O.block_scores(x_in.astype(np.float16), O.SCORE_NORM), keeps[i])
            ids = idbufs[i].cpu().numpy()
            assert np.array_equal(ids, np.asarray(want, dtype=np.int32)), (run, i)
            ref = _masked_ref(x_in, ws[i].float().cpu().numpy(), ids)
            assert O.max_err_ratio(bufs[i + 1].float().cpu().numpy(), ref) <= TOL
    lst.close()


def test_a_k_shard_takes_its_part_of_the_mask(dev):
    ops = _ops()
    from bas import abi
    batch, k, n, n_keep = 16, 2752, 512, 16
    x_h = O.make_activations(batch, k, seed=120, dist="laplace")
    w_h = O.make_weight(n, k, seed=121)
    x = torch.from_numpy(x_h).to(dev)
    want = np.asarray(O.topk_ids(O.block_scores(x_h, O.SCORE_NORM), n_keep), dtype=np.int32)
    calls = [{"select": x, "n_keep": n_keep, "score_kind": abi.SCORE_NORM}]
    outs, bounds = [], [(0, 21), (21, 43), (40, 43)]
    for b0, b1 in bounds:
        w = torch.from_numpy(np.ascontiguousarray(w_h[:, b0 * 64:b1 * 64])).to(dev)
        outs.append(torch.full((batch, n), float("nan"), dtype=torch.float16, device=dev))
        calls.append({"x": x[:, b0 * 64:b1 * 64], "packed": ops.pack_weight(w), "out": outs[-1], "mask_from": 0, "mask_block0": b0})
    lst = ops.GemmList(calls)
    lst.run()
    torch.cuda.synchronize()
    assert lst.read_status() == 0
    lst.close()
    for (b0, b1), o in zip(bounds, outs):
        ids = [j for j in want if b0 <= j < b1]
        ref = _masked_ref(x_h, w_h, ids)
        got = o.float().cpu().numpy()
        if ids:
            assert O.max_err_ratio(got, ref) <= TOL
        else:
            assert not np.any(got)


def test_argument_checks(dev):
    ops = _ops()
    from bas import abi
    x = torch.zeros(16, 4096, dtype=torch.float16, device=dev)
    w = ops.pack_weight(torch.zeros(256, 4096, dtype=torch.float16, device=dev))
    out = torch.zeros(16, 256, dtype=torch.float16, device=dev)
    sel = {"select": x, "n_keep": 8, "score_kind": abi.SCORE_NORM}
    gemm = {"x": x, "packed": w, "out": out, "mask_from": 0}
    with pytest.raises(abi.BasError):                       # the entry must come first
        ops.GemmList([dict(gemm), dict(sel)])
    with pytest.raises(abi.BasError):                       # a mask from a contraction
        ops.GemmList([dict(sel), dict(gemm), dict(gemm, mask_from=1)])
    with pytest.raises(abi.BasError):                       # more blocks than the entry has
        ops.GemmList([dict(sel), dict(gemm, mask_block0=1)])
    with pytest.raises(abi.BasError):                       # keeps more than there are
        ops.GemmList([dict(sel, n_keep=65), dict(gemm)])
    with pytest.raises(abi.BasError):                       # different dependency than its entry
        ops.GemmList([dict(gemm, mask_from=None, ids=torch.arange(4, dtype=torch.int32, device=dev)), dict(sel),
                      dict(gemm, mask_from=1, depends_on=0)])
    with pytest.raises(abi.BasError):                       # a list of entries alone
        ops.GemmList([dict(sel)])
    with pytest.raises(abi.BasError):                       # clusters
        ops.GemmList([dict(sel), dict(gemm)], cluster=2)
