"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle and the golden
vectors recorded from the reference.  Bit-exact for ids, bitmaps and the packed layout;
max|dY| <= 2e-3 * max|Y_ref| for the fp16-in / fp32-accumulate contraction."""

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


def _run_gemm(dev, x, w, ids=None, bitmap=None, family=0, count=None, k_host=None, ids_stable=False, cluster=0,
              pairs=0):
    ops = _ops()
    tx, tw = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
    packed = ops.pack_weight(tw)
    out = torch.full((x.shape[0], w.shape[0]), float("nan"), dtype=torch.float16, device=dev)
    kw = {}
    if bitmap is not None:
        kw["bitmap"] = torch.from_numpy(bitmap).to(dev)
        if k_host is not None:
            kw["k_host"] = k_host
    else:
        kw["ids"] = torch.from_numpy(np.ascontiguousarray(ids, dtype=np.int32)).to(dev)
        if count is not None:
            kw["count"] = torch.tensor([count], dtype=torch.int32, device=dev)
            kw["k_host"] = k_host
    ops.gemm(tx, packed, out, family=family, ids_stable=ids_stable, cluster=cluster, pairs=pairs, **kw)
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 0
    return out.cpu().numpy()


# ---------------------------------------------------------------------------------------------
# prepack
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("n,k", [(128, 64), (96, 200), (300, 520), (203, 203), (4096, 4096)])
def test_pack_is_bit_exact(dev, n, k):
    w = O.make_weight(n, k, seed=n + k)
    packed = _ops().pack_weight(torch.from_numpy(w).to(dev)).cpu().numpy()
    want = O.pack_weight_blocks(w)
    assert packed.nbytes == want.nbytes
    assert np.array_equal(packed.view(np.float16).reshape(want.shape), want)


def test_pack_accepts_strided_rows(dev):
    w = O.make_weight(130, 256, seed=3)
    big = torch.zeros(130, 300, dtype=torch.float16, device=dev)
    big[:, :256] = torch.from_numpy(w).to(dev)
    packed = _ops().pack_weight(big[:, :256]).cpu().numpy()
    assert np.array_equal(packed.view(np.float16).reshape(4, 136, 64), O.pack_weight_blocks(w))


# ---------------------------------------------------------------------------------------------
# contraction
# ---------------------------------------------------------------------------------------------

SMALL = [(b, 1024, 512, nk) for b in (1, 2, 3, 4, 5, 8, 9, 16, 17, 32, 33, 48, 64) for nk in (1, 7, 16)]
RAGGED = [(3, 200, 96, 3), (16, 200, 96, 4), (2, 72, 40, 2), (20, 136, 130, 3), (1, 64, 128, 1), (64, 64, 8, 1)]
LLAMA = [(2, 11008, 4096, 34), (16, 11008, 4096, 62), (64, 11008, 4096, 83), (16, 4096, 4096, 32),
         (4, 4096, 11008, 13), (32, 4096, 11008, 51), (8, 11008, 4096, 51), (1, 4096, 4096, 64)]


@pytest.mark.parametrize("b,k,n,n_keep", SMALL + RAGGED + LLAMA)
def test_gemm_matches_oracle(dev, b, k, n, n_keep):
    nb = (k + 63) // 64
    x = O.make_activations(b, k, seed=b * 1000 + n_keep, dist="laplace" if k == 11008 else "normal")
    w = O.make_weight(n, k, seed=k + n, std=0.02 if k >= 4096 else 0.05)
    ids = O.random_active_blocks(nb, min(n_keep, nb), seed=b + k)
    y = _run_gemm(dev, x, w, ids=ids)
    ref = O.masked_gemm(x, w, ids)
    assert np.isfinite(y).all()
    err = O.max_err_ratio(y, ref)
    assert err <= TOL, f"B={b} K={k} N={n} keep={n_keep}: err ratio {err:.3e}"


@pytest.mark.parametrize("b", [1, 2, 4, 8])
def test_small_batches_agree_on_both_kernel_families(dev, b):
    x = O.make_activations(b, 2048, seed=b)
    w = O.make_weight(640, 2048, seed=9)
    ids = O.random_active_blocks(32, 11, seed=b)
    ref = O.masked_gemm(x, w, ids)
    y1 = _run_gemm(dev, x, w, ids=ids, family=1)
    y2 = _run_gemm(dev, x, w, ids=ids, family=2)
    assert O.max_err_ratio(y1, ref) <= TOL and O.max_err_ratio(y2, ref) <= TOL
    assert O.max_err_ratio(y1, y2.astype(np.float32)) <= 1e-3


@pytest.mark.parametrize("b", [9, 16, 33, 64])
@pytest.mark.parametrize("cluster", [1, 2, 4])
def test_cluster_sizes_agree(dev, b, cluster):
    """The tcgen05 kernel with the active blocks split over 1, 2 or 4 CTAs per column range."""
    x = O.make_activations(b, 11008, seed=b, dist="laplace")
    w = O.make_weight(4096, 11008, seed=2)
    for n_keep in (1, 3, 62):
        ids = O.random_active_blocks(172, n_keep, seed=b + n_keep)
        y = _run_gemm(dev, x, w, ids=ids, cluster=cluster)
        assert O.max_err_ratio(y, O.masked_gemm(x, w, ids)) <= TOL


@pytest.mark.parametrize("pairs", [2, 3, 4])
@pytest.mark.parametrize("b,k,n,cluster", [(16, 11008, 4096, 0), (64, 11008, 4096, 0), (5, 4096, 11008, 0),
                                           (16, 512, 24000, 1), (48, 1024, 20000, 1)])
def test_pair_counts_agree(dev, b, k, n, cluster, pairs):
    """2, 3 or 4 copy/MMA warp pairs sharing the ring, in cluster mode and with several sub-tiles
    per CTA (groups that straddle sub-tile boundaries)."""
    x = O.make_activations(b, k, seed=b + pairs, dist="laplace")
    w = O.make_weight(n, k, seed=4)
    nb = k // 64
    for n_keep in sorted({1, 2, 5, nb // 3, nb}):
        ids = O.random_active_blocks(nb, n_keep, seed=b + n_keep)
        y = _run_gemm(dev, x, w, ids=ids, cluster=cluster, pairs=pairs, ids_stable=bool(n_keep & 1))
        assert O.max_err_ratio(y, O.masked_gemm(x, w, ids)) <= TOL


@pytest.mark.parametrize("b,n", [(2, 24000), (16, 24000), (64, 20000)])
def test_wide_outputs_use_several_sub_tiles(dev, b, n):
    """More than 128 columns per CTA: the column range is walked in sub-tiles."""
    x = O.make_activations(b, 512, seed=b)
    w = O.make_weight(n, 512, seed=3)
    ids = O.random_active_blocks(8, 5, seed=b)
    y = _run_gemm(dev, x, w, ids=ids)
    assert O.max_err_ratio(y, O.masked_gemm(x, w, ids)) <= TOL


@pytest.mark.parametrize("b", [2, 16])
def test_unsorted_ids_and_bitmap_give_the_same_sum(dev, b):
    x = O.make_activations(b, 4096, seed=5)
    w = O.make_weight(1024, 4096, seed=5)
    ids = O.random_active_blocks(64, 20, seed=1)
    ref = O.masked_gemm(x, w, ids)
    rng = np.random.default_rng(0)
    y_sorted = _run_gemm(dev, x, w, ids=ids)
    y_perm = _run_gemm(dev, x, w, ids=rng.permutation(ids))
    y_bitmap = _run_gemm(dev, x, w, bitmap=O.build_bitmap(ids, 64))
    y_bitmap_hint = _run_gemm(dev, x, w, bitmap=O.build_bitmap(ids, 64), k_host=20)
    for y in (y_sorted, y_perm, y_bitmap, y_bitmap_hint):
        assert O.max_err_ratio(y, ref) <= TOL
    # told how many blocks to expect, the byte-map call picks the same grid as the list call and
    # compacts to the same list: same bits
    assert np.array_equal(y_sorted, y_bitmap_hint)


@pytest.mark.parametrize("b", [2, 16])
def test_device_side_count_and_empty_set(dev, b):
    x = O.make_activations(b, 1024, seed=1)
    w = O.make_weight(256, 1024, seed=1)
    ids = O.random_active_blocks(16, 9, seed=2)
    # only the first 5 ids count; the rest of the buffer is ignored
    y = _run_gemm(dev, x, w, ids=ids, count=5, k_host=9)
    assert O.max_err_ratio(y, O.masked_gemm(x, w, ids[:5])) <= TOL
    # device-side count of zero and an all-zero bitmap both write zeros
    assert not _run_gemm(dev, x, w, ids=ids, count=0, k_host=9).any()
    assert not _run_gemm(dev, x, w, bitmap=np.zeros(16, np.uint8)).any()
    # host-side empty list
    assert not _run_gemm(dev, x, w, ids=ids[:0]).any()


@pytest.mark.parametrize("b", [2, 16])
def test_full_mask_equals_dense(dev, b):
    x = O.make_activations(b, 4096, seed=11)
    w = O.make_weight(4096, 4096, seed=11)
    y = _run_gemm(dev, x, w, ids=np.arange(64, dtype=np.int32))
    dense = (torch.from_numpy(x).to(dev).float() @ torch.from_numpy(w).to(dev).float().T).cpu().numpy()
    assert O.max_err_ratio(y, dense) <= TOL


@pytest.mark.parametrize("b", [2, 64])
def test_block_additivity_at_full_size(dev, b):
    """Y(A u B) = Y(A) + Y(B) for disjoint block sets: a size-independent property checked on the
    down-projection shape without running the CPU oracle at that size."""
    x = O.make_activations(b, 11008, seed=21, dist="laplace")
    w = O.make_weight(4096, 11008, seed=21)
    ids = O.random_active_blocks(172, 83, seed=3)
    ya = _run_gemm(dev, x, w, ids=ids[:40]).astype(np.float32)
    yb = _run_gemm(dev, x, w, ids=ids[40:]).astype(np.float32)
    yab = _run_gemm(dev, x, w, ids=ids).astype(np.float32)
    scale = np.abs(yab).max()
    assert np.abs(ya + yb - yab).max() <= 2e-3 * scale


@pytest.mark.parametrize("x_stable", [False, True])
@pytest.mark.parametrize("b", [2, 16, 64])
def test_back_to_back_launches_with_stable_ids(dev, b, x_stable):
    """Chained launches overlap (programmatic dependent launch); with stable ids the next kernel
    streams weights while the previous one drains, with stable X it also multiplies and waits
    only before it stores.  Every result must still be exact."""
    ops = _ops()
    k, n = 11008, 4096
    w = O.make_weight(n, k, seed=41)
    packed = ops.pack_weight(torch.from_numpy(w).to(dev))
    xs = [O.make_activations(b, k, seed=600 + i, dist="laplace") for i in range(4)]
    idl = [O.random_active_blocks(172, 40 + 10 * i, seed=i) for i in range(4)]
    txs = [torch.from_numpy(x).to(dev) for x in xs]
    tids = [torch.from_numpy(i).to(dev) for i in idl]
    outs = [torch.full((b, n), float("nan"), dtype=torch.float16, device=dev) for _ in range(4)]
    torch.cuda.synchronize()
    for rep in range(3):
        for i in range(4):
            ops.gemm(txs[i], packed, outs[i], ids=tids[i], ids_stable=True, x_stable=x_stable, next_independent=x_stable)
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 0
    for i in range(4):
        assert O.max_err_ratio(outs[i].cpu().numpy(), O.masked_gemm(xs[i], w, idl[i])) <= TOL


def test_stable_x_chain_writing_one_output(dev):
    """Calls that declare X stable still write Y in stream order: a chain of calls that all store
    to ONE output buffer (different active sets, different rows of work) leaves the last call's
    result, and a call whose output is a later call's input is ordered by leaving the flag off."""
    ops = _ops()
    b, k, n = 16, 4096, 4096
    w = O.make_weight(n, k, seed=51)
    packed = ops.pack_weight(torch.from_numpy(w).to(dev))
    x = O.make_activations(b, k, seed=52)
    tx = torch.from_numpy(x).to(dev)
    idl = [O.random_active_blocks(64, nk, seed=nk) for nk in (60, 5, 33, 12)]
    tids = [torch.from_numpy(i).to(dev) for i in idl]
    out = torch.full((b, n), float("nan"), dtype=torch.float16, device=dev)
    mid = torch.empty((b, n), dtype=torch.float16, device=dev)
    torch.cuda.synchronize()
    for i in range(4):
        ops.gemm(tx, packed, out, ids=tids[i], ids_stable=True, x_stable=True, next_independent=True)
    torch.cuda.synchronize()
    assert O.max_err_ratio(out.cpu().numpy(), O.masked_gemm(x, w, idl[3])) <= TOL
    # producer -> consumer: the second call reads what the first stored, so it does not set the flag
    ops.gemm(tx, packed, mid, ids=tids[0], ids_stable=True, x_stable=True)
    ops.gemm(mid, packed, out, ids=tids[2], ids_stable=True)
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 0
    y1 = mid.cpu().numpy()
    assert O.max_err_ratio(y1, O.masked_gemm(x, w, idl[0])) <= TOL
    assert O.max_err_ratio(out.cpu().numpy(), O.masked_gemm(y1, w, idl[2])) <= TOL


@pytest.mark.parametrize("b,k,n", [(16, 4096, 11008), (2, 4096, 2048), (64, 4096, 1024), (33, 1024, 4096 + 40),
                                   (32, 4096, 11008), (8, 2048, 12304), (48, 1024, 11008)])
def test_stable_x_chain_in_cuda_graph(dev, b, k, n):
    """A CUDA graph of eight calls that declare ids and X stable (the form the benchmark times), over
    output widths on both sides of the small-grid rule (wide outputs run two 128-column passes per CTA
    into separate accumulator columns up to 32 rows, one pass beyond), replayed twice: every output
    exact."""
    ops = _ops()
    w = O.make_weight(n, k, seed=61)
    packed = ops.pack_weight(torch.from_numpy(w).to(dev))
    nb = k // 64
    xs = [O.make_activations(b, k, seed=700 + i) for i in range(4)]
    idl = [O.random_active_blocks(nb, max(1, nb // 4 + 3 * i), seed=10 + i) for i in range(4)]
    txs = [torch.from_numpy(x).to(dev) for x in xs]
    tids = [torch.from_numpy(i).to(dev) for i in idl]
    outs = [torch.full((b, n), float("nan"), dtype=torch.float16, device=dev) for _ in range(4)]
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for i in range(4):      # warm-up outside the capture (tensor maps, function attributes)
            ops.gemm(txs[i], packed, outs[i], ids=tids[i], ids_stable=True, x_stable=True, next_independent=True)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        for rep in range(2):
            for i in range(4):
                ops.gemm(txs[i], packed, outs[i], ids=tids[i], ids_stable=True, x_stable=True, next_independent=True)
    for o in outs:
        o.fill_(float("nan"))
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        g.replay()
        g.replay()
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 0
    for i in range(4):
        assert O.max_err_ratio(outs[i].cpu().numpy(), O.masked_gemm(xs[i], w, idl[i])) <= TOL


@pytest.mark.parametrize("form", ["empty", "bitmap", "cluster2", "cluster4", "capped", "bf16", "count"])
def test_stable_x_variants(dev, form):
    """Calls that declare X stable on the kernel's other paths: an empty active set (zero fill), a byte
    map, forced cluster sizes and a capped grid (partials combined through the cluster before the
    store), bfloat16, and a device-side count (which makes the kernel ignore both promises).  Three
    calls back to back into one output; the last one's result must be there."""
    ops = _ops()
    b, k, n = 16, 4096, 4096
    nb = k // 64
    w = O.make_weight(n, k, seed=71)
    x = O.make_activations(b, k, seed=72)
    dt = torch.bfloat16 if form == "bf16" else torch.float16
    if form == "bf16":
        w, x = O.round_to_bf16(w.astype(np.float32)), O.round_to_bf16(x.astype(np.float32))
    tw, tx = torch.from_numpy(w).to(dev).to(dt), torch.from_numpy(x).to(dev).to(dt)
    packed = ops.pack_weight(tw)
    out = torch.full((b, n), float("nan"), dtype=dt, device=dev)
    idl = [O.random_active_blocks(nb, nk, seed=nk) for nk in (40, 9, 0 if form == "empty" else 21)]
    torch.cuda.synchronize()
    for ids in idl:
        kw = dict(ids_stable=True, x_stable=True, next_independent=True)
        if form == "bitmap":
            kw["bitmap"] = torch.from_numpy(O.build_bitmap(ids, nb)).to(dev)
        else:
            kw["ids"] = torch.from_numpy(ids).to(dev)
        if form == "cluster2":
            kw["cluster"] = 2
        elif form == "cluster4":
            kw["cluster"] = 4
        elif form == "capped":
            kw["max_ctas"] = 64
        elif form == "count":
            kw["count"] = torch.tensor([ids.size], dtype=torch.int32, device=dev)
            kw["k_host"] = nb
            kw["ids"] = torch.from_numpy(np.concatenate([ids, np.zeros(nb - ids.size, np.int32)])).to(dev)
        ops.gemm(tx, packed, out, **kw)
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 0
    ref = O.masked_gemm(x, w, idl[-1])
    got = out.float().cpu().numpy()
    if form == "empty":
        assert not got.any()
    else:
        assert O.max_err_ratio(got, ref) <= (2.0 ** -7 if form == "bf16" else TOL)


@pytest.mark.parametrize("b", [2, 16])
def test_all_ids_bad_writes_zeros(dev, b):
    ops = _ops()
    x = O.make_activations(b, 1024, seed=1)
    w = O.make_weight(256, 1024, seed=1)
    out = torch.full((b, 256), float("nan"), dtype=torch.float16, device=dev)
    ids = torch.tensor([16, 99, -3], dtype=torch.int32, device=dev)
    ops.gemm(torch.from_numpy(x).to(dev), ops.pack_weight(torch.from_numpy(w).to(dev)), out, ids=ids)
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 1
    assert not out.cpu().numpy().any()


def test_bad_block_id_is_skipped_and_flagged(dev):
    ops = _ops()
    x = O.make_activations(2, 1024, seed=1)
    w = O.make_weight(256, 1024, seed=1)
    tx, tw = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
    out = torch.empty(2, 256, dtype=torch.float16, device=dev)
    ids = torch.tensor([3, 99, 7, -1], dtype=torch.int32, device=dev)
    ops.gemm(tx, ops.pack_weight(tw), out, ids=ids)
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 1                       # BAS_DEV_BAD_BLOCK_ID
    assert ops.read_status(dev) == 0                       # reading clears it
    assert O.max_err_ratio(out.cpu().numpy(), O.masked_gemm(x, w, np.array([3, 7]))) <= TOL


@pytest.mark.parametrize("b", [2, 16, 64])
def test_result_is_deterministic_and_workspace_reusable(dev, b):
    x = O.make_activations(b, 11008, seed=31, dist="laplace")
    w = O.make_weight(4096, 11008, seed=31)
    ids = O.random_active_blocks(172, 62, seed=31)
    ys = [_run_gemm(dev, x, w, ids=ids) for _ in range(3)]
    assert np.array_equal(ys[0], ys[1]) and np.array_equal(ys[0], ys[2])


def test_gemm_against_reference_kernel_outputs(dev, golden):
    data, meta = golden
    for gi, c in enumerate(meta["gemm"]):
        nb = (c["k"] + 63) // 64
        x = O.make_activations(c["batch"], c["k"], c["seed"], c["dist"])
        w = O.make_weight(c["n"], c["k"], c["seed"], std=0.05)
        ids = O.random_active_blocks(nb, c["n_keep"], c["seed"])
        if c["k"] % 8:
            continue
        y = _run_gemm(dev, x, w, ids=ids)
        ref = O.masked_gemm(x, w, ids)
        assert O.max_err_ratio(y, ref) <= TOL
        for name in ("triton_list", "triton_bitmap", "torch_f16"):
            assert O.max_err_ratio(y, data[f"gemm{gi}_{name}"].astype(np.float32)) <= 2 * TOL, (gi, name)


# ---------------------------------------------------------------------------------------------
# selection
# ---------------------------------------------------------------------------------------------

def _select(dev, x, n_keep, kind, want_scores=False):
    ops = _ops()
    tx = torch.from_numpy(x).to(dev)
    nb = x.shape[1] // 64
    bm = torch.full((nb,), 7, dtype=torch.uint8, device=dev)
    sc = torch.empty(nb, dtype=torch.float64, device=dev)
    ids, cnt = ops.select_topk(tx, n_keep, kind, bitmap_out=bm, scores_out=sc)
    torch.cuda.synchronize()
    return ids.cpu().numpy(), int(cnt.item()), bm.cpu().numpy(), sc.cpu().numpy()


def test_selection_matches_reference_golden(dev, golden):
    data, meta = golden
    for ci, c in enumerate(meta["select"]):
        if c["k"] % 8:
            continue
        x = O.make_activations(c["batch"], c["k"], c["seed"], c["dist"])
        nb = c["k"] // 64
        n_keep = O.n_keep_from_density(c["density"], nb)
        for kind, name in ((O.SCORE_NORM, "norm"), (O.SCORE_ENERGY, "energy")):
            ids, cnt, bm, sc = _select(dev, x, n_keep, kind)
            ref = data[f"select{ci}_{name}_ids"]
            assert cnt == n_keep
            assert np.array_equal(ids, ref), f"case {ci} {name}"
            assert np.array_equal(bm, O.build_bitmap(ref, nb))
            np.testing.assert_allclose(sc, O.block_scores(x, kind), rtol=1e-14)


@pytest.mark.parametrize("b,k", [(1, 64), (2, 11008), (7, 4096), (64, 11008), (16, 704), (33, 8192)])
@pytest.mark.parametrize("kind", [0, 1])
def test_selection_matches_oracle(dev, b, k, kind):
    x = O.make_activations(b, k, seed=b + k + kind, dist="laplace")
    nb = k // 64
    for n_keep in sorted({1, max(1, nb // 3), nb}):
        ids, cnt, bm, sc = _select(dev, x, n_keep, kind)
        want = O.topk_ids(O.block_scores(x, kind), n_keep)
        assert cnt == n_keep and np.array_equal(ids, want)
        assert bm.sum() == n_keep


def test_weighted_selection_matches_reference_golden(dev, golden):
    """Channel weights and block prior of _select_active_blocks
    (scripts/bench_roundrobin_e2e_decode.py:104-112) through bas_select_topk_weighted: ids bit-exact
    against the vectors recorded from the reference and against the oracle, scores to fp64 rounding."""
    ops = _ops()
    data, meta = golden
    n_cases = 0
    for ci, c in enumerate(meta["select"]):
        if f"select{ci}_scale_ids" not in data or c["k"] % 8:
            continue
        x = O.make_activations(c["batch"], c["k"], c["seed"], c["dist"])
        nb = c["k"] // 64
        n_keep = O.n_keep_from_density(c["density"], nb)
        scale = O.make_channel_scale(c["k"], c["seed"])
        prior = O.make_block_prior(nb, c["seed"])
        tx = torch.from_numpy(x).to(dev)
        tscale = torch.from_numpy(scale).to(dev)
        tprior = torch.from_numpy(prior).to(dev)
        for name, sc, mult, o_mult in (
                ("scale", tscale, None, None),
                ("prior", None, ops.prior_multiplier(tprior, 0.5, 0.05), O.prior_multiplier(prior, 0.5, 0.05)),
                ("scale_prior", tscale, ops.prior_multiplier(tprior), O.prior_multiplier(prior))):
            got_scores = torch.empty(nb, dtype=torch.float64, device=dev)
            bm = torch.empty(nb, dtype=torch.uint8, device=dev)
            ids, cnt = ops.select_topk(tx, n_keep, O.SCORE_NORM, chan_scale=sc, block_mult=mult,
                                       scores_out=got_scores, bitmap_out=bm)
            ref = data[f"select{ci}_{name}_ids"]
            assert int(cnt.item()) == n_keep
            assert np.array_equal(ids.cpu().numpy(), ref), f"case {ci} {name}"
            assert np.array_equal(bm.cpu().numpy(), O.build_bitmap(ref, nb))
            want = O.weighted_block_scores(x, scale if sc is not None else None, o_mult, O.SCORE_NORM)
            np.testing.assert_allclose(got_scores.cpu().numpy(), want, rtol=1e-13)
            if mult is not None:   # torch on the device and numpy agree on the float32 factor
                np.testing.assert_allclose(mult.cpu().numpy(), o_mult, rtol=2e-7)
        n_cases += 1
    assert n_cases >= 9


def test_weighted_selection_in_sparse_linear(dev):
    """The decode operator with a block prior and channel weights: same ids as the oracle, output
    within the contraction tolerance; a prior of the wrong length is ignored like in the reference."""
    ops = _ops()
    b, k, n = 16, 4096, 512
    x = O.make_activations(b, k, 41, "normal")
    w = O.make_weight(n, k, 42)
    scale = O.make_channel_scale(k, 43)
    prior = O.make_block_prior(k // 64, 44)
    tx, tw = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
    y = ops.sparse_linear(tx, tw, 0.36, block_mult=ops.prior_multiplier(torch.from_numpy(prior).to(dev)),
                          block_score_scale=torch.from_numpy(scale).to(dev), cache_prefix="weighted_sel")
    ids = O.select_active_blocks(x, 0.36, block_prior=prior, block_score_scale=scale)
    ref = O.masked_gemm(x, w, ids)
    assert O.max_err_ratio(y.float().cpu().numpy(), ref) <= 2e-3
    assert not np.array_equal(ids, O.select_active_blocks(x, 0.36))
    y2 = ops.sparse_linear(tx, tw, 0.36, block_mult=torch.ones(5, device=dev), cache_prefix="weighted_sel")
    ref2 = O.masked_gemm(x, w, O.select_active_blocks(x, 0.36))
    assert O.max_err_ratio(y2.float().cpu().numpy(), ref2) <= 2e-3


@pytest.mark.parametrize("b", [2, 16, 64])
def test_selection_with_stable_inputs_in_a_chain(dev, b):
    """Online selection over several steps, the selection of step i+1 declaring its inputs stable so
    that it scores while the contraction of step i runs (two alternating id buffers): every step's
    ids are bit-exact and every step's output within tolerance."""
    ops = _ops()
    k, n, steps = 11008, 4096, 6
    nb = k // 64
    n_keep = O.n_keep_from_density(0.36, nb)
    w = O.make_weight(n, k, seed=81)
    packed = ops.pack_weight(torch.from_numpy(w).to(dev))
    xs = [O.make_activations(b, k, seed=800 + i, dist="laplace") for i in range(steps)]
    txs = [torch.from_numpy(x).to(dev) for x in xs]
    bufs = [(torch.full((nb,), -1, dtype=torch.int32, device=dev), torch.zeros(1, dtype=torch.int32, device=dev))
            for _ in range(2)]
    outs = [torch.full((b, n), float("nan"), dtype=torch.float16, device=dev) for _ in range(steps)]
    torch.cuda.synchronize()
    for i in range(steps):          # nothing but the library's own launches in the stream: they overlap
        ids_buf, cnt_buf = bufs[i & 1]
        sel, cnt = ops.select_topk(txs[i], n_keep, O.SCORE_ENERGY, ids_out=ids_buf, count_out=cnt_buf,
                                   inputs_stable=True)
        ops.gemm(txs[i], packed, outs[i], ids=sel, count=cnt, k_host=n_keep)
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 0
    for i in range(steps):
        want = O.topk_ids(O.block_scores(xs[i], O.SCORE_ENERGY), n_keep)
        if i >= steps - 2:          # the two buffers still hold the last two steps' ids
            assert int(bufs[i & 1][1].item()) == n_keep
            assert np.array_equal(bufs[i & 1][0][:n_keep].cpu().numpy(), want), f"step {i}"
        # a step that multiplied through another step's mask would miss the tolerance by far
        assert O.max_err_ratio(outs[i].cpu().numpy(), O.masked_gemm(xs[i], w, want)) <= TOL, f"step {i}"


def test_selection_ties_go_to_lower_index(dev):
    x = np.zeros((4, 640), np.float16)
    x[:, 64:128] = 1.0
    x[:, 320:384] = 1.0
    x[:, 512:576] = 1.0
    ids, cnt, _, _ = _select(dev, x, 2, O.SCORE_NORM)
    assert ids.tolist() == [1, 5]
    ids, cnt, _, _ = _select(dev, x, 5, O.SCORE_ENERGY)
    assert ids.tolist() == [0, 1, 2, 5, 8]


def test_budget_selection_matches_reference_golden(dev, golden):
    ops = _ops()
    data, meta = golden
    for ci, c in enumerate(meta["select"]):
        if c["k"] % 8:
            continue
        x = O.make_activations(c["batch"], c["k"], c["seed"], c["dist"])
        tx = torch.from_numpy(x).to(dev)
        for keep in (0.5, 0.9, 0.99):
            ids, cnt = ops.select_budget(tx, keep)
            torch.cuda.synchronize()
            n = int(cnt.item())
            ref = data[f"select{ci}_budget{int(round(keep * 100))}_ids"]
            assert np.array_equal(ids[:n].cpu().numpy(), ref), f"case {ci} keep {keep}"


def test_bitmap_builder(dev):
    ops = _ops()
    for nb, n_keep, seed in [(64, 32, 0), (172, 62, 1), (172, 0, 2), (7, 7, 3)]:
        ids = O.random_active_blocks(nb, n_keep, seed)
        bm = ops.build_bitmap(torch.from_numpy(ids).to(dev), nb, dev)
        assert np.array_equal(bm.cpu().numpy(), O.build_bitmap(ids, nb))


# ---------------------------------------------------------------------------------------------
# fused select -> GEMM, the drop-in module and the host-buffer operator
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("b,density", [(2, 0.197), (16, 0.36), (64, 0.48)])
def test_sparse_linear_chain(dev, b, density):
    ops = _ops()
    k, n = 11008, 4096
    w = O.make_weight(n, k, seed=77)
    tw = torch.from_numpy(w).to(dev)
    for step in range(3):
        x = O.make_activations(b, k, seed=500 + step, dist="laplace")
        tx = torch.from_numpy(x).to(dev).reshape(b, 1, k)
        y = ops.sparse_linear(tx, tw, density, score_kind=O.SCORE_ENERGY)
        torch.cuda.synchronize()
        ids = O.select_active_blocks(x, density, O.SCORE_ENERGY)
        assert y.shape == (b, 1, n)
        assert O.max_err_ratio(y.reshape(b, n).cpu().numpy(), O.masked_gemm(x, w, ids)) <= TOL
    assert ops.read_status(dev) == 0


def test_drop_in_wrappers_and_graph_capture(dev):
    import kernels.shared_mask_batched_triton_min_runtime as K

    b, k, n = 16, 4096, 4096
    x = O.make_activations(b, k, seed=0)
    w = O.make_weight(n, k, seed=0)
    ids = O.select_active_blocks(x, 0.5, O.SCORE_NORM)
    ref = O.masked_gemm(x, w, ids)
    tx = torch.from_numpy(x).to(dev).reshape(b, 1, k)
    tw = torch.from_numpy(w).to(dev)
    tids = torch.from_numpy(ids).to(dev)
    bitmap = K._build_active_k_bitmap(tids, 64, "cuda")
    assert np.array_equal(bitmap.cpu().numpy(), O.build_bitmap(ids, 64))
    K._get_prepacked_weight_block_major(tw, 64, cache_prefix="t")

    calls = {
        "list": lambda o: K._prepacked_block_sparse_gemm_from_active_blocks_splitk(
            tx, tw, tids, o, cache_prefix="t", num_split_k=4, tile_b=16, tile_n=64, tile_warps=2, tile_stages=3),
        "bitmap": lambda o: K._prepacked_block_sparse_gemm_from_active_blocks_bitmap_preload(
            tx, tw, tids, o, cache_prefix="t", total_k_blocks=64, prebuilt_bitmap=bitmap),
        "bitmap_sk": lambda o: K._prepacked_block_sparse_gemm_from_active_blocks_bitmap_preload_splitk(
            tx, tw, tids, o, cache_prefix="t", total_k_blocks=64, prebuilt_bitmap=bitmap, num_split_k=2),
        "generic": lambda o: K._prepacked_block_sparse_gemm_from_active_blocks(
            tx, tw, tids, o, cache_prefix="t", use_run_compressed=False),
    }
    for name, fn in calls.items():
        out = torch.zeros(b, 1, n, dtype=torch.float16, device=dev)
        fn(out)
        torch.cuda.synchronize()
        assert O.max_err_ratio(out.reshape(b, n).cpu().numpy(), ref) <= TOL, name

    # the reference's timing protocol: warm up on a side stream, capture one call, replay
    out = torch.zeros(b, 1, n, dtype=torch.float16, device=dev)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for _ in range(3):
            calls["bitmap"](out)
        torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        calls["bitmap"](out)
    out.zero_()
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    assert O.max_err_ratio(out.reshape(b, n).cpu().numpy(), ref) <= TOL

    # empty list -> zeros; active_blocks_limit keeps a prefix
    out.fill_(1)
    K._prepacked_block_sparse_gemm_from_active_blocks_splitk(tx, tw, tids[:0], out)
    assert not out.any()
    K._prepacked_block_sparse_gemm_from_active_blocks(tx, tw, tids, out, active_blocks_limit=5)
    torch.cuda.synchronize()
    assert O.max_err_ratio(out.reshape(b, n).cpu().numpy(), O.masked_gemm(x, w, ids[:5])) <= TOL


def test_batches_above_64_rows_are_sliced(dev):
    import kernels.shared_mask_batched_triton_min_runtime as K

    b, k, n = 100, 1024, 256
    x = O.make_activations(b, k, seed=4)
    w = O.make_weight(n, k, seed=4)
    ids = O.random_active_blocks(16, 6, seed=4)
    out = torch.zeros(b, 1, n, dtype=torch.float16, device=dev)
    K._prepacked_block_sparse_gemm_from_active_blocks_splitk(
        torch.from_numpy(x).to(dev).reshape(b, 1, k), torch.from_numpy(w).to(dev), torch.from_numpy(ids).to(dev), out)
    torch.cuda.synchronize()
    assert O.max_err_ratio(out.reshape(b, n).cpu().numpy(), O.masked_gemm(x, w, ids)) <= TOL


@pytest.mark.parametrize("b,k,n", [(16, 4096, 4096), (2, 200, 96), (5, 203, 130)])
def test_host_buffer_operator(dev, b, k, n):
    import ctypes
    from bas import abi as L

    x = O.make_activations(b, k, seed=8)
    w = O.make_weight(n, k, seed=8)
    nb = k // 64
    h = ctypes.c_void_p()
    L.check(L.lib.bas_linear_create(ctypes.byref(h), w.ctypes.data, n, k, 64), "create")
    try:
        y = np.empty((b, n), np.float16)
        n_keep = max(1, nb // 2)
        ids_out = np.full(nb, -1, np.int32)
        L.check(L.lib.bas_linear_forward_host(h, x.ctypes.data, b, n_keep, O.SCORE_NORM, y.ctypes.data,
                                              ids_out.ctypes.data), "forward_host")
        want_ids = O.topk_ids(O.block_scores(x, O.SCORE_NORM), n_keep)
        assert np.array_equal(ids_out[:n_keep], want_ids)
        assert O.max_err_ratio(y, O.masked_gemm(x, w, want_ids)) <= TOL
        # caller-provided ids, including the ragged last block
        ids = np.arange((k + 63) // 64, dtype=np.int32)[::-1].copy()
        L.check(L.lib.bas_linear_forward_host_ids(h, x.ctypes.data, b, ids.ctypes.data, ids.size, y.ctypes.data),
                "forward_host_ids")
        assert O.max_err_ratio(y, O.masked_gemm(x, w, ids)) <= TOL
        L.check(L.lib.bas_linear_forward_host_ids(h, x.ctypes.data, b, None, 0, y.ctypes.data), "empty")
        assert not y.any()
    finally:
        L.lib.bas_linear_destroy(h)


def test_host_buffer_operator_back_to_back_batches(dev):
    """Calls of different batch sizes in immediate succession on rotating handles: every call must
    return its own result (a chain of early-starting kernels must never hand back stale data)."""
    import ctypes
    from bas import abi as L

    k, n, nb = 11008, 4096, 172
    keep = {2: 34, 16: 62, 64: 83}
    w = O.make_weight(n, k, seed=0)
    handles = []
    for _ in range(2):
        h = ctypes.c_void_p()
        L.check(L.lib.bas_linear_create(ctypes.byref(h), w.ctypes.data, n, k, 64), "create")
        handles.append(h)
    try:
        xs = {b: O.make_activations(b, k, seed=1000 + b, dist="laplace") for b in keep}
        want = {}
        for b in keep:
            ids = O.topk_ids(O.block_scores(xs[b], O.SCORE_NORM), keep[b])
            want[b] = (ids, O.masked_gemm(xs[b], w, ids))
        for i in range(36):
            b = (2, 16, 64)[i % 3]
            y = np.empty((b, n), np.float16)
            ids = np.full(nb, -1, np.int32)
            L.check(L.lib.bas_linear_forward_host(handles[i % 2], xs[b].ctypes.data, b, keep[b], O.SCORE_NORM,
                                                  y.ctypes.data, ids.ctypes.data), "forward_host")
            assert np.array_equal(ids[:keep[b]], want[b][0]), f"call {i} B={b}"
            assert O.max_err_ratio(y, want[b][1]) <= TOL, f"call {i} B={b}"
    finally:
        for h in handles:
            L.lib.bas_linear_destroy(h)


def test_linear_stack_single_rank(dev):
    """One decoder layer's seven masked projections through the tensor-parallel wrapper at world 1."""
    from bas import tp

    stack = tp.DecodeLinearStack(layers=1, batch=16, sparsity=0.638, device=dev, seed=1)
    stack.step()
    torch.cuda.synchronize()
    assert len(stack.items) == 7
    gen = torch.Generator(device=dev)
    for si, (lin, x, bitmap, out, _) in enumerate(stack.items):
        spec = lin.spec
        gen.manual_seed(1 * 1_000_003 + si)
        w = (torch.randn(spec.n, spec.k, generator=gen, device=dev, dtype=torch.float32) * 0.02).half()
        mask = bitmap.float().repeat_interleave(64)
        ref = (x.float() * mask) @ w.float().t()
        err = ((out.float() - ref).abs().max() / ref.abs().max()).item()
        assert err <= TOL, (spec.name, err)
        assert int(bitmap.sum().item()) == round((1 - 0.638) * (spec.k // 64))


def test_linear_stack_with_stacked_projections(dev):
    """q/k/v and gate/up as one masked GEMM each over their stacked output columns."""
    from bas import tp

    stack = tp.DecodeLinearStack(layers=1, batch=16, sparsity=0.638, device=dev, seed=1, fuse_shared_inputs=True)
    stack.step()
    torch.cuda.synchronize()
    assert [lin.spec.name for lin, *_ in stack.items] == ["qkv_proj", "o_proj", "gate_up_proj", "down_proj"]
    members = {"qkv_proj": (0, 1, 2), "o_proj": (3,), "gate_up_proj": (4, 5), "down_proj": (6,)}
    gen = torch.Generator(device=dev)
    for lin, x, bitmap, out, _ in stack.items:
        ws = []
        for si in members[lin.spec.name]:
            spec = tp.LLAMA2_7B_LAYER[si]
            gen.manual_seed(1 * 1_000_003 + si)
            ws.append((torch.randn(spec.n, spec.k, generator=gen, device=dev, dtype=torch.float32) * 0.02).half())
        w = torch.cat(ws)
        assert out.shape == (16, w.shape[0])
        ref = (x.float() * bitmap.float().repeat_interleave(64)) @ w.float().t()
        err = ((out.float() - ref).abs().max() / ref.abs().max()).item()
        assert err <= TOL, (lin.spec.name, err)


# ---------------------------------------------------------------------------------------------
# bfloat16 (the reference's kernels take fp16 or bf16 tensors alike)
# ---------------------------------------------------------------------------------------------
# bf16 keeps 8 significant bits: one unit in the last place of the largest output is
# 2^-8 * max|ref|, and the fp32-accumulated result may round to the neighbour of the fp64 oracle's.
TOL_BF16 = 2.0 ** -7


def _bf16_inputs(b, k, n, seed, dist="normal"):
    x = O.round_to_bf16(O.make_activations(b, k, seed=seed, dist=dist).astype(np.float32))
    w = O.round_to_bf16(O.make_weight(n, k, seed=seed + 1).astype(np.float32))
    return x, w


@pytest.mark.parametrize("b,k,n,n_keep", [(2, 4096, 1024, 20), (16, 11008, 4096, 62), (64, 11008, 4096, 83),
                                          (5, 512, 24000, 5), (33, 1088, 4104, 9)])
def test_bf16_gemm_matches_oracle(dev, b, k, n, n_keep):
    ops = _ops()
    x, w = _bf16_inputs(b, k, n, seed=b)
    ids = O.random_active_blocks((k + 63) // 64, n_keep, seed=b)
    tx = torch.from_numpy(x).to(dev).to(torch.bfloat16)
    tw = torch.from_numpy(w).to(dev).to(torch.bfloat16)
    assert torch.equal(tx.float().cpu(), torch.from_numpy(x))      # the conversion lost nothing
    packed = ops.pack_weight(tw)
    out = torch.full((b, n), float("nan"), dtype=torch.bfloat16, device=dev)
    for kw in ({"ids": torch.from_numpy(ids).to(dev)},
               {"bitmap": torch.from_numpy(O.build_bitmap(ids, (k + 63) // 64)).to(dev), "ids_stable": True}):
        out.fill_(float("nan"))
        ops.gemm(tx, packed, out, **kw)
        torch.cuda.synchronize()
        assert ops.read_status(dev) == 0
        assert O.max_err_ratio(out.float().cpu().numpy(), O.masked_gemm(x, w, ids)) <= TOL_BF16


def test_bf16_and_fp16_must_not_be_mixed(dev):
    ops = _ops()
    x = torch.zeros(2, 128, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(64, 128, dtype=torch.bfloat16, device=dev)
    out = torch.zeros(2, 64, dtype=torch.float16, device=dev)
    with pytest.raises(TypeError):
        ops.gemm(x, ops.pack_weight(w), out, ids=torch.zeros(1, dtype=torch.int32, device=dev))
    with pytest.raises(Exception):      # the CUDA-core kernel is fp16 only
        ops.gemm(x, ops.pack_weight(w), out.to(torch.bfloat16), ids=torch.zeros(1, dtype=torch.int32, device=dev),
                 family=1)


@pytest.mark.parametrize("b,k,kind", [(16, 11008, 1), (3, 4096, 0), (64, 4160, 1)])
def test_bf16_selection_is_bit_exact(dev, b, k, kind):
    ops = _ops()
    x = O.round_to_bf16(O.make_activations(b, k, seed=77 + b, dist="laplace").astype(np.float32))
    tx = torch.from_numpy(x).to(dev).to(torch.bfloat16)
    nb = k // 64
    scores = O.block_scores(x, kind)
    n_keep = O.n_keep_from_density(0.36, nb)
    got_scores = torch.empty(nb, dtype=torch.float64, device=dev)
    ids, count = ops.select_topk(tx, n_keep, kind, scores_out=got_scores)
    assert int(count.item()) == n_keep
    assert np.array_equal(ids.cpu().numpy(), O.topk_ids(scores, n_keep))
    assert np.array_equal(got_scores.cpu().numpy(), scores)
    if kind == 1:
        ids_b, count_b = ops.select_budget(tx, 0.8, 2)
        want = O.energy_budget_ids(scores, 0.8, 2)
        assert int(count_b.item()) == want.size
        assert np.array_equal(ids_b[: want.size].cpu().numpy(), want)


# ---------------------------------------------------------------------------------------------
# row-parallel sum formed inside the kernel: the one-rank case (publish, collect nothing, convert)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("b,k,n,n_keep", [(16, 11008, 4096, 62), (64, 11008, 4096, 83), (2, 4096, 4096, 13),
                                          (5, 512, 24000, 5), (33, 1088, 4104, 9)])
def test_in_kernel_sum_with_one_rank_equals_plain_call(dev, b, k, n, n_keep):
    ops = _ops()
    nb = (k + 63) // 64
    x = torch.from_numpy(O.make_activations(b, k, seed=b)).to(dev)
    w = torch.from_numpy(O.make_weight(n, k, seed=b + 1)).to(dev)
    packed = ops.pack_weight(w)
    group = ops.ExchangeGroup(dev, 64, n)
    try:
        for rep in range(5):          # call numbers 1..5: both partial buffers, several times
            ids = torch.from_numpy(O.random_active_blocks(nb, max(1, n_keep - rep), seed=rep)).to(dev)
            want = torch.empty(b, n, dtype=torch.float16, device=dev)
            got = torch.full((b, n), float("nan"), dtype=torch.float16, device=dev)
            ops.gemm(x, packed, want, ids=ids)
            ops.gemm(x, packed, got, ids=ids, tp=group, ids_stable=bool(rep & 1))
            torch.cuda.synchronize()
            assert ops.read_status(dev) == 0
            assert torch.equal(got, want)
        # an empty active set known only on the device: this rank's partial is zero
        got = torch.full((b, n), float("nan"), dtype=torch.float16, device=dev)
        ops.gemm(x, packed, got, ids=ids, count=torch.zeros(1, dtype=torch.int32, device=dev), k_host=int(ids.numel()),
                 tp=group)
        torch.cuda.synchronize()
        assert ops.read_status(dev) == 0
        assert float(got.float().abs().max().item()) == 0.0
    finally:
        group.close()


def test_in_kernel_sum_group_shared_by_calls_of_different_shape(dev):
    """One exchange group, calls whose grids differ in size from one call to the next."""
    ops = _ops()
    group = ops.ExchangeGroup(dev, 64, 4104)
    try:
        cases = [(16, 11008, 4096, 62), (2, 4096, 512, 3), (64, 11008, 4096, 83), (33, 1088, 4104, 9), (5, 512, 1000, 2)]
        prepared = []
        for b, k, n, n_keep in cases:
            x = torch.from_numpy(O.make_activations(b, k, seed=b)).to(dev)
            packed = ops.pack_weight(torch.from_numpy(O.make_weight(n, k, seed=b + 1)).to(dev))
            ids = torch.from_numpy(O.random_active_blocks((k + 63) // 64, n_keep, seed=b)).to(dev)
            want = torch.empty(b, n, dtype=torch.float16, device=dev)
            ops.gemm(x, packed, want, ids=ids)
            prepared.append((x, packed, ids, want, torch.empty_like(want)))
        for rep in range(3):
            for x, packed, ids, want, got in prepared:
                got.fill_(float("nan"))
                ops.gemm(x, packed, got, ids=ids, tp=group, ids_stable=True)
            torch.cuda.synchronize()
            assert ops.read_status(dev) == 0
            for x, packed, ids, want, got in prepared:
                assert torch.equal(got, want)
    finally:
        group.close()


@pytest.mark.parametrize("max_ctas", [16, 40, 100])
@pytest.mark.parametrize("b,k,n,n_keep,cluster", [(16, 11008, 4096, 62, 0), (64, 4096, 2048, 23, 4), (2, 4096, 512, 23, 0),
                                                  (16, 1024, 11008, 6, 0), (48, 2048, 1000, 30, 2)])
def test_grid_size_does_not_change_the_result(dev, b, k, n, n_keep, cluster, max_ctas):
    x = O.make_activations(b, k, seed=b + max_ctas)
    w = O.make_weight(n, k, seed=7)
    ids = O.random_active_blocks(k // 64, n_keep, seed=max_ctas)
    ops = _ops()
    tx, tw = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
    out = torch.full((b, n), float("nan"), dtype=torch.float16, device=dev)
    ops.gemm(tx, ops.pack_weight(tw), out, ids=torch.from_numpy(ids).to(dev), cluster=cluster, max_ctas=max_ctas)
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 0
    assert O.max_err_ratio(out.cpu().numpy(), O.masked_gemm(x, w, ids)) <= TOL


@pytest.mark.parametrize("pin", [False, True])
def test_host_buffer_operator_overlapped_submits(dev, pin):
    """Three forwards in flight on three handles (pageable or page-locked caller buffers), collected
    afterwards; a second submit on a busy handle is refused."""
    import ctypes
    from bas import abi as L

    k, n, nb = 11008, 4096, 172
    keep = {2: 34, 16: 62, 64: 83}
    w = O.make_weight(n, k, seed=0)
    handles = []
    for _ in range(3):
        h = ctypes.c_void_p()
        L.check(L.lib.bas_linear_create(ctypes.byref(h), w.ctypes.data, n, k, 64), "create")
        handles.append(h)
    keepalive = []

    def host_array(shape):
        if not pin:
            return np.empty(shape, np.float16)
        t = torch.empty(shape, dtype=torch.float16, pin_memory=True)
        keepalive.append(t)
        return t.numpy()

    try:
        xs, ys, want = {}, {}, {}
        for b in keep:
            xs[b] = host_array((b, k))
            xs[b][...] = O.make_activations(b, k, seed=1000 + b, dist="laplace")
            ys[b] = host_array((b, n))
            ids = O.topk_ids(O.block_scores(xs[b], O.SCORE_NORM), keep[b])
            want[b] = (ids, O.masked_gemm(xs[b], w, ids))
        ids_out = {b: np.full(nb, -1, np.int32) for b in keep}
        for rep in range(6):
            for b in keep:
                ys[b][...] = np.float16(np.nan)
            order = list(keep)[rep % 3:] + list(keep)[:rep % 3]
            for h, b in zip(handles, order):
                L.check(L.lib.bas_linear_submit_host(h, xs[b].ctypes.data, b, keep[b], O.SCORE_NORM, ys[b].ctypes.data,
                                                     ids_out[b].ctypes.data), "submit")
            assert L.lib.bas_linear_submit_host(handles[0], xs[2].ctypes.data, 2, keep[2], O.SCORE_NORM,
                                                ys[2].ctypes.data, None) != 0
            for h in handles:
                L.check(L.lib.bas_linear_wait(h), "wait")
            assert L.lib.bas_linear_wait(handles[0]) != 0          # nothing in flight any more
            for b in keep:
                assert np.array_equal(ids_out[b][:keep[b]], want[b][0]), (rep, b)
                assert O.max_err_ratio(ys[b], want[b][1]) <= TOL, (rep, b)
    finally:
        for h in handles:
            L.lib.bas_linear_destroy(h)


def test_sparse_linear_budget_mode_fixed_ids_and_dense_fallback(dev):
    """The decode operator's other modes: energy budget with the count kept on the device, reuse of
    a given mask, and the dense path for prefill shapes and density 1."""
    ops = _ops()
    b, k, n = 16, 4096, 1024
    w = O.make_weight(n, k, seed=9)
    tw = torch.from_numpy(w).to(dev)
    x = O.make_activations(b, k, seed=21, dist="laplace")
    tx = torch.from_numpy(x).to(dev)
    energy = O.block_scores(x, O.SCORE_ENERGY)
    for keep in (0.5, 0.9, 0.999):
        ids = O.energy_budget_ids(energy, keep, 2)
        y = ops.sparse_linear(tx, tw, 0.0, energy_keep=keep, min_keep=2)
        torch.cuda.synchronize()
        assert y.shape == (b, n)
        assert O.max_err_ratio(y.cpu().numpy(), O.masked_gemm(x, w, ids)) <= TOL, keep
    fixed = O.random_active_blocks(k // 64, 11, seed=4)
    y = ops.sparse_linear(tx, tw, 0.3, fixed_active_blocks=torch.from_numpy(fixed).to(dev))
    torch.cuda.synchronize()
    assert O.max_err_ratio(y.cpu().numpy(), O.masked_gemm(x, w, fixed)) <= TOL
    dense = (tx.float() @ tw.float().t()).cpu().numpy()
    y = ops.sparse_linear(tx, tw, 1.0)
    assert O.max_err_ratio(y.float().cpu().numpy(), dense) <= TOL
    prefill = torch.from_numpy(O.make_activations(6, k, seed=3)).to(dev).reshape(2, 3, k)      # 3 positions: dense
    y = ops.sparse_linear(prefill, tw, 0.3)
    assert y.shape == (2, 3, n)
    want = (prefill.float() @ tw.float().t()).cpu().numpy()
    assert O.max_err_ratio(y.float().cpu().numpy(), want) <= TOL
    assert ops.read_status(dev) == 0


# ---------------------------------------------------------------------------------------------
# selection inside the contraction kernel
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("b,k,n,kind", [(16, 11008, 4096, 1), (2, 4096, 4096, 0), (64, 11008, 4096, 0), (33, 1088, 1000, 1),
                                        (16, 4096, 11008, 0), (5, 4160, 512, 1)])
def test_select_gemm_matches_the_two_launch_chain(dev, b, k, n, kind):
    """Ids bit-exact against the oracle, sums within tolerance, optional outputs filled - whether the
    shape runs the selection inside the contraction kernel or falls back to two launches."""
    ops = _ops()
    nb = k // 64
    w = O.make_weight(n, k, seed=b)
    packed = ops.pack_weight(torch.from_numpy(w).to(dev))
    for step, density in enumerate((0.36, 0.1, 0.9)):
        x = O.make_activations(b, k, seed=40 + step + b, dist="laplace")
        tx = torch.from_numpy(x).to(dev)
        scores = O.block_scores(x, kind)
        n_keep = O.n_keep_from_density(density, nb)
        want_ids = O.topk_ids(scores, n_keep)
        out = torch.full((b, n), float("nan"), dtype=torch.float16, device=dev)
        ids_out = torch.full((nb,), -1, dtype=torch.int32, device=dev)
        count_out = torch.zeros(1, dtype=torch.int32, device=dev)
        bitmap = torch.full((nb,), 7, dtype=torch.uint8, device=dev)
        got_scores = torch.zeros(nb, dtype=torch.float64, device=dev)
        ops.select_gemm(tx, packed, out, n_keep, kind, ids_out=ids_out, count_out=count_out, bitmap_out=bitmap,
                        scores_out=got_scores)
        torch.cuda.synchronize()
        assert ops.read_status(dev) == 0
        assert int(count_out.item()) == n_keep
        assert np.array_equal(ids_out[:n_keep].cpu().numpy(), want_ids)
        assert np.array_equal(bitmap.cpu().numpy(), O.build_bitmap(want_ids, nb))
        assert np.array_equal(got_scores.cpu().numpy(), scores)
        assert O.max_err_ratio(out.cpu().numpy(), O.masked_gemm(x, w, want_ids)) <= TOL
    # energy budget, variable count
    x = O.make_activations(b, k, seed=99 + b, dist="laplace")
    energy = O.block_scores(x, O.SCORE_ENERGY)
    for keep in (0.5, 0.95):
        want_ids = O.energy_budget_ids(energy, keep, 2)
        out = torch.full((b, n), float("nan"), dtype=torch.float16, device=dev)
        ids_out, count_out = ops.select_gemm(torch.from_numpy(x).to(dev), packed, out, 2, O.SCORE_ENERGY, energy_keep=keep)
        torch.cuda.synchronize()
        assert int(count_out.item()) == want_ids.size
        assert np.array_equal(ids_out[: want_ids.size].cpu().numpy(), want_ids)
        assert O.max_err_ratio(out.cpu().numpy(), O.masked_gemm(x, w, want_ids)) <= TOL


def test_select_gemm_ties_and_chained_calls(dev):
    """Equal scores go to the lower id inside the kernel too; calls in a row hand back their own masks."""
    ops = _ops()
    b, k, n = 16, 4096, 2048
    nb = k // 64
    w = O.make_weight(n, k, seed=1)
    packed = ops.pack_weight(torch.from_numpy(w).to(dev))
    x = np.zeros((b, k), np.float16)
    x[:, : 64 * 10] = 1.0                     # ten blocks with the same score, the rest zero
    out = torch.empty(b, n, dtype=torch.float16, device=dev)
    ids, count = ops.select_gemm(torch.from_numpy(x).to(dev), packed, out, 14, O.SCORE_NORM)
    torch.cuda.synchronize()
    assert np.array_equal(ids[:14].cpu().numpy(), np.arange(14, dtype=np.int32))
    xs = [O.make_activations(b, k, seed=300 + i, dist="laplace") for i in range(6)]
    txs = [torch.from_numpy(v).to(dev) for v in xs]
    outs = [torch.empty(b, n, dtype=torch.float16, device=dev) for _ in xs]
    idbufs = [torch.empty(nb, dtype=torch.int32, device=dev) for _ in xs]
    cnt = torch.empty(1, dtype=torch.int32, device=dev)
    for i in range(6):
        ops.select_gemm(txs[i], packed, outs[i], 23, O.SCORE_ENERGY, ids_out=idbufs[i], count_out=cnt)
    torch.cuda.synchronize()
    for i in range(6):
        want = O.topk_ids(O.block_scores(xs[i], O.SCORE_ENERGY), 23)
        assert np.array_equal(idbufs[i][:23].cpu().numpy(), want), i
        assert O.max_err_ratio(outs[i].cpu().numpy(), O.masked_gemm(xs[i], w, want)) <= TOL, i


@pytest.mark.parametrize("b,k,n", [(4, 4096, 2048), (16, 11008, 4096)])
def test_select_gemm_bf16(dev, b, k, n):
    """bf16 activations through the one-call selection + contraction (in-kernel selection for the
    small case, the two-launch chain for the large one)."""
    ops = _ops()
    nb = k // 64
    x, w = _bf16_inputs(b, k, n, seed=60 + b, dist="laplace")
    tx = torch.from_numpy(x).to(dev).to(torch.bfloat16)
    packed = ops.pack_weight(torch.from_numpy(w).to(dev).to(torch.bfloat16))
    scores = O.block_scores(x, O.SCORE_ENERGY)
    n_keep = O.n_keep_from_density(0.36, nb)
    want = O.topk_ids(scores, n_keep)
    out = torch.full((b, n), float("nan"), dtype=torch.bfloat16, device=dev)
    ids, count = ops.select_gemm(tx, packed, out, n_keep, O.SCORE_ENERGY)
    torch.cuda.synchronize()
    assert ops.read_status(dev) == 0
    assert int(count.item()) == n_keep
    assert np.array_equal(ids[:n_keep].cpu().numpy(), want)
    assert O.max_err_ratio(out.float().cpu().numpy(), O.masked_gemm(x, w, want)) <= TOL_BF16


@pytest.mark.parametrize("b,k", [(2, 1024), (16, 4096), (64, 11008)])
def test_selection_with_non_finite_activations(dev, b, k):
    """NaN and infinities in X (and an infinity times a zero channel weight) take the defined path:
    NaN ranks above +inf, equal scores to the lower id, exactly n_keep ids, nothing out of bounds -
    top-k, weighted, budget and the one-call selection + contraction alike."""
    ops = _ops()
    nb = k // 64
    x = O.make_activations(b, k, seed=b + k, dist="laplace")
    x[0, 64 * 3 + 5] = np.nan
    x[b - 1, 64 * 7] = np.inf
    x[b // 2, 64 * 9 + 1] = -np.inf
    x[0, 64 * 11] = np.inf
    x[0, 64 * 11 + 1] = np.nan
    tx = torch.from_numpy(x).to(dev)
    guard = 7
    for kind in (O.SCORE_NORM, O.SCORE_ENERGY):
        for n_keep in (1, 3, nb // 3, nb):
            ids_buf = torch.full((nb + guard,), -7, dtype=torch.int32, device=dev)
            cnt = torch.zeros(1, dtype=torch.int32, device=dev)
            ops.select_topk(tx, n_keep, kind, ids_out=ids_buf, count_out=cnt)
            torch.cuda.synchronize()
            got = ids_buf.cpu().numpy()
            with np.errstate(invalid="ignore", over="ignore"):
                want = O.topk_ids(O.block_scores(x, kind), n_keep)
            assert int(cnt.item()) == n_keep
            assert np.array_equal(got[:n_keep], want), (kind, n_keep)
            assert (got[n_keep:] == -7).all(), "wrote past n_keep ids"
    # an infinite activation under a zero channel weight is not a number: weighted mode
    scale = O.make_channel_scale(k, seed=1)
    scale[64 * 7] = 0.0
    ids_buf = torch.full((nb + guard,), -7, dtype=torch.int32, device=dev)
    cnt = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.select_topk(tx, 5, O.SCORE_NORM, ids_out=ids_buf, count_out=cnt, chan_scale=torch.from_numpy(scale).to(dev))
    torch.cuda.synchronize()
    with np.errstate(invalid="ignore", over="ignore"):
        want = O.topk_ids(O.weighted_block_scores(x, scale, None), 5)
    assert np.array_equal(ids_buf[:5].cpu().numpy(), want) and (ids_buf[5:].cpu().numpy() == -7).all()
    # budget: the total is not a number, so every block is kept
    ids_buf = torch.full((nb + guard,), -7, dtype=torch.int32, device=dev)
    ops.select_budget(tx, 0.5, 1, ids_out=ids_buf, count_out=cnt)
    torch.cuda.synchronize()
    assert int(cnt.item()) == nb and np.array_equal(ids_buf[:nb].cpu().numpy(), np.arange(nb, dtype=np.int32))
    # selection + contraction in one call: same ids on both of its paths; the kernel must not fault
    w = O.make_weight(256, k, seed=2)
    out = torch.empty(b, 256, dtype=torch.float16, device=dev)
    ids_buf = torch.full((nb + guard,), -7, dtype=torch.int32, device=dev)
    ops.select_gemm(tx, ops.pack_weight(torch.from_numpy(w).to(dev)), out, 6, O.SCORE_ENERGY, ids_out=ids_buf, count_out=cnt)
    torch.cuda.synchronize()
    with np.errstate(invalid="ignore", over="ignore"):
        want = O.topk_ids(O.block_scores(x, O.SCORE_ENERGY), 6)
    assert int(cnt.item()) == 6 and np.array_equal(ids_buf[:6].cpu().numpy(), want)
    assert ops.read_status(dev) == 0
