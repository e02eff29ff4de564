"""GPU test of the step-level host-buffer operator (bas_step_*): all calls of a step submitted as one
unit - uploads, device-side selection, one list launch, downloads - with several steps in flight,
from pageable and from page-locked buffers, against the oracle."""

import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import bas_oracle as O  # noqa: E402

TOL = 2e-3


def _ptr_array(arrs):
    return (ctypes.c_void_p * len(arrs))(*[a.ctypes.data if a is not None else None for a in arrs])


@pytest.mark.parametrize("pin", [False, True])
def test_steps_in_flight_match_oracle(pin):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from bas import abi

    shapes = [(2, 1024, 512, 5, O.SCORE_NORM), (16, 2048, 1024, 12, O.SCORE_ENERGY), (64, 1024, 512, 9, O.SCORE_NORM),
              (5, 200, 96, 2, O.SCORE_NORM)]                      # the last: K not a multiple of 64 (nor of 8 x 25)
    w_shared = O.make_weight(512, 1024, seed=1)
    ws = [w_shared, O.make_weight(1024, 2048, seed=2), w_shared, O.make_weight(96, 200, seed=3)]
    calls = (abi.StepCall * len(shapes))()
    for c, ((b, k, n, n_keep, kind), w) in zip(calls, zip(shapes, ws)):
        c.w_host, c.n, c.k, c.batch, c.n_keep, c.score_kind = w.ctypes.data, n, k, b, n_keep, kind
    h = ctypes.c_void_p()
    abi.check(abi.lib.bas_step_create(ctypes.byref(h), calls, len(shapes), 3), "bas_step_create")
    keep = []

    def host(shape, dtype):
        if pin:
            t = torch.empty(shape, dtype=dtype, pin_memory=True)
            keep.append(t)
            return t.numpy()
        return np.empty(shape, dtype=np.float16 if dtype == torch.float16 else np.int32)

    n_steps = 7
    # steps 0..2 use buffer set 0..2, later steps reuse them (recurring buffers are replayed as graphs)
    sets = []
    for s in range(3):
        xs = [host((b, k), torch.float16) for b, k, *_ in shapes]
        ys = [host((b, n), torch.float16) for b, _, n, *_ in shapes]
        ids = [np.full(k // 64, -1, np.int32) for _, k, *_ in shapes]
        sets.append((xs, ys, ids))
    inputs = {}
    try:
        in_flight = []
        for step in range(n_steps):
            xs, ys, ids = sets[step % 3]
            if len(in_flight) == 3:                              # every slot busy: collect the oldest first
                done = in_flight.pop(0)
                abi.check(abi.lib.bas_step_wait(h), "bas_step_wait")
                _check(done, inputs[done], sets[done % 3], shapes, ws)
            for c, (b, k, *_rest) in enumerate(shapes):
                xs[c][...] = O.make_activations(b, k, seed=1000 * step + c, dist="laplace")
                ys[c][...] = np.nan
            inputs[step] = [x.copy() for x in xs]
            abi.check(abi.lib.bas_step_submit(h, _ptr_array(xs), _ptr_array(ys), _ptr_array(ids)), "bas_step_submit")
            in_flight.append(step)
        while in_flight:
            done = in_flight.pop(0)
            abi.check(abi.lib.bas_step_wait(h), "bas_step_wait")
            _check(done, inputs[done], sets[done % 3], shapes, ws)
        assert abi.lib.bas_step_wait(h) != 0                     # nothing left to wait for
    finally:
        abi.lib.bas_step_destroy(h)


def _check(step, xs_in, buffers, shapes, ws):
    _, ys, ids = buffers
    for c, ((b, k, n, n_keep, kind), w) in enumerate(zip(shapes, ws)):
        want = O.topk_ids(O.block_scores(xs_in[c], kind), n_keep)
        assert np.array_equal(ids[c][:n_keep], want), (step, c)
        ref = O.masked_gemm(xs_in[c], w, want)
        assert O.max_err_ratio(ys[c].astype(np.float32), ref) <= TOL, (step, c)
