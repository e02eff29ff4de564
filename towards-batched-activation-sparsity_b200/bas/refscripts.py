"""Run the reference's own two kernel-benchmark scripts, unmodified, against this package.

``scripts/profile_kernel_configs.py`` (writes the per-shape lookup tables, :260-301) and
``scripts/bench_perstep_actual_kernel_speedup.py`` (replays the thesis's per-step oracle schedules
x 224 projections with them, :210-322) import ``kernels.shared_mask_batched_triton_min_runtime``
after putting their own repository root first on ``sys.path`` (:25-35), and ``matplotlib`` at module
top (:19-21).  So the drop-in module is registered in ``sys.modules`` under the reference's module
names before the scripts start, and an inert ``matplotlib`` (absent from this image) is provided whose
``subplots`` returns a figure and an axes object, so that the scripts end cleanly.

    python -m bas.refscripts --reference baseline/_ref --out out_dir --batch-sizes 2,16,64

prints one JSON line with the mean kernel speed-up over dense per batch size - the thesis's
headline metric (results/kernel/perstep_actual_kernel_speedup.json:17-54)."""

from __future__ import annotations

import argparse
import contextlib
import io
import json
import runpy
import sys
from pathlib import Path
from unittest import mock


def _register_drop_in() -> None:
    import kernels as drop_in_pkg                                   # this package's drop-in
    import kernels.shared_mask_batched_triton_min_runtime as drop_in

    if not hasattr(drop_in, "_ops"):
        raise ImportError("the module registered as `kernels` is not this package's drop-in")
    sys.modules["kernels"] = drop_in_pkg
    sys.modules["kernels.shared_mask_batched_triton_min_runtime"] = drop_in


def _inert_matplotlib() -> None:
    try:
        import matplotlib  # noqa: F401
        return
    except ImportError:
        pass
    for name in ("matplotlib", "matplotlib.pyplot", "matplotlib.ticker"):
        sys.modules[name] = mock.MagicMock()
    sys.modules["matplotlib"].pyplot = sys.modules["matplotlib.pyplot"]
    sys.modules["matplotlib.pyplot"].subplots.return_value = (mock.MagicMock(), mock.MagicMock())


def _run(script: Path, argv: list, quiet: bool) -> None:
    saved = sys.argv
    sys.argv = [script.name] + argv
    try:
        sink = io.StringIO()
        with (contextlib.redirect_stdout(sink) if quiet else contextlib.nullcontext()):
            try:
                runpy.run_path(str(script), run_name="__main__")
            except SystemExit as exc:
                if exc.code not in (None, 0):
                    raise RuntimeError(f"{script.name} exited with {exc.code}") from exc
    finally:
        sys.argv = saved


def run_thesis_protocol(reference: Path, out_dir: Path, batch_sizes=(2, 16, 64), warmup: int = 30, iterations: int = 100,
                        repeats: int = 2, quiet: bool = True, bench_warmup: int = 80, bench_iters: int = 200,
                        bench_repeats: int = 3) -> dict:
    """Both scripts, in the order of docs/REPRODUCING.md: tuner, then the per-step benchmark.  Returns
    ``{"rows": [{batch_size, kernel_speedup, ...}], "lookup_dir", "out_dir"}``."""
    reference, out_dir = Path(reference).resolve(), Path(out_dir).resolve()
    scripts = reference / "scripts"
    perstep = reference / "results" / "oracle" / "perstep_batch_sweep.json"
    for need in (scripts / "profile_kernel_configs.py", scripts / "bench_perstep_actual_kernel_speedup.py", perstep):
        if not need.exists():
            raise FileNotFoundError(f"{need} is missing (fill it with baseline/fill_ref.py)")
    _register_drop_in()
    _inert_matplotlib()
    lookup = out_dir / "lookup"
    lookup.mkdir(parents=True, exist_ok=True)
    bs = ",".join(str(int(b)) for b in batch_sizes)
    _run(scripts / "profile_kernel_configs.py",
         ["--out_dir", str(lookup), "--batch_sizes", bs, "--warmup", str(warmup), "--iterations", str(iterations),
          "--repeats", str(repeats)], quiet)
    result = out_dir / "perstep"
    _run(scripts / "bench_perstep_actual_kernel_speedup.py",
         ["--perstep_json", str(perstep), "--lookup_dir", str(lookup), "--out_dir", str(result), "--batch_sizes", bs,
          "--warmup", str(bench_warmup), "--iters", str(bench_iters), "--repeats", str(bench_repeats)], quiet)
    data = json.loads((result / "perstep_actual_kernel_speedup.json").read_text())
    return {"rows": data["rows"], "lookup_dir": str(lookup), "out_dir": str(result)}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--reference", default="baseline/_ref", help="root holding the reference's scripts/ and results/")
    ap.add_argument("--out", default="gpurun_out/thesis_protocol")
    ap.add_argument("--batch-sizes", default="2,4,8,16,32,64")
    ap.add_argument("--verbose", action="store_true", help="let the scripts' own progress lines through")
    a = ap.parse_args()
    res = run_thesis_protocol(Path(a.reference), Path(a.out), [int(v) for v in a.batch_sizes.split(",")], quiet=not a.verbose)
    print(json.dumps(res))


if __name__ == "__main__":
    main()
