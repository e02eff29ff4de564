#!/usr/bin/env python
"""Fill the git-ignored ``baseline/_ref/`` with the parts of the reference that the benchmark runs
beside this repository's kernels on the GPU box (which has no copy of the reference):

* ``kernels/``  - the reference's Triton module, timed as "the existing kernel on this GPU";
* ``scripts/profile_kernel_configs.py``, ``scripts/bench_perstep_actual_kernel_speedup.py`` - run
  UNMODIFIED against this repository's drop-in module (``bas/refscripts.py``);
* ``results/oracle/perstep_batch_sweep.json`` - the thesis's per-step oracle schedules they replay.

    python baseline/fill_ref.py [/path/to/reference]

Nothing here is imported by the package; the copies never enter the history (``.gitignore``) but do
travel to the GPU box with the working tree.  The reference has no ``setup.py`` / ``pyproject.toml``,
so there is nothing to ``pip install``: its scripts find ``kernels`` through their own ``sys.path``."""

from __future__ import annotations

import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
WANTED = ["kernels", "scripts/profile_kernel_configs.py", "scripts/bench_perstep_actual_kernel_speedup.py",
          "results/oracle/perstep_batch_sweep.json"]


def fill(reference: Path, dest: Path = HERE / "_ref") -> Path:
    if not reference.is_dir():
        raise SystemExit(f"{reference} is not a directory")
    dest.mkdir(parents=True, exist_ok=True)
    for rel in WANTED:
        src, dst = reference / rel, dest / rel
        if src.is_dir():
            shutil.copytree(src, dst, dirs_exist_ok=True, ignore=shutil.ignore_patterns("__pycache__"))
        else:
            dst.parent.mkdir(parents=True, exist_ok=True)
            shutil.copy2(src, dst)
    return dest


if __name__ == "__main__":
    print(fill(Path(sys.argv[1] if len(sys.argv) > 1 else "/root/reference")))
