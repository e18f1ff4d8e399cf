#!/usr/bin/env python
"""Stages the UNMODIFIED reference checkout where the tests and the benchmark's reference arm can reach it.

    python oracle/stage_reference.py /path/to/reference      (or set SPEAR_REFERENCE)

Test infrastructure, not a product path.  The reference's Python package (`spear/`) and its own test suites
(`tests/btp/`, `tests/phalanx/`) are placed, byte for byte, under the git-ignored `oracle/_ref/`, next to the
reference CUDA extension that `oracle/build_reference_kernel.sh` builds there.  Nothing is added to the tracked
tree.  The machines that run the GPU tests have no reference checkout; they get `oracle/_ref/` together with
the other built artefacts.  Users:

  * `bench.py --impl reference` and its `cpu_baseline` leg time the reference's own
    `spear/ops/btp/reference.py::block_two_pass_log` on the host cores;
  * `oracle/run_reference_suite.py` runs the reference's own pytest suites on a GPU with this repository's
    binding standing in for the reference's compiled extension `spear._btp`.

A file `oracle/_ref/STAGED` lists what was staged with SHA-256 digests, so that a test can tell whether the
staged copy is complete and untouched.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
PARTS = ("spear", os.path.join("tests", "btp"), os.path.join("tests", "phalanx"))


def default_reference() -> str | None:
    """SPEAR_REFERENCE, else a checkout named `reference` beside this repository."""
    cand = os.environ.get("SPEAR_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "spear", "ops", "btp")) else None


def _digest(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        h.update(f.read())
    return h.hexdigest()


def staged_files() -> dict[str, str]:
    """{relative path: sha256} recorded by the last staging run ({} when nothing is staged)."""
    manifest = os.path.join(OUT, "STAGED")
    if not os.path.exists(manifest):
        return {}
    with open(manifest) as f:
        return dict(line.rstrip("\n").split("  ", 1)[::-1] for line in f if line.strip())


def is_staged() -> bool:
    files = staged_files()
    return bool(files) and all(os.path.exists(os.path.join(OUT, rel)) for rel in files)


def verify() -> list[str]:
    """Relative paths whose staged copy is missing or differs from what was staged."""
    bad = []
    for rel, digest in staged_files().items():
        p = os.path.join(OUT, rel)
        if not os.path.exists(p) or _digest(p) != digest:
            bad.append(rel)
    return bad


def stage(reference: str) -> int:
    os.makedirs(OUT, exist_ok=True)
    lines = []
    for part in PARTS:
        src, dst = os.path.join(reference, part), os.path.join(OUT, part)
        if not os.path.isdir(src):
            raise SystemExit(f"{src} does not exist: not a checkout of the reference")
        if os.path.isdir(dst):
            shutil.rmtree(dst)
        shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__", "*.pyc", "*.so"))
        for root, _, names in os.walk(dst):
            for name in sorted(names):
                p = os.path.join(root, name)
                lines.append(f"{_digest(p)}  {os.path.relpath(p, OUT)}")
    with open(os.path.join(OUT, "STAGED"), "w") as f:
        f.write("\n".join(sorted(lines)) + "\n")
    return len(lines)


if __name__ == "__main__":
    ref = sys.argv[1] if len(sys.argv) > 1 else default_reference()
    if not ref:
        raise SystemExit("give the path of the reference checkout (argument or SPEAR_REFERENCE)")
    print(f"staged {stage(ref)} files of {ref} under {OUT}")
