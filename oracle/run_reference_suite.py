#!/usr/bin/env python
"""Runs the reference's OWN pytest suites on a GPU with this repository's binding as `spear._btp`.

    python oracle/run_reference_suite.py [--junit out.xml] [pytest selection ...]

Test infrastructure, not a product path.  `oracle/stage_reference.py` has placed the unmodified reference
package and its tests under `oracle/_ref/`.  This script registers `spear_b200._btp` as the compiled
extension the reference imports (spear/ops/btp/interface.py:16) and then hands the selected test files of
the reference (default: tests/btp and tests/phalanx, whole) to pytest in this process.  Everything above the
extension - the reference's `btp()` wrapper, its autograd function and custom-op registration, its `Phalanx`
layer, its samplers, PyTorch references, metrics and tolerances - is the reference's own code.

The reference's pytest options (coverage plugin, strict markers; pyproject.toml:103-116) are not applied: no
configuration file travels with the staged tests.
"""

from __future__ import annotations

import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.path.join(HERE, "_ref")


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--junit", default=None, help="write a JUnit XML report here")
    ap.add_argument("selection", nargs="*", help="paths (relative to the staged reference) and -k/-x style options")
    args, extra = ap.parse_known_args()
    if not os.path.isdir(os.path.join(REF, "spear")) or not os.path.isdir(os.path.join(REF, "tests")):
        raise SystemExit(f"{REF} holds no staged reference: run oracle/stage_reference.py where the reference is mounted")
    sys.path[:0] = [ROOT, REF]
    os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
    sys.dont_write_bytecode = True

    import spear_b200

    spear = spear_b200.install_as_spear_backend()
    if not os.path.abspath(spear.__file__).startswith(REF + os.sep):
        raise SystemExit(f"`import spear` resolved to {spear.__file__}, not to the staged reference")

    import pytest

    tests = os.path.join(REF, "tests")
    selection = [a if a.startswith("-") else os.path.join(REF, a) for a in args.selection] or [tests]
    argv = ["-q", "-p", "no:cacheprovider", "--rootdir", tests, "--confcutdir", tests, "-o", "addopts=", "-rA"]
    if args.junit:
        argv += ["--junitxml", args.junit]
    return int(pytest.main(argv + extra + selection))


if __name__ == "__main__":
    sys.exit(main())
