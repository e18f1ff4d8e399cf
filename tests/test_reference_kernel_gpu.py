"""Accuracy next to the reference's own CUDA kernels.

The reference kernels (its csrc/btp sources compiled for sm_100 by oracle/build_reference_kernel.sh into the
git-ignored oracle/_ref/_btp.so) and the kernels of this repository run on identical seeded inputs; both are
compared with the float64 oracle.  The bar: relative L2 error of y, dx and dA no larger than the reference
kernel's own.  Skipped where the yardstick library has not been built.  Only shapes whose sequences fit one CTA of
the reference kernel are used (L/16 <= wpb): there none of its cluster-barrier waits is entered."""

from __future__ import annotations

import os

import pytest
import torch

from conftest import ROOT

pytestmark = pytest.mark.gpu

REF_LIB = os.path.join(ROOT, "oracle", "_ref", "_btp.so")


@pytest.mark.skipif(not os.path.exists(REF_LIB), reason="oracle/_ref/_btp.so has not been built")
@pytest.mark.parametrize("B,H,L,wpb", [(256, 32, 128, 32), (256, 32, 128, 8), (2, 8, 512, 32), (8, 4, 64, 4)])
def test_errors_are_no_larger_than_the_reference_kernels(B, H, L, wpb):
    import compare_reference_kernel as C  # oracle/ is on sys.path (conftest)
    from spear_b200 import _btp as ours

    assert L // 16 <= wpb
    ref = C.load_reference_extension()
    res = C.run(B, H, L, wpb, ref, ours, nsets=1)
    for key in ("rel_l2_y", "rel_l2_dx", "rel_l2_dA"):
        mine, theirs = res["this_repo"][key], res["reference_kernel"][key]
        assert mine <= 1e-2, f"{key} {mine:.3e}"
        assert mine <= theirs, f"{key}: {mine:.4e} here, {theirs:.4e} in the reference kernel"
