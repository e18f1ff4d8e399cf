"""With `spear_b200.install_as_spear_backend()`, the UNMODIFIED reference package imports and its
wrapper reaches this package's binding.  Uses the copy of the reference that oracle/stage_reference.py staged
under oracle/_ref (or the checkout SPEAR_REFERENCE names); skipped where neither exists.  Runs in a child
process because both packages define the `spear_btp` ops."""

from __future__ import annotations

import os
import subprocess
import sys

import pytest

from conftest import ROOT

REFERENCE = os.environ.get("SPEAR_REFERENCE") or os.path.join(ROOT, "oracle", "_ref")

CHILD = r"""
import sys, inspect
sys.path.insert(0, {root!r}); sys.path.insert(0, {ref!r})
import spear_b200
import spear_b200._btp as native
spear = spear_b200.install_as_spear_backend()   # imports the reference package, unmodified
from spear.ops.btp import btp as ref_btp
from spear.ops.btp import interface as ref_iface
from spear_b200.ops.btp import btp as our_btp   # registers nothing twice: the ops already exist
assert ref_iface.spear._btp is native
ref_sig = list(inspect.signature(ref_btp).parameters)
our_sig = list(inspect.signature(our_btp).parameters)
assert our_sig[:len(ref_sig)] == ref_sig, (ref_sig, our_sig)
assert inspect.signature(native.forward).parameters.keys() >= {{"coeff", "x", "y", "checkpoint", "k", "wpb"}}
import torch
from spear.nn.phalanx import Phalanx as RefPhalanx
from spear_b200.nn.phalanx import Phalanx as OurPhalanx
ref_args = inspect.signature(RefPhalanx.__init__).parameters
our_args = inspect.signature(OurPhalanx.__init__).parameters
assert list(ref_args) == list(our_args)
assert all(ref_args[k].default == our_args[k].default for k in ref_args)
r, o = RefPhalanx(dim=64, dtype=torch.bfloat16, kv_heads=2), OurPhalanx(dim=64, dtype=torch.bfloat16, kv_heads=2)
assert list(r.state_dict()) == list(o.state_dict())
o.load_state_dict(r.state_dict())
try:
    ref_btp(torch.rand(1, 2, 32), torch.rand(1, 2, 16, 32))   # CPU tensors: must fail loudly, not fall back
except (RuntimeError, NotImplementedError):
    print("DROPIN-OK")
"""


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "spear")), reason="reference checkout not present")
def test_reference_package_runs_on_this_binding():
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    r = subprocess.run([sys.executable, "-c", CHILD.format(root=ROOT, ref=REFERENCE)], env=env, capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "DROPIN-OK" in r.stdout
