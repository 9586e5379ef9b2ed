"""The drop-in boundary driven from the reference's side: the reference's portable C++ (its tensor
library, block decoders and test support) linked with tests/shim/cuda_command_context.cpp -- the
reference's backend-buffer factories and MetalCommandContext implemented over the C ABI -- runs the
packed-row projection checks of tests/tensor/gemma3_metal_tests.cpp:1144-1366 on the GPU, and its operator
tests (tied Q6_K embedding and head :511-552, per-head norm and scaled rotation at positions up to 131071
:554-633, the pinned binary16 narrowing cases :87-128, the non-finite status word :130-160, candidate
selection :1112-1142) with the reference's own inputs and tolerances.

The runner is built where the reference tree is available (tests/shim/Makefile, also run by
__graft_entry__.build()); a checkout without it has nothing to run."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
RUNNER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "shim", "_build", "packed_rows_runner")


def test_reference_interface_drives_the_library(gf):
    if not os.path.exists(RUNNER):
        pytest.skip("tests/shim/_build/packed_rows_runner has not been built (needs the reference tree)")
    done = subprocess.run([RUNNER], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    last = done.stdout.strip().splitlines()[-1]
    assert last.startswith("OK ") and int(last.split()[1]) > 1000
    assert done.stdout.count("rows 1-8 invariant") == 14 and done.stdout.count("cancellation K=") == 2


def test_reference_operator_tests_pass_over_the_library(gf):
    runner = os.path.join(os.path.dirname(RUNNER), "operators_runner")
    if not os.path.exists(runner):
        pytest.skip("tests/shim/_build/operators_runner has not been built (needs the reference tree)")
    done = subprocess.run([runner], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    lines = done.stdout.strip().splitlines()
    assert lines[-1].startswith("OK ") and int(lines[-1].split()[1]) > 20000
    assert len(lines) == 7          # embedding/head, two rotation policies, narrowing, status, selection, OK
