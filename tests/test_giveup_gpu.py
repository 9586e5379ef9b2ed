"""The give-up path of the bounded device-side waits, run on purpose without faulting anything.

The shipped library has no way to make a wait expire, so these tests drive the TESTING build
(guffin_b200/libguffin_b200_testing.so, -DGF_TESTING) in a child process: a one-shot host-side seam
makes the next weight-streaming launch claim 16 bytes more than its first copy brings and poll only
1024 times, or makes one CTA of the next decode pass kernel leave out a barrier arrival.  All copies
land, a wait runs out, the kernel returns with its error word set.  This is the reference's pattern
of host-side failure points compiled only into test builds (tests/support/target_verifier_test_hooks.cpp,
src/engine/target_verifier_runtime.cpp:355-357) applied to the device-side waits."""
import json
import os
import subprocess
import sys

import pytest

from guffin_b200 import lib

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_child(scenario):
    proc = subprocess.run([sys.executable, "-m", "tests.giveup_child", scenario], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    return json.loads(proc.stdout.strip().splitlines()[-1])


@pytest.mark.parametrize("scenario", ["matmul", "static"])
def test_streaming_wait_that_gives_up_is_reported_once_and_only_by_its_own_check(gf, scenario):
    """gf_matmul / gf_matmul_static: the launch itself succeeds, the matching check returns
    GF_ERR_TIMEOUT exactly once (the static entry point's word lives in the library's static storage
    and is read without allocating), the other entry point's check stays clean, and the next call
    computes the same floats as before."""
    out = run_child(scenario)
    assert out["launch"] == 0 and out["other_check"] == 0
    assert out["check"] == lib.GF_ERR_TIMEOUT and out["check_again"] == 0
    assert out["launch_after"] == 0 and out["check_after"] == 0 and out["equal_after"]


@pytest.mark.parametrize("scenario", ["model", "pass"])
def test_plan_is_poisoned_by_a_wait_that_gives_up_and_reset_restores_it(gf, scenario):
    """A resident plan whose pass contained the expired wait (a weight ring wait in the
    kernel-per-operator schedule; a grid barrier of the decode pass kernel): gf_model_status returns
    GF_ERR_TIMEOUT, the poisoned plan refuses further passes with GF_ERR_STATE, and after
    gf_model_reset the same tokens give bit-identical logits."""
    out = run_child(scenario)
    assert out["forward"] == 0
    assert out["status"] == lib.GF_ERR_TIMEOUT
    assert out["forward_poisoned"] == lib.GF_ERR_STATE
    assert out["status_after_reset"] == 0 and out["equal_after_reset"]
