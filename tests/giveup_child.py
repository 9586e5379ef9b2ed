"""Child process of tests/test_giveup_gpu.py: runs against the TESTING build of the library (the one
with the host-side fault seam), makes one bounded device-side wait run out on purpose, and prints
what the C ABI reported as one JSON line.  Nothing here faults or hangs the GPU: every copy the
kernels ask for still lands, only a wait expires.

    python -m tests.giveup_child matmul | static | model | pass
"""
import ctypes as C
import json
import sys

import numpy as np

from guffin_b200 import build, lib

lib.LIB_PATH = build.TESTING_LIB          # before anything loads the shipped library
from guffin_b200 import model as gm, synthetic as syn  # noqa: E402


def status_of(call):
    try:
        call()
        return 0
    except lib.GuffinError as error:
        return error.status


def main(scenario: str) -> dict:
    L = lib.load()
    L.gf_testing_arm_fault.argtypes = [C.c_int, C.c_uint32]
    L.gf_testing_arm_fault.restype = C.c_int
    rng = np.random.default_rng(3)
    out = {"scenario": scenario}
    if scenario in ("matmul", "static"):
        dtype, k, n, rows = syn.Q4_K, 3840, 512, 2
        weight = lib.PackedWeight(dtype, k, n, syn.make_weight(rng, dtype, k, n))
        x = rng.standard_normal((rows, k)).astype(np.float32)
        want = lib.matmul(weight, x)
        xd, yd = lib.DeviceBuffer.from_numpy(x), lib.DeviceBuffer(rows * n * 4)
        run = (lambda: L.gf_matmul(dtype, weight.packed.ptr, xd.ptr, yd.ptr, rows, k, n, None, None)) if scenario == "matmul" \
            else (lambda: L.gf_matmul_static(dtype, weight.packed.ptr, xd.ptr, yd.ptr, rows, k, n, None))
        check = L.gf_matmul_check if scenario == "matmul" else L.gf_matmul_static_check
        other = L.gf_matmul_static_check if scenario == "matmul" else L.gf_matmul_check
        assert run() == 0 and check(None) == 0                       # healthy call first
        lib.check(L.gf_testing_arm_fault(1, 1024))
        out["launch"] = run()
        out["other_check"] = other(None)                              # the other entry point's error word is untouched
        out["check"] = check(None)                                    # GF_ERR_TIMEOUT, read and cleared
        out["check_again"] = check(None)
        out["launch_after"] = run()
        out["check_after"] = check(None)
        out["equal_after"] = bool(np.array_equal(yd.download(np.float32).reshape(rows, n), want))
        return out
    config = syn.model_config("tiny-target")
    weights = syn.make_model_weights("tiny-target", 91)
    tokens = rng.integers(0, config["vocab"], 24).astype(np.uint32)
    model = gm.Model(config, weights, 64, 2)
    model.use_pass_kernel(1 if scenario == "pass" else 0)
    model.use_graph(False)                                            # the fault is consumed when a launch is prepared
    model.prefill(tokens[:9])
    model.forward(tokens[9:11], logits=True)
    healthy = model.logits(1).copy()
    assert model.status() == 0
    lib.check(L.gf_testing_arm_fault(2 if scenario == "pass" else 1, 4096 if scenario == "pass" else 1024))
    out["forward"] = status_of(lambda: model.forward(tokens[9:11], logits=True))     # enqueues; the kernel gives up on the device
    out["status"] = status_of(model.status)                           # GF_ERR_TIMEOUT
    out["forward_poisoned"] = status_of(lambda: model.forward(tokens[9:11], logits=True))   # GF_ERR_STATE until reset
    model.reset()
    model.prefill(tokens[:9])
    model.forward(tokens[9:11], logits=True)
    out["status_after_reset"] = status_of(model.status)
    out["equal_after_reset"] = bool(np.array_equal(model.logits(1), healthy))
    return out


if __name__ == "__main__":
    print(json.dumps(main(sys.argv[1])))
