"""Runs one dequant-GEMV shape a few times on seeded synthetic blocks: the small, single-kernel
command to put under a profiler.

    python -m guffin_b200.gemv_case <dtype 8|12|14> <K> <N> <rows> [launches]
"""
import sys

import numpy as np

from guffin_b200 import lib, synthetic as syn


def main(argv) -> int:
    dtype, k, n, rows = (int(a) for a in argv[1:5])
    launches = int(argv[5]) if len(argv) > 5 else 3
    L = lib.load()
    rng = np.random.default_rng(0)
    weight = lib.PackedWeight(dtype, k, n, syn.make_weight(rng, dtype, k, n))
    x = lib.DeviceBuffer.from_numpy(rng.standard_normal((rows, k)).astype(np.float32))
    y = lib.DeviceBuffer(rows * n * 4)
    workspace_bytes = L.gf_matmul_workspace_bytes(dtype, rows, k, n)
    workspace = lib.DeviceBuffer(workspace_bytes) if workspace_bytes else None
    for _ in range(launches):
        lib.check(L.gf_matmul(dtype, weight.packed.ptr, x.ptr, y.ptr, rows, k, n, workspace.ptr if workspace else None, None))
    lib.check(L.gf_matmul_check(None))
    print(f"ok: {launches} launches of dtype={dtype} K={k} N={n} rows={rows} ({weight.nbytes / 1e6:.1f} MB of weights)")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
