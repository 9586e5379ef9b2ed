"""Runs the decode attention operator a few times on seeded synthetic caches: the small,
single-kernel command to put under a profiler.

    python -m guffin_b200.attention_case <cached rows> <rows> <heads> <kv_heads> <window> <kv_f16 0|1> [launches]
"""
import sys

import numpy as np

from guffin_b200 import lib, model  # noqa: F401  (model declares the operator signatures)


def main(argv) -> int:
    base, rows, heads, kv_heads, window, kv_f16 = (int(a) for a in argv[1:7])
    launches = int(argv[7]) if len(argv) > 7 else 3
    L = lib.load()
    rng = np.random.default_rng(0)
    ring_rows = 1 << max(1, int(np.ceil(np.log2(base + rows))))
    kv_dtype = np.float16 if kv_f16 else np.float32
    q = rng.standard_normal((rows, heads * 256)).astype(np.float32)
    ring = [rng.standard_normal((ring_rows, kv_heads * 256)).astype(kv_dtype) for _ in range(2)]
    private = [rng.standard_normal((rows, kv_heads * 256)).astype(kv_dtype) for _ in range(2)]
    buffers = [lib.DeviceBuffer.from_numpy(a) for a in (q, ring[0], ring[1], private[0], private[1])]
    out = lib.DeviceBuffer(q.nbytes)
    workspace = lib.DeviceBuffer(L.gf_attention_workspace_bytes(rows, heads))
    position = lib.DeviceBuffer.from_numpy(np.array([base], np.uint32))
    for _ in range(launches):
        lib.check(L.gf_attention(buffers[0].ptr, buffers[1].ptr, buffers[2].ptr, buffers[3].ptr, buffers[4].ptr, out.ptr,
                                 workspace.ptr, position.ptr, rows, heads, kv_heads, 256, ring_rows, window,
                                 1.0 / 16.0, 0.0, kv_f16, None))
    result = out.download(np.float32)
    kv_bytes = 2 * kv_heads * 256 * (2 if kv_f16 else 4) * (min(base, window) if window else base)
    print(f"ok: {launches} launches, base={base} rows={rows} heads={heads}/{kv_heads} window={window}, "
          f"{kv_bytes / 1e6:.2f} MB of K/V per row, |out| = {float(np.abs(result).mean()):.4f}")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
