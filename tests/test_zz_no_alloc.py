"""gf_matmul_static: the projection for callers that cannot allocate device memory (its split-K
scratch is a fixed array inside the library).  Collected last on purpose: if it fails, a run
that stops at the first failure has already exercised everything else."""
import ctypes as C

import numpy as np
import pytest

from guffin_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


def _free_bytes(gf):
    free, total = C.c_size_t(), C.c_size_t()
    gf.check(gf.load().gf_memory_info(C.byref(free), C.byref(total)))
    return free.value


def _static(gf, weight, x_dev, y_dev, rows):
    L = gf.load()
    gf.check(L.gf_matmul_static(weight.dtype, weight.packed.ptr, x_dev.ptr, y_dev.ptr, rows, weight.k, weight.n, None))
    gf.check(L.gf_matmul_static_check(None))            # synchronises; GF_OK means no wait gave up
    return y_dev.download(np.float32).reshape(rows, weight.n)


# The last three shapes split K across CTAs at two rows (the 12B ffn_down shape in both of its block
# formats: nine chunks, 276 KB of partial sums; and a narrow, very deep one), so their arrival counters
# and partial sums really live in the built-in array; the first three need no scratch or one row only.
SHAPES = [(syn.Q4_K, 4096, 3840, 2), (syn.Q6_K, 15360, 256, 1), (syn.Q8_0, 2048, 640, 2),
          (syn.Q4_K, 15360, 3840, 2), (syn.Q6_K, 15360, 3840, 2), (syn.Q4_K, 65536, 256, 2)]


@pytest.mark.parametrize("dtype,k,n,rows", SHAPES)
def test_static_scratch_matmul_matches_matmul_twice_in_a_row(gf, dtype, k, n, rows):
    """Same bytes as gf_matmul (the split is identical, so the floats are too), on two
    back-to-back calls with different activations: the second call must not see the first
    call's counters or partial sums.  Device memory in use is the same before and after the
    static calls: the entry point allocates nothing."""
    L = gf.load()
    rng = np.random.default_rng(k + n)
    weight = gf.PackedWeight(dtype, k, n, syn.make_weight(rng, dtype, k, n))
    if (dtype, k, n, rows) in SHAPES[3:]:
        assert L.gf_matmul_workspace_bytes(dtype, rows, k, n) > 0          # the case that uses the array
    y_dev = gf.DeviceBuffer(rows * n * 4)
    inputs = [rng.standard_normal((rows, k)).astype(np.float32) for _ in range(2)]
    wants = [gf.matmul(weight, x) for x in inputs]
    x_devs = [gf.DeviceBuffer.from_numpy(x) for x in inputs]
    gf.check(L.gf_stream_synchronize(None))
    _static(gf, weight, x_devs[0], y_dev, rows)           # the first call on a device looks the array's address up
    before = _free_bytes(gf)
    for x_dev, want in zip(x_devs, wants):
        got = _static(gf, weight, x_dev, y_dev, rows)
        np.testing.assert_array_equal(got, want)
    assert _free_bytes(gf) == before
    for buffer in x_devs:
        buffer.free()
    y_dev.free()
    weight.packed.free()


def test_two_split_shapes_back_to_back_on_one_stream(gf):
    """Two different split-K shapes share the array's counters: queued on one stream without a
    host synchronisation between them, each must start from zeroed counters of its own size."""
    L = gf.load()
    rng = np.random.default_rng(5)
    cases = []
    for dtype, k, n in ((syn.Q6_K, 15360, 3840), (syn.Q4_K, 65536, 256), (syn.Q4_K, 15360, 3840)):
        weight = gf.PackedWeight(dtype, k, n, syn.make_weight(rng, dtype, k, n))
        x = rng.standard_normal((2, k)).astype(np.float32)
        cases.append((weight, gf.DeviceBuffer.from_numpy(x), gf.DeviceBuffer(2 * n * 4), gf.matmul(weight, x)))
    for _ in range(2):
        for weight, x_dev, y_dev, _ in cases:
            gf.check(L.gf_matmul_static(weight.dtype, weight.packed.ptr, x_dev.ptr, y_dev.ptr, 2, weight.k, weight.n, None))
        gf.check(L.gf_matmul_static_check(None))
        for weight, _, y_dev, want in cases:
            np.testing.assert_array_equal(y_dev.download(np.float32).reshape(2, weight.n), want)
    for weight, x_dev, y_dev, _ in cases:
        x_dev.free(); y_dev.free(); weight.packed.free()


def test_static_scratch_rejects_shapes_beyond_its_capacity(gf):
    L = gf.load()
    assert L.gf_matmul_static_capacity() == 8 << 20
    # Four rows over K = 65536 cannot keep their activations in one CTA's shared memory, so K must
    # split, and 2^18 columns of partial sums per chunk exceed the array.  The size check comes
    # first, so no buffers are needed to see the refusal.
    assert L.gf_matmul_workspace_bytes(syn.Q8_0, 4, 1 << 16, 1 << 18) > L.gf_matmul_static_capacity()
    status = L.gf_matmul_static(syn.Q8_0, None, None, None, 4, 1 << 16, 1 << 18, None)
    assert status == gf.GF_ERR_INVALID
    message = L.gf_last_error()
    assert b"scratch" in message and str(8 << 20).encode() in message
