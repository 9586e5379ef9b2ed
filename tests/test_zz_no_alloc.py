"""gf_matmul_static: the projection for callers that cannot allocate device memory (its split-K
scratch is a fixed array inside the library).  Collected last on purpose: if it fails, a run
that stops at the first failure has already exercised everything else."""
import numpy as np
import pytest

from guffin_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


def _static(gf, weight, x_dev, y_dev, rows):
    L = gf.load()
    gf.check(L.gf_matmul_static(weight.dtype, weight.packed.ptr, x_dev.ptr, y_dev.ptr, rows, weight.k, weight.n, None))
    gf.check(L.gf_stream_synchronize(None))
    return y_dev.download(np.float32).reshape(rows, weight.n)


@pytest.mark.parametrize("dtype,k,n,rows", [(syn.Q4_K, 4096, 3840, 2), (syn.Q6_K, 15360, 256, 1), (syn.Q8_0, 2048, 640, 2),
                                             (syn.Q4_K, 3840, 15360, 2)])
def test_static_scratch_matmul_matches_matmul_twice_in_a_row(gf, dtype, k, n, rows):
    """Same bytes as gf_matmul (the split is identical, so the floats are too), on two
    back-to-back calls with different activations: the second call must not see the first
    call's counters or partial sums."""
    rng = np.random.default_rng(k + n)
    weight = gf.PackedWeight(dtype, k, n, syn.make_weight(rng, dtype, k, n))
    y_dev = gf.DeviceBuffer(rows * n * 4)
    for call in range(2):
        x = rng.standard_normal((rows, k)).astype(np.float32)
        x_dev = gf.DeviceBuffer.from_numpy(x)
        want = gf.matmul(weight, x)
        got = _static(gf, weight, x_dev, y_dev, rows)
        np.testing.assert_array_equal(got, want)
        x_dev.free()
    y_dev.free()
    weight.packed.free()


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
