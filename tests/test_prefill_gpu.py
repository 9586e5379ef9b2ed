"""Prompt ingestion on the tensor cores: the 128-row bf16 GEMM with in-kernel dequantisation
(tcgen05 / TMEM) against the CPU oracle, and chunked prefill against token-at-a-time decoding."""
import numpy as np
import pytest

from guffin_b200 import synthetic as syn

pytestmark = pytest.mark.gpu


def bf16_round(a):
    """Round-to-nearest-even to bfloat16, returned as float32."""
    bits = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    bits = (bits + 0x7fff + ((bits >> 16) & 1)) & 0xffff0000
    return bits.astype(np.uint32).view(np.float32)


def rel_l2(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


@pytest.mark.parametrize("dtype,k,n,rows", [(syn.Q4_K, 512, 128, 128), (syn.Q4_K, 3840, 256, 37), (syn.Q6_K, 1024, 384, 128),
                                             (syn.Q6_K, 256, 128, 1), (syn.Q8_0, 640, 256, 100), (syn.Q8_0, 128, 128, 128),
                                             (syn.Q4_K, 15360, 128, 128)])
def test_prefill_matmul_matches_bf16_reference_and_oracle(gf, oracle, dtype, k, n, rows):
    """Against the same product with both operands rounded to bf16 and summed in double precision the
    kernel may differ only by its f32 accumulation (1e-5: a layout or descriptor mistake shows as an
    error of order one); against the f32 oracle by the bf16 rounding of the operands (stated
    tolerance 1e-2 relative L2, measured about 3e-3).  Rows beyond the live ones come back zero."""
    rng = np.random.default_rng(k + n + rows)
    native = syn.make_weight(rng, dtype, k, n)
    weight = gf.PackedWeight(dtype, k, n, native)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    got = gf.prefill_matmul(weight, x)
    assert got.shape == (128, n)
    w = oracle.dequantize(dtype, native).reshape(n, k)
    exact = bf16_round(x).astype(np.float64) @ bf16_round(w).astype(np.float64).T
    assert rel_l2(got[:rows], exact) < 1e-5
    assert np.abs(got[:rows] - exact).max() <= 1e-4 * np.abs(exact).max()
    want = oracle.matmul(dtype, x, native, k, n)
    assert rel_l2(got[:rows], want) < 1e-2
    assert not got[rows:].any()
    weight.packed.free()
