"""GPU parity for weight preparation, dequantisation and the streaming dequant-GEMV, through
the C ABI, against the CPU oracle on identical seeded bytes."""
import numpy as np
import pytest

from guffin_b200 import synthetic as syn
from tests import blocks
from tests.golden import make_golden as golden

pytestmark = pytest.mark.gpu
DTYPES = [syn.Q4_K, syn.Q6_K, syn.Q8_0]


def rel_l2(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n", [8, 9, 64, 61])
def test_pack_round_trip_is_lossless(gf, dtype, n):
    k = 768 if dtype != syn.Q8_0 else 640
    rng = np.random.default_rng(n * 7 + dtype)
    native = syn.make_weight(rng, dtype, k, n)
    weight = gf.PackedWeight(dtype, k, n, native)
    np.testing.assert_array_equal(weight.unpack(), native)
    if n % 16:     # missing columns of the last group of sixteen are zero bytes
        padded = (n + 15) // 16 * 16
        column_bytes = native.size // n
        extended = np.concatenate([native, np.zeros((padded - n) * column_bytes, np.uint8)])
        np.testing.assert_array_equal(weight.packed.download(np.uint8),
                                      gf.PackedWeight(dtype, k, padded, extended).packed.download(np.uint8))


def test_weight_transforms_bit_exact(gf, oracle):
    """The Gemma 2 load-time transforms on the device against the reference's own bytes (the committed
    fixture made by the compiled reference) and against the CPU oracle on fresh blocks."""
    want, d = np.load(golden.HERE / "ref_requant.npz"), golden.requant_inputs()
    status, q8 = gf.quantize_f16_q8_0(d["f16"])
    assert status == 0
    np.testing.assert_array_equal(q8, want["q8"])
    status, q4 = gf.requantize_q6k_q4k(d["q6k"])
    assert status == 0
    np.testing.assert_array_equal(q4, want["q4"])
    rng = np.random.default_rng(5)
    for sigma in (1e-3, 0.05, 2.0):                                   # 10,000 blocks per scale of d
        q6k = syn.make_weight(rng, syn.Q6_K, 2560, 1000, sigma=sigma)
        status, q4 = gf.requantize_q6k_q4k(q6k)
        rc, q4_cpu = oracle.requantize_q6k_q4k(q6k)
        assert status == 0 and rc == 0
        np.testing.assert_array_equal(q4, q4_cpu)
    values = (rng.standard_normal(3584 * 300) * rng.choice([1e-4, 1e-2, 1.0, 60.0], 3584 * 300)).astype(np.float16)
    status, q8 = gf.quantize_f16_q8_0(values.view(np.uint16))
    rc, q8_cpu = oracle.quantize_f16_q8_0(values.view(np.uint16))
    assert status == 0 and rc == 0
    np.testing.assert_array_equal(q8, q8_cpu)
    bad = values.view(np.uint16).copy()
    bad[77] = 0x7c00                                                  # infinity: the reference throws, the device flags it
    assert gf.quantize_f16_q8_0(bad)[0] == 1


@pytest.mark.parametrize("dtype", DTYPES)
def test_dequantize_bit_exact(gf, oracle, dtype):
    rng = np.random.default_rng(dtype)
    native = syn.make_weight(rng, dtype, 1024, 37, sigma=0.05)
    np.testing.assert_array_equal(gf.dequantize(dtype, native), oracle.dequantize(dtype, native))


def test_dequantize_reference_known_answers(gf):
    block, expected = blocks.reference_q8_0_kat()
    values = gf.dequantize(syn.Q8_0, block)
    assert all(values[i] == np.float32(v) for i, v in expected.items())
    block, expected, _, _ = blocks.reference_q4_k_kat()
    values = gf.dequantize(syn.Q4_K, block)
    assert all(values[i] == np.float32(v) for i, v in expected.items())
    block, expected, _, _ = blocks.reference_q6_k_kat()
    values = gf.dequantize(syn.Q6_K, block)
    assert all(values[i] == np.float32(v) for i, v in expected.items())


def test_dequantize_matches_reference_fixture(gf):
    want, data = np.load(golden.HERE / "ref_ops.npz"), golden.ops_inputs()
    for name, dtype in (("q4k", syn.Q4_K), ("q6k", syn.Q6_K), ("q80", syn.Q8_0)):
        np.testing.assert_array_equal(gf.dequantize(dtype, data[f"{name}_w"]), want[f"{name}_deq"])


SHAPES = {
    # (K, N): unit tails, odd column counts, split-K shapes, one-unit matrices
    syn.Q4_K: [(256, 8), (3840, 64), (768, 61), (4096, 200), (2048, 7), (15360, 16)],
    syn.Q6_K: [(256, 8), (3840, 64), (768, 61), (15360, 24), (4096, 33)],
    syn.Q8_0: [(128, 8), (640, 256), (2048, 61), (1024, 640), (640, 1000)],
}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [1, 2, 3, 4, 6, 8])
def test_matmul_matches_oracle(gf, oracle, dtype, rows):
    for k, n in SHAPES[dtype]:
        rng = np.random.default_rng(k * 31 + n * 7 + rows)
        native = syn.make_weight(rng, dtype, k, n, sigma=0.02)
        x = rng.standard_normal((rows, k)).astype(np.float32)
        weight = gf.PackedWeight(dtype, k, n, native)
        got = gf.matmul(weight, x)
        exact, abs_sum = oracle.matmul_f64(dtype, x, native, k, n)
        # gamma_n * sum|x*w| + 1e-6 with n = K/32 + 32: the bound the reference holds its own
        # packed-row kernels to (tests/tensor/gemma3_metal_tests.cpp:1271-1285).
        terms = k / 32 + 32
        unit = 2.0 ** -24
        bound = (terms * unit / (1 - terms * unit)) * abs_sum + 1e-6
        assert np.all(np.abs(got - exact) <= bound), (dtype, k, n, np.abs(got - exact).max(), bound.min())
        assert rel_l2(got, oracle.matmul(dtype, x, native, k, n)) < 1e-5     # north-star gate is 1e-3
        weight.packed.free()


@pytest.mark.parametrize("dtype,k,n", [(syn.Q4_K, 3840, 512), (syn.Q6_K, 15360, 64), (syn.Q8_0, 640, 2048)])
def test_rows_are_count_invariant(gf, dtype, k, n):
    """A row's floats are identical whether it is computed alone or beside other rows
    (tests/tensor/gemma3_metal_tests.cpp:1223-1256)."""
    rng = np.random.default_rng(99)
    native = syn.make_weight(rng, dtype, k, n)
    weight = gf.PackedWeight(dtype, k, n, native)
    x = rng.standard_normal((8, k)).astype(np.float32)
    together = gf.matmul(weight, x)
    for rows in (1, 2, 3, 4, 5, 7):
        np.testing.assert_array_equal(gf.matmul(weight, x[:rows]), together[:rows])
    np.testing.assert_array_equal(gf.matmul(weight, x[2:3]), together[2:3])
    np.testing.assert_array_equal(gf.matmul(weight, x[6:8]), together[6:8])
    np.testing.assert_array_equal(gf.matmul_host(weight, x[:2]), together[:2])


@pytest.mark.parametrize("dtype,k,n", [(syn.Q4_K, 3840, 65536), (syn.Q6_K, 3840, 32768)])
def test_rows_are_count_invariant_on_wide_matrices(gf, dtype, k, n):
    """At widths where the chunk limit of the planner binds: row counts 1 to 4 (decode and
    verification) give bit-identical rows, and so do 5 to 8 among themselves; the eight-row
    instance stages a smaller activation slice, may therefore split K differently, and then
    differs from the narrow instances by rounding only."""
    rng = np.random.default_rng(7)
    weight = gf.PackedWeight(dtype, k, n, syn.make_weight(rng, dtype, k, n))
    x = rng.standard_normal((8, k)).astype(np.float32)
    narrow = gf.matmul(weight, x[:4])
    for rows in (1, 2, 3):
        np.testing.assert_array_equal(gf.matmul(weight, x[:rows]), narrow[:rows])
    wide = gf.matmul(weight, x)
    for rows in (5, 6, 7):
        np.testing.assert_array_equal(gf.matmul(weight, x[:rows]), wide[:rows])
    assert rel_l2(wide[:4], narrow) < 1e-6
    weight.packed.free()


@pytest.mark.parametrize("dtype,k,n", [(syn.Q4_K, 3840, 64), (syn.Q6_K, 768, 40), (syn.Q8_0, 640, 48)])
def test_non_finite_activation_poisons_its_row_only(gf, dtype, k, n):
    """An infinity or NaN among the activations of a row makes that row's outputs NaN (the f32
    reference propagates them through the dot product); the other row is untouched."""
    rng = np.random.default_rng(5)
    weight = gf.PackedWeight(dtype, k, n, syn.make_weight(rng, dtype, k, n))
    x = rng.standard_normal((2, k)).astype(np.float32)
    clean = gf.matmul(weight, x)
    for bad in (np.inf, np.nan):
        poisoned = x.copy()
        poisoned[1, k // 3] = bad
        y = gf.matmul(weight, poisoned)
        np.testing.assert_array_equal(y[0], clean[0])
        assert np.isnan(y[1]).all()


def test_q4k_scale_min_cancellation(gf, oracle):
    """Large d*scale*q against large dmin*min: the adversarial case of
    tests/tensor/gemma3_metal_tests.cpp:1291-1365."""
    k, n = 3840, 16
    scales, minima = [63] * 8, [63] * 8
    nibbles = [15 if i % 2 == 0 else 14 for i in range(256)]
    block = blocks.q4k_block(blocks.f16_bits(4.0), blocks.f16_bits(59.0 / 63.0 * 63.0 / 59.0 * 59.5), scales, minima, nibbles)
    native = np.tile(block, n * (k // 256))
    x = np.tile(np.array([1.0, -1.0], np.float32), k // 2).reshape(1, k)
    weight = gf.PackedWeight(syn.Q4_K, k, n, native)
    got = gf.matmul(weight, x)
    exact, abs_sum = oracle.matmul_f64(syn.Q4_K, x, native, k, n)
    terms = k / 32 + 32
    bound = (terms * 2.0 ** -24 / (1 - terms * 2.0 ** -24)) * abs_sum + 1e-6
    assert np.all(np.abs(got - exact) <= bound)


def test_matmul_linearity_at_full_size(gf):
    """Config-1 shape (15360 x 3840 Q4_K): a size-independent property instead of the slow
    oracle -- f(x1) + f(x2) == f(x1 + x2) within f32 rounding, and f(0) == 0 exactly."""
    k, n = 3840, 15360
    rng = np.random.default_rng(1)
    weight = gf.PackedWeight(syn.Q4_K, k, n, syn.make_weight(rng, syn.Q4_K, k, n))
    x = rng.standard_normal((2, k)).astype(np.float32)
    y = gf.matmul(weight, x)
    y_sum = gf.matmul(weight, (x[0] + x[1]).reshape(1, k))
    assert rel_l2(y_sum[0], (y[0].astype(np.float64) + y[1])) < 1e-5
    assert not gf.matmul(weight, np.zeros((1, k), np.float32)).any()


def test_matmul_spot_check_against_oracle_at_full_size(gf, oracle):
    """Config-1 and config-2 matrices: 64 seeded output columns each against the oracle."""
    rng = np.random.default_rng(2)
    for dtype, k, n in ((syn.Q4_K, 3840, 15360), (syn.Q6_K, 15360, 3840), (syn.Q8_0, 640, 262144)):
        native = syn.make_weight(rng, dtype, k, n)
        x = rng.standard_normal((2, k)).astype(np.float32)
        y = gf.matmul(gf.PackedWeight(dtype, k, n, native), x)
        columns = rng.choice(n, 64, replace=False)
        row_bytes = k // syn.BLOCK_ELEMENTS[dtype] * syn.BLOCK_BYTES[dtype]
        sub = np.concatenate([native[c * row_bytes:(c + 1) * row_bytes] for c in columns])
        want = oracle.matmul(dtype, x, sub, k, 64)
        assert rel_l2(y[:, columns], want) < 1e-5
