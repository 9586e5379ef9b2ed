"""Prompt ingestion on the tensor cores: the 256-row bf16 GEMM (two 128-row products per dequantised weight tile) with in-kernel dequantisation
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
                                             (syn.Q4_K, 15360, 128, 128), (syn.Q4_K, 3840, 256, 200), (syn.Q6_K, 1024, 384, 256),
                                             (syn.Q8_0, 640, 128, 129)])
def test_prefill_matmul_matches_bf16_reference_and_oracle(gf, oracle, dtype, k, n, rows):
    """Against the same product with both operands rounded to bf16 and summed in double precision the
    kernel may differ only by its f32 accumulation (5e-5: a layout or descriptor mistake shows as an
    error of order one); against the f32 oracle by the bf16 rounding of the operands (stated
    tolerance 1e-2 relative L2, measured about 3e-3).  Rows beyond the live ones come back zero."""
    rng = np.random.default_rng(k + n + rows)
    native = syn.make_weight(rng, dtype, k, n)
    weight = gf.PackedWeight(dtype, k, n, native)
    x = rng.standard_normal((rows, k)).astype(np.float32)
    got = gf.prefill_matmul(weight, x)
    assert got.shape == ((rows + 127) // 128 * 128, n)
    w = oracle.dequantize(dtype, native).reshape(n, k)
    exact = bf16_round(x).astype(np.float64) @ bf16_round(w).astype(np.float64).T
    assert rel_l2(got[:rows], exact) < 5e-5                                  # 1.8e-5 at K = 15360: the accumulator does not round to nearest
    assert np.abs(got[:rows] - exact).max() <= 3e-4 * np.abs(exact).max()
    want = oracle.matmul(dtype, x, native, k, n)
    assert rel_l2(got[:rows], want) < 1e-2
    assert not got[rows:].any()
    weight.packed.free()


@pytest.fixture(scope="module")
def gm(gf):
    from guffin_b200 import model
    return model


@pytest.mark.parametrize("geometry,seed", [("tiny-target", 81), ("tiny-draft", 82), ("tiny-gemma2", 83)])
def test_tensor_prefill_matches_exact_row_path(gf, gm, oracle, geometry, seed):
    """A 150-token prompt through the chunked tensor-core path (several chunks, the sliding layers'
    rings wrap) against the exact row path on the same plan geometry: committed K/V rows of every layer
    and the next-token logits agree within the stated bf16 tolerance (operands rounded to 8 bits of
    mantissa in every projection of every layer: 3e-2 relative L2), the positions are equal, and
    decoding continues identically in structure (one more verified pass on both)."""
    from oracle.pyoracle import OracleModel
    config = syn.model_config(geometry)
    weights = syn.make_model_weights(geometry, seed)
    tokens = np.random.default_rng(seed).integers(0, config["vocab"], 160).astype(np.uint32)
    tensor, exact = gm.Model(config, weights, 192, 2), gm.Model(config, weights, 192, 2)
    exact.use_tensor_prefill(False)
    tensor.prefill(tokens[:150])
    exact.prefill(tokens[:150])
    assert tensor.position == exact.position == 150
    assert tensor.prefill_logits_row == 0 and exact.prefill_logits_row == 1          # 150 rows in passes of two
    got, want = tensor.logits(0), exact.logits(1)
    worst_kv = 0.0
    for layer in range(config["layers"]):
        first = 150 - 16                      # rows every layer still holds (the smallest ring keeps 32)
        gk, gv = tensor.read_kv(layer, first, 16)
        wk, wv = exact.read_kv(layer, first, 16)
        worst_kv = max(worst_kv, rel_l2(gk, wk), rel_l2(gv, wv))
    logit_error = rel_l2(got, want)
    print(f"{geometry}: tensor prefill vs exact rows: K/V rel-L2 {worst_kv:.2e}, logits rel-L2 {logit_error:.2e}")
    assert worst_kv < 3e-2 and logit_error < 3e-2
    # The oracle (f32, token at a time) agrees with the tensor path within the same tolerance.
    ref = OracleModel(oracle, config, weights, context=192)
    for token in tokens[:149]:
        ref.append(token, want_logits=False)
    assert rel_l2(got, ref.append(tokens[149])) < 3e-2
    for model in (tensor, exact):
        model.forward(tokens[150:152], logits=True)
        model.publish(2)
        assert model.status() == 0
    assert rel_l2(tensor.logits(1), exact.logits(1)) < 3e-2


@pytest.mark.parametrize("base,rows,window,ring_rows,heads,kv_heads,softcap", [
    (700, 128, 0, 1024, 4, 2, 0.0),         # global layer, a full chunk
    (300, 37, 64, 128, 4, 2, 0.0),          # sliding window inside the ring (wrapped) and into the private rows
    (0, 100, 16, 32, 2, 2, 0.0),            # first chunk of a prompt: private rows only, one head per KV head
    (90, 128, 0, 128, 4, 1, 50.0),          # four heads per KV head, score softcap
    (5, 3, 4, 8, 4, 2, 0.0),                # a few rows
])
def test_prefill_attention_matches_oracle(gf, oracle, base, rows, window, ring_rows, heads, kv_heads, softcap):
    """The chunk attention kernel against the oracle's row attention over each row's logical key
    range (causal, sliding window including the row itself, ring slots overwritten by later
    positions): f16 queries and softmax weights on the tensor cores, tolerance 2e-3."""
    L = gf.load()
    hd, kvw = 256, kv_heads * 256
    rng = np.random.default_rng(base + rows)
    keys = rng.standard_normal((base + rows, kvw)).astype(np.float16)
    values = rng.standard_normal((base + rows, kvw)).astype(np.float16)
    q = rng.standard_normal((rows, heads * hd)).astype(np.float32)
    ring_k, ring_v = np.zeros((ring_rows, kvw), np.float16), np.zeros((ring_rows, kvw), np.float16)
    for p in range(base):
        ring_k[p & (ring_rows - 1)], ring_v[p & (ring_rows - 1)] = keys[p], values[p]
    bufs = [gf.DeviceBuffer.from_numpy(np.ascontiguousarray(a)) for a in (q, ring_k, ring_v, keys[base:], values[base:])]
    out = gf.DeviceBuffer(q.nbytes)
    pos = gf.DeviceBuffer.from_numpy(np.array([base], np.uint32))
    gf.check(L.gf_prefill_attention(bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, bufs[3].ptr, bufs[4].ptr, out.ptr, pos.ptr,
                                    rows, heads, kv_heads, hd, ring_rows, window, 0.0625, softcap, None))
    gf.check(L.gf_stream_synchronize(None))
    got = out.download(np.float32).reshape(rows, -1)
    for r in range(rows):
        p = base + r
        first = max(0, p + 1 - window) if window else 0
        want = oracle.attention_row(q[r], keys[first:p + 1].astype(np.float32), values[first:p + 1].astype(np.float32),
                                    heads, kv_heads, hd, 0.0625, softcap)
        assert np.abs(got[r] - want).max() <= 2e-3 * max(1.0, np.abs(want).max()), (base, r, window)
