"""GPU parity for the block-schedule operators, candidate selection and the whole-model pass,
through the C ABI, against the CPU oracle and the fixtures made by the reference's own code."""
import ctypes as C

import numpy as np
import pytest

from guffin_b200 import synthetic as syn
from oracle.pyoracle import OracleModel
from tests.golden import make_golden as golden

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gm(gf):
    from guffin_b200 import model
    return model


def dev(gf, array):
    return gf.DeviceBuffer.from_numpy(np.ascontiguousarray(array))


def rel_l2(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


# ------------------------------------------------------------------ operators

def test_rms_norm_and_residual(gf, gm, oracle):
    want_fixture, d = np.load(golden.HERE / "ref_ops.npz"), golden.ops_inputs()
    L = gf.load()
    x, g = dev(gf, d["norm_x"]), dev(gf, d["norm_g"])
    out = gf.DeviceBuffer(d["norm_x"].nbytes)
    gf.check(L.gf_rms_norm(x.ptr, g.ptr, out.ptr, 3, 640, 1e-6, None))
    got = out.download(np.float32).reshape(3, 640)
    np.testing.assert_allclose(got, want_fixture["norm_y"], rtol=2e-6, atol=1e-7)
    residual = np.random.default_rng(5).standard_normal((3, 640)).astype(np.float32)
    r = dev(gf, residual)
    gf.check(L.gf_rms_norm_add(x.ptr, g.ptr, r.ptr, out.ptr, 3, 640, 1e-6, None))
    got = out.download(np.float32).reshape(3, 640)
    np.testing.assert_allclose(got, residual + oracle.rms_norm(d["norm_x"], d["norm_g"]), rtol=2e-6, atol=1e-6)
    assert L.gf_rms_norm(x.ptr, g.ptr, out.ptr, 3, 640, 0.0, None) == gf.GF_ERR_INVALID   # epsilon must be positive


def test_gelu_tanh_multiply(gf, gm):
    want, d = np.load(golden.HERE / "ref_ops.npz"), golden.ops_inputs()
    L = gf.load()
    gate, up = dev(gf, d["gate"]), dev(gf, d["up"])
    out = gf.DeviceBuffer(d["gate"].nbytes)
    gf.check(L.gf_gelu_tanh_multiply(gate.ptr, up.ptr, out.ptr, d["gate"].size, None))
    np.testing.assert_allclose(out.download(np.float32), want["geglu_y"], rtol=2e-5, atol=1e-6)  # 1 + tanh cancels for negative gates


@pytest.mark.parametrize("kv_f16", [0, 1])
@pytest.mark.parametrize("base,scale,position", [(1e4, 1.0, 1021), (1e6, 0.125, 30000), (1e6, 1.0, 7)])
def test_qk_norm_rope_store(gf, gm, oracle, kv_f16, base, scale, position):
    L = gf.load()
    rng = np.random.default_rng(int(position))
    rows, heads, kv_heads, hd = 2, 4, 2, 256
    raw_q = rng.standard_normal((rows, heads * hd)).astype(np.float32)
    raw_k = rng.standard_normal((rows, kv_heads * hd)).astype(np.float32)
    raw_v = rng.standard_normal((rows, kv_heads * hd)).astype(np.float32)
    qn = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kn = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    element = 2 if kv_f16 else 4
    bufs = [dev(gf, a) for a in (raw_q, raw_k, raw_v, qn, kn)]
    q_out = gf.DeviceBuffer(raw_q.nbytes)
    pk, pv = gf.DeviceBuffer(rows * kv_heads * hd * element), gf.DeviceBuffer(rows * kv_heads * hd * element)
    pos = dev(gf, np.array([position], np.uint32))
    status = dev(gf, np.zeros(4, np.uint32))
    gf.check(L.gf_qk_norm_rope_store(bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, bufs[3].ptr, bufs[4].ptr, q_out.ptr, pk.ptr,
                                     pv.ptr, pos.ptr, status.ptr, rows, heads, kv_heads, hd, 1e-6, base, scale, kv_f16, None))
    positions = [position, position + 1]
    q_want = oracle.rope_neox(oracle.rms_norm(raw_q.reshape(rows * heads, hd), qn).reshape(rows, -1), positions, heads, hd, base, scale)
    k_want = oracle.rope_neox(oracle.rms_norm(raw_k.reshape(rows * kv_heads, hd), kn).reshape(rows, -1), positions, kv_heads, hd, base, scale)
    np.testing.assert_allclose(q_out.download(np.float32).reshape(rows, -1), q_want, rtol=1e-5, atol=2e-6)
    if kv_f16:
        k_got = pk.download(np.float16).astype(np.float32).reshape(rows, -1)
        v_got = pv.download(np.float16).reshape(rows, -1)
        np.testing.assert_array_equal(v_got.view(np.uint16), raw_v.astype(np.float16).view(np.uint16))   # RNE, bit-exact
        assert np.abs(k_got - k_want).max() <= 2e-3     # one half ulp of |k| <= 4
    else:
        np.testing.assert_allclose(pk.download(np.float32).reshape(rows, -1), k_want, rtol=1e-5, atol=2e-6)
        np.testing.assert_array_equal(pv.download(np.float32).reshape(rows, -1), raw_v)
    assert status.download(np.uint32)[0] == 0


def test_f16_kv_overflow_sets_status_bit(gf, gm):
    L = gf.load()
    rows, heads, kv_heads, hd = 1, 2, 1, 256
    raw_q = np.ones((rows, heads * hd), np.float32)
    raw_k = np.ones((rows, kv_heads * hd), np.float32)
    raw_v = np.full((rows, kv_heads * hd), 1e6, np.float32)           # exceeds binary16
    bufs = [dev(gf, a) for a in (raw_q, raw_k, raw_v)]
    q_out = gf.DeviceBuffer(raw_q.nbytes)
    pk, pv = gf.DeviceBuffer(hd * 2), gf.DeviceBuffer(hd * 2)
    pos, status = dev(gf, np.array([3], np.uint32)), dev(gf, np.zeros(4, np.uint32))
    gf.check(L.gf_qk_norm_rope_store(bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, None, None, q_out.ptr, pk.ptr, pv.ptr,
                                     pos.ptr, status.ptr, rows, heads, kv_heads, hd, 1e-6, 1e4, 1.0, 1, None))
    assert status.download(np.uint32)[0] & 8


def _attention_case(gf, oracle, base, rows, window, ring_rows, heads, kv_heads, kv_f16, softcap, seed):
    """Builds committed ring rows for positions [0, base) and `rows` private rows, runs
    gf_attention, and compares each row with the oracle over its logical key range."""
    L = gf.load()
    hd, kvw = 256, kv_heads * 256
    rng = np.random.default_rng(seed)
    keys = rng.standard_normal((base + rows, kvw)).astype(np.float32)
    values = rng.standard_normal((base + rows, kvw)).astype(np.float32)
    q = rng.standard_normal((rows, heads * hd)).astype(np.float32)
    store = np.float16 if kv_f16 else np.float32
    keys_c, values_c = keys.astype(store), values.astype(store)
    ring_k, ring_v = np.zeros((ring_rows, kvw), store), np.zeros((ring_rows, kvw), store)
    for p in range(base):                       # later positions overwrite older slots, as the ring does
        ring_k[p & (ring_rows - 1)], ring_v[p & (ring_rows - 1)] = keys_c[p], values_c[p]
    bufs = [dev(gf, a) for a in (q, ring_k, ring_v, keys_c[base:], values_c[base:])]
    out = gf.DeviceBuffer(q.nbytes)
    ws = gf.DeviceBuffer(L.gf_attention_workspace_bytes(rows, heads))
    pos = dev(gf, np.array([base], np.uint32))
    gf.check(L.gf_attention(bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, bufs[3].ptr, bufs[4].ptr, out.ptr, ws.ptr, pos.ptr,
                            rows, heads, kv_heads, hd, ring_rows, window, 0.0625, softcap, kv_f16, None))
    got = out.download(np.float32).reshape(rows, -1)
    for r in range(rows):
        p = base + r
        first = max(0, p + 1 - window) if window else 0
        want = oracle.attention_row(q[r], keys_c[first:p + 1].astype(np.float32), values_c[first:p + 1].astype(np.float32),
                                    heads, kv_heads, hd, 0.0625, softcap)
        assert np.abs(got[r] - want).max() <= 3e-5 * max(1.0, np.abs(want).max()), (base, r, window)


@pytest.mark.parametrize("kv_f16", [0, 1])
def test_attention_global_local_and_ring_wrap(gf, gm, oracle, kv_f16):
    # global layer, several partitions; two rows (H1 verification)
    _attention_case(gf, oracle, base=700, rows=2, window=0, ring_rows=1024, heads=4, kv_heads=2, kv_f16=kv_f16, softcap=0.0, seed=1)
    # sliding layer: window shorter than history, ring has wrapped, window includes the row itself
    _attention_case(gf, oracle, base=100, rows=2, window=16, ring_rows=32, heads=4, kv_heads=2, kv_f16=kv_f16, softcap=0.0, seed=2)
    # window reaching into the private rows only (window smaller than the pass)
    _attention_case(gf, oracle, base=40, rows=4, window=2, ring_rows=8, heads=4, kv_heads=2, kv_f16=kv_f16, softcap=0.0, seed=3)
    # first tokens of a sequence, drafter head ratio 4:1, Gemma 2 score softcap
    _attention_case(gf, oracle, base=0, rows=1, window=8, ring_rows=16, heads=4, kv_heads=1, kv_f16=kv_f16, softcap=50.0, seed=4)
    _attention_case(gf, oracle, base=3, rows=3, window=0, ring_rows=16, heads=4, kv_heads=1, kv_f16=kv_f16, softcap=50.0, seed=5)
    # rows served in groups: an odd row count (the last group has one live row), groups of four
    # (head ratio 1), eight rows (prefill), and a window edge that falls inside a group
    _attention_case(gf, oracle, base=300, rows=3, window=0, ring_rows=512, heads=4, kv_heads=2, kv_f16=kv_f16, softcap=0.0, seed=6)
    _attention_case(gf, oracle, base=90, rows=5, window=64, ring_rows=128, heads=2, kv_heads=2, kv_f16=kv_f16, softcap=0.0, seed=7)
    _attention_case(gf, oracle, base=200, rows=8, window=128, ring_rows=256, heads=4, kv_heads=2, kv_f16=kv_f16, softcap=0.0, seed=8)
    _attention_case(gf, oracle, base=1, rows=2, window=2, ring_rows=4, heads=4, kv_heads=2, kv_f16=kv_f16, softcap=0.0, seed=9)
    # a context long enough that every partition walks several block iterations
    _attention_case(gf, oracle, base=5000, rows=2, window=0, ring_rows=8192, heads=16, kv_heads=8, kv_f16=kv_f16, softcap=0.0, seed=10)


def test_attention_rejects_unaligned_pointers(gf, gm):
    """The kernels move 16-byte vectors; a pointer off that boundary is an argument error, not a launch."""
    L = gf.load()
    q = dev(gf, np.zeros((1, 4 * 256 + 4), np.float32))
    ring = [dev(gf, np.zeros((16, 512), np.float32)) for _ in range(2)]
    private = [dev(gf, np.zeros((1, 512), np.float32)) for _ in range(2)]
    out = gf.DeviceBuffer(4 * 256 * 4)
    ws = gf.DeviceBuffer(L.gf_attention_workspace_bytes(1, 4))
    pos = dev(gf, np.array([3], np.uint32))
    with pytest.raises(gf.GuffinError):
        gf.check(L.gf_attention(q.ptr + 4, ring[0].ptr, ring[1].ptr, private[0].ptr, private[1].ptr, out.ptr, ws.ptr, pos.ptr,
                                1, 4, 2, 256, 16, 0, 0.0625, 0.0, 0, None))


def test_attention_matches_reference_fixture(gf, gm):
    """The reference's causal_grouped_attention_* + softmax composition, stored by make_golden."""
    want, d = np.load(golden.HERE / "ref_ops.npz"), golden.ops_inputs()
    L = gf.load()
    count = d["att_k"].shape[0]
    ring = 64
    bufs = [dev(gf, a) for a in (d["att_q"], np.vstack([d["att_k"][:-1], np.zeros((ring - count + 1, 512), np.float32)]),
                                 np.vstack([d["att_v"][:-1], np.zeros((ring - count + 1, 512), np.float32)]),
                                 d["att_k"][-1:], d["att_v"][-1:])]
    out = gf.DeviceBuffer(d["att_q"].nbytes)
    ws = gf.DeviceBuffer(L.gf_attention_workspace_bytes(1, 4))
    pos = dev(gf, np.array([count - 1], np.uint32))
    gf.check(L.gf_attention(bufs[0].ptr, bufs[1].ptr, bufs[2].ptr, bufs[3].ptr, bufs[4].ptr, out.ptr, ws.ptr, pos.ptr,
                            1, 4, 2, 256, ring, 0, 0.0625, 50.0, 0, None))
    np.testing.assert_allclose(out.download(np.float32), want["att_y"], rtol=0, atol=3e-5)


def test_embedding_gather_and_bad_token(gf, gm, oracle):
    L = gf.load()
    rng = np.random.default_rng(6)
    for dtype, k in ((syn.Q6_K, 512), (syn.Q8_0, 640), (syn.Q4_K, 256)):
        vocab = 50
        native = syn.make_weight(rng, dtype, k, vocab, sigma=0.05)
        weight = gf.PackedWeight(dtype, k, vocab, native)
        tokens = np.array([0, 49, 17, 8], np.uint32)
        out = gf.DeviceBuffer(4 * k * 4)
        status = dev(gf, np.zeros(4, np.uint32))
        tok = dev(gf, tokens)
        scale = np.float32(np.sqrt(np.float32(k)))
        gf.check(L.gf_embedding(dtype, weight.packed.ptr, k, vocab, tok.ptr, 4, float(scale), out.ptr, status.ptr, None))
        table = oracle.dequantize(dtype, native).reshape(vocab, k)
        np.testing.assert_array_equal(out.download(np.float32).reshape(4, k), table[tokens] * scale)    # bit-exact
        assert status.download(np.uint32)[0] == 0
        tok.upload(np.array([0, 50, 1, 2], np.uint32))
        gf.check(L.gf_embedding(dtype, weight.packed.ptr, k, vocab, tok.ptr, 4, float(scale), out.ptr, status.ptr, None))
        got = out.download(np.float32).reshape(4, k)
        assert status.download(np.uint32)[0] & 1 and np.isnan(got[1]).all() and not np.isnan(got[0]).any()


# ------------------------------------------------------------------ candidate selection

@pytest.mark.parametrize("vocab,softcap", [(262144, 0.0), (256000, 30.0), (2048, 0.0), (5000, 0.0)])
def test_candidates_match_oracle_bit_exact(gf, gm, oracle, vocab, softcap):
    L = gf.load()
    rng = np.random.default_rng(vocab)
    rows = 2
    logits = (rng.standard_normal((rows, vocab)) * 4).astype(np.float32)
    logits[0, 100] = logits[0, 7] = logits[0].max() + 1.0          # exact tie at the top: lower id first
    logits[1, :64] = 3.25                                          # a run of ties crossing the cut-off
    history = [rng.choice(vocab, 5, replace=False).astype(np.uint32), np.zeros(0, np.uint32)]
    requests = (gm.SelectionRequest * rows)(gm.selection_request(40 + 5, history[0]), gm.selection_request(40))
    bufs = dev(gf, logits)
    req = gf.DeviceBuffer(C.sizeof(requests))
    gf.check(L.gf_upload(req.ptr, C.addressof(requests), C.sizeof(requests), None))
    ws = gf.DeviceBuffer(L.gf_token_candidates_workspace_bytes(rows, vocab))
    res = gf.DeviceBuffer(rows * C.sizeof(gm.CandidateResult))
    gf.check(L.gf_token_candidates(bufs.ptr, rows, vocab, softcap, req.ptr, ws.ptr, res.ptr, None))
    raw = res.download(np.uint8)
    results = (gm.CandidateResult * rows).from_buffer_copy(raw.tobytes())
    for r in range(rows):
        retain = requests[r].retain
        want = oracle.select_candidates(logits[r], softcap, retain, history[r])
        got = results[r].pairs()
        assert results[r].status == 0 and results[r].count == want.size
        np.testing.assert_array_equal(got["token"], want["token"])
        if softcap == 0.0:
            np.testing.assert_array_equal(got["logit"], want["logit"])
        else:
            np.testing.assert_allclose(got["logit"], want["logit"], rtol=2e-6)


def test_candidates_greedy_and_status_bits(gf, gm):
    L = gf.load()
    vocab = 4096
    logits = np.linspace(-1, 1, vocab, dtype=np.float32).reshape(1, vocab)
    logits[0, 77] = np.inf
    requests = (gm.SelectionRequest * 1)(gm.selection_request(1 + 1, [vocab + 5]))    # history id out of range
    bufs, req = dev(gf, logits), gf.DeviceBuffer(C.sizeof(requests))
    gf.check(L.gf_upload(req.ptr, C.addressof(requests), C.sizeof(requests), None))
    ws = gf.DeviceBuffer(L.gf_token_candidates_workspace_bytes(1, vocab))
    res = gf.DeviceBuffer(C.sizeof(gm.CandidateResult))
    gf.check(L.gf_token_candidates(bufs.ptr, 1, vocab, 0.0, req.ptr, ws.ptr, res.ptr, None))
    result = gm.CandidateResult.from_buffer_copy(res.download(np.uint8).tobytes())
    assert result.status & 1 and result.status & 2          # non-finite logit, bad history token
    assert result.candidates[0].token == vocab - 1          # the infinity was excluded from the ranking


# ------------------------------------------------------------------ whole model

def _gpu_model(gm, geometry, seed, context, rows=2):
    config = syn.model_config(geometry)
    weights = syn.make_model_weights(geometry, seed)
    return gm.Model(config, weights, context, rows), config, weights


@pytest.mark.parametrize("fixture", ["py_target", "py_draft"])
def test_model_matches_python_reference_fixture(gf, gm, fixture):
    """Token-by-token decode on the GPU against the logits, K and V the reference's Torch
    oracle produced for the same synthetic GGUF (tests/golden/make_golden.py)."""
    want = np.load(golden.HERE / f"{fixture}.npz")
    _, geometry, seed, _, length, _ = golden.MODEL_CASES[fixture]
    model, config, _ = _gpu_model(gm, geometry, seed, context=64)
    tokens = golden.model_tokens(fixture)
    selected = {int(p): i for i, p in enumerate(want["selected"])}
    for position, token in enumerate(tokens):
        model.forward([token], logits=position in selected)
        if position in selected:
            got, ref = model.logits(0), want["logits"][selected[position]]
            assert rel_l2(got, ref) < 1e-3                                   # north-star gate
            assert np.abs(got - ref).max() <= 2e-3 * np.abs(ref).max()
        model.publish(1)
    assert model.status() == 0 and model.position == length


@pytest.mark.parametrize("geometry,seed", [("tiny-target", 21), ("tiny-draft", 22), ("tiny-gemma2", 23)])
def test_decode_verify_and_rollback_match_oracle(gf, gm, oracle, geometry, seed):
    """Ordinary decode (M=1), width-two verification (M=2) and rollback of the second row, all
    against the CPU oracle's token-at-a-time forward, including ring wrap of the sliding layers."""
    model, config, weights = _gpu_model(gm, geometry, seed, context=96)
    ref = OracleModel(oracle, config, weights, context=96)
    rng = np.random.default_rng(seed)
    tokens = rng.integers(0, config["vocab"], 60).astype(np.uint32)
    model.prefill(tokens[:37])                                              # chunked: 18 passes of 2 + 1
    for t in tokens[:37]:
        last = ref.append(t)
    assert rel_l2(model.logits(0 if 37 % 2 else 1), last) < 2e-4
    position = 37
    while position + 2 <= 58:
        pair = tokens[position:position + 2]
        model.forward(pair, logits=True)
        want0 = ref.append(pair[0])
        want1 = ref.append(pair[1])
        assert rel_l2(model.logits(0), want0) < 2e-4 and rel_l2(model.logits(1), want1) < 2e-4
        if position % 4 == 1:            # "rejected": keep row 0 only; the oracle forgets row 1 too
            model.publish(1)
            ref.truncate(position + 1)
            position += 1
        else:
            model.publish(2)
            position += 2
    assert model.position == position and model.status() == 0
    # Row-count invariance at model level: the same token decoded alone gives identical floats.
    model.forward(tokens[position:position + 2], logits=True)
    two = model.logits(0).copy()
    model.forward(tokens[position:position + 1], logits=True)
    np.testing.assert_array_equal(model.logits(0), two)


def test_gemma2_load_time_transforms_in_the_plan(gf, gm, oracle):
    """A Gemma 2 file in the form of the retained 9B: one binary16 table serving as embedding and tied
    head, and a Q6_K ffn_down.  The plan gathers embeddings from the binary16 rows, quantises the head to
    Q8_0 and binds ffn_down as Q4_K on the device; a second plan given the CPU oracle's Q8_0 head and
    Q4_K ffn_down blocks explicitly must produce the same logits bit for bit, and both agree with the
    oracle's forward over those blocks."""
    config = syn.model_config("tiny-gemma2")
    base = syn.make_model_weights("tiny-gemma2", 91)
    rng = np.random.default_rng(92)
    H, V, F = config["hidden"], config["vocab"], config["ffn"]
    table = (rng.standard_normal(V * H) / np.sqrt(H)).astype(np.float16)       # unit-RMS rows after sqrt(hidden)
    rc, head_q8 = oracle.quantize_f16_q8_0(table.view(np.uint16))
    assert rc == 0
    loaded, explicit, cpu = dict(base), dict(base), dict(base)
    del loaded["output.weight"]
    loaded["token_embd.weight"] = (1, H, V, table.view(np.uint16))              # GF_F16
    explicit["token_embd.weight"] = (1, H, V, table.view(np.uint16))
    explicit["output.weight"] = (syn.Q8_0, H, V, head_q8)
    # The oracle has no binary16 gather: a Q8_0 table whose blocks decode to the same f32 rows does not
    # exist in general, so its embedding is checked separately below and its forward starts from the
    # head-quantised table (the logits then differ by the embedding's quantisation only at the input).
    for layer in range(config["layers"]):
        key = f"blk.{layer}.ffn_down.weight"
        q6k = syn.make_weight(rng, syn.Q6_K, F, H)
        rc, q4k = oracle.requantize_q6k_q4k(q6k)
        assert rc == 0
        loaded[key] = (syn.Q6_K, F, H, q6k, "requantize")
        explicit[key] = (syn.Q4_K, F, H, q4k)
    a, b = gm.Model(config, loaded, 64, 2), gm.Model(config, explicit, 64, 2)
    tokens = rng.integers(0, V, 21).astype(np.uint32)
    a.prefill(tokens)
    b.prefill(tokens)
    row = 0 if tokens.size % 2 else 1
    np.testing.assert_array_equal(a.logits(row), b.logits(row))
    assert a.status() == 0 and np.isfinite(a.logits(row)).all() and np.abs(a.logits(row)).max() > 0
    assert a.weight_bytes(native=True) == b.weight_bytes(native=True)
    # the binary16 gather itself: row = f32(table[token]) * sqrt(hidden)
    from guffin_b200 import lib
    import ctypes as C
    table_dev, tokens_dev = lib.DeviceBuffer.from_numpy(table.view(np.uint16)), lib.DeviceBuffer.from_numpy(tokens[:5])
    out_dev, status_dev = lib.DeviceBuffer(5 * H * 4), lib.DeviceBuffer(16)
    status_dev.zero()
    scale = np.float32(np.sqrt(np.float32(H)))
    lib.check(gf.load().gf_embedding(1, table_dev.ptr, H, V, tokens_dev.ptr, 5, C.c_float(scale), out_dev.ptr, status_dev.ptr, None))
    want = table.reshape(V, H)[tokens[:5]].astype(np.float32) * scale
    np.testing.assert_array_equal(out_dev.download(np.float32).reshape(5, H), want)
    for buf in (table_dev, tokens_dev, out_dev, status_dev):
        buf.free()


@pytest.mark.parametrize("geometry,seed", [("tiny-target", 41), ("tiny-draft", 42)])
def test_eight_row_prefill_equals_two_row_prefill(gf, gm, oracle, geometry, seed):
    """Prompt ingestion in passes of eight rows (the batched prefill path) leaves the same cache and
    gives the same next-token logits as passes of two rows, and both agree with the oracle
    (run_gemma3_resident_prefill chunks rows the same way, gemma_target_runtime.cpp:420-455)."""
    wide, config, weights = _gpu_model(gm, geometry, seed, context=96, rows=8)
    narrow, _, _ = _gpu_model(gm, geometry, seed, context=96, rows=2)
    ref = OracleModel(oracle, config, weights, context=96)
    tokens = np.random.default_rng(seed).integers(0, config["vocab"], 45).astype(np.uint32)
    wide.prefill(tokens[:43])                     # five passes of eight and one of three
    narrow.prefill(tokens[:43])
    for t in tokens[:43]:
        last = ref.append(t)
    assert wide.position == narrow.position == 43
    assert rel_l2(wide.logits(2), last) < 2e-4                 # 43 = 5 * 8 + 3: the last row of the last pass
    assert rel_l2(wide.logits(2), narrow.logits(0)) < 1e-5
    # Decoding on from both caches gives the same floats up to summation order in attention.
    wide.forward(tokens[43:45], logits=True)
    narrow.forward(tokens[43:45], logits=True)
    want0 = ref.append(tokens[43]); want1 = ref.append(tokens[44])
    for row, want in ((0, want0), (1, want1)):
        assert rel_l2(wide.logits(row), want) < 2e-4
        assert rel_l2(wide.logits(row), narrow.logits(row)) < 1e-5
    assert wide.status() == 0 and narrow.status() == 0


def _write_gguf(path, weights, alignment=64):
    """A GGUF v3 file with a metadata section of every value kind and the tensors of `weights`."""
    import struct

    def string(text):
        raw = text.encode()
        return struct.pack("<Q", len(raw)) + raw

    metadata = [
        string("general.architecture") + struct.pack("<I", 8) + string("gemma3"),
        string("general.alignment") + struct.pack("<II", 4, alignment),
        string("gemma3.attention.layer_norm_rms_epsilon") + struct.pack("<If", 6, 1e-6),
        string("tokenizer.ggml.tokens") + struct.pack("<IIQ", 9, 8, 3) + string("a") + string("bc") + string(""),
        string("tokenizer.ggml.scores") + struct.pack("<IIQ", 9, 6, 4) + struct.pack("<4f", 0, 1, 2, 3),
        string("some.flag") + struct.pack("<IB", 7, 1),
        string("some.count") + struct.pack("<IQ", 10, 1 << 40),
    ]
    tensors = [("rope_freqs.weight", (4,), 0, np.zeros(4, np.float32).tobytes())]      # a tensor the path ignores
    for name, value in weights.items():
        if isinstance(value, tuple):
            dtype, k, n, data = value
            tensors.append((name, (k, n), dtype, np.ascontiguousarray(data).tobytes()))
        else:
            tensors.append((name, (value.size,), 0, np.ascontiguousarray(value, np.float32).tobytes()))
    head = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(metadata)) + b"".join(metadata)
    offset, payload = 0, []
    for name, dims, ggml_type, data in tensors:
        head += string(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", ggml_type, offset)
        pad = (-len(data)) % alignment
        payload.append(data + b"\0" * pad)
        offset += len(data) + pad
    head += b"\0" * ((-len(head)) % alignment)
    with open(path, "wb") as f:
        f.write(head)
        for chunk in payload:
            f.write(chunk)


@pytest.mark.parametrize("geometry,seed", [("tiny-target", 61), ("tiny-gemma2", 62)])
def test_gguf_file_loads_like_the_tensor_dictionary(gf, gm, tmp_path, geometry, seed):
    """gf_model_load_gguf binds the same tensors as tensor-by-tensor set_matrix / set_vector calls:
    identical logits, metadata of every kind skipped, unknown tensors ignored, damage refused."""
    config = syn.model_config(geometry)
    weights = syn.make_model_weights(geometry, seed)
    path = tmp_path / "model.gguf"
    _write_gguf(path, weights)
    from_file = gm.Model(config, path, 64, 2)
    from_dict = gm.Model(config, weights, 64, 2)
    assert from_file.bound_tensors == len(weights)
    tokens = np.random.default_rng(seed).integers(0, config["vocab"], 6).astype(np.uint32)
    for model in (from_file, from_dict):
        model.prefill(tokens)
    np.testing.assert_array_equal(from_file.logits(1), from_dict.logits(1))
    # A truncated file and a wrong magic are refused with GF_ERR_INVALID before anything is bound.
    raw = path.read_bytes()
    (tmp_path / "cut.gguf").write_bytes(raw[:len(raw) // 2])
    (tmp_path / "magic.gguf").write_bytes(b"GGML" + raw[4:])
    for bad in ("cut.gguf", "magic.gguf", "absent.gguf"):
        with pytest.raises(gf.GuffinError) as error:
            gm.Model(config, tmp_path / bad, 64, 2)
        assert error.value.status == gf.GF_ERR_INVALID


def test_gguf_file_with_a_binary16_table(gf, gm, tmp_path):
    """A file in the form of the retained Gemma 2 9B -- one binary16 token_embd, no output tensor -- binds
    through gf_model_load_gguf like the same tensors handed over one by one."""
    config = syn.model_config("tiny-gemma2")
    weights = dict(syn.make_model_weights("tiny-gemma2", 63))
    del weights["output.weight"]
    H, V = config["hidden"], config["vocab"]
    table = (np.random.default_rng(63).standard_normal(V * H) / np.sqrt(H)).astype(np.float16)
    weights["token_embd.weight"] = (1, H, V, table.view(np.uint16))
    path = tmp_path / "f16.gguf"
    _write_gguf(path, weights)
    from_file, from_dict = gm.Model(config, path, 48, 2), gm.Model(config, weights, 48, 2)
    assert from_file.bound_tensors == len(weights)
    tokens = np.random.default_rng(64).integers(0, V, 7).astype(np.uint32)
    for model in (from_file, from_dict):
        model.prefill(tokens)
    np.testing.assert_array_equal(from_file.logits(0), from_dict.logits(0))


def test_reset_returns_the_plan_to_its_first_token(gf, gm):
    """gf_model_reset forgets the committed positions: the same prompt gives the same floats again."""
    model, config, _ = _gpu_model(gm, "tiny-target", 71, context=64)
    tokens = np.random.default_rng(71).integers(0, config["vocab"], 9).astype(np.uint32)
    model.prefill(tokens)
    first = model.logits(0).copy()
    model.forward(tokens[:2], logits=True)          # leave an unpublished pass behind
    model.reset()
    assert model.position == 0 and model.status() == 0
    model.prefill(tokens)
    np.testing.assert_array_equal(model.logits(0), first)


def test_graph_replay_equals_direct_launches(gf, gm):
    model, config, _ = _gpu_model(gm, "tiny-target", 31, context=64)
    direct, _, _ = _gpu_model(gm, "tiny-target", 31, context=64)
    model.use_pass_kernel(0); direct.use_pass_kernel(0)       # the kernel-per-operator schedule, replayed and launched directly
    direct.use_graph(False)
    tokens = np.random.default_rng(3).integers(0, config["vocab"], 12).astype(np.uint32)
    for i in range(0, 12, 2):
        model.forward(tokens[i:i + 2]); direct.forward(tokens[i:i + 2])
        np.testing.assert_array_equal(model.logits(1), direct.logits(1))
        model.publish(2); direct.publish(2)


@pytest.mark.parametrize("geometry,seed", [("tiny-target", 71), ("tiny-draft", 72), ("tiny-gemma2", 73)])
def test_decode_pass_kernel_equals_kernel_per_operator_schedule(gf, gm, geometry, seed):
    """The persistent decode pass kernel (attention inside it, mode 1; attention as launches between
    its segments, mode 2) gives bit-identical logits and K/V rows to the kernel-per-operator
    schedule (mode 0): same decomposition, same order of every sum.  One- and two-row passes, a
    rollback, and enough tokens for the sliding layers' rings to wrap."""
    config = syn.model_config(geometry)
    weights = syn.make_model_weights(geometry, seed)
    tokens = np.random.default_rng(seed).integers(0, config["vocab"], 80).astype(np.uint32)
    outputs = []
    for mode in (0, 1, 2):
        model = gm.Model(config, weights, 96, 2)
        model.use_pass_kernel(mode)
        logits, position, step = [], 0, 0
        while position + 2 <= 60:
            rows = 1 if step % 3 == 2 else 2
            model.forward(tokens[position:position + rows], logits=True)
            logits.append(model.logits(rows - 1).copy())
            keep = 1 if (rows == 2 and step % 4 == 1) else rows          # a rejected second row now and then
            model.publish(keep)
            position += keep
            step += 1
        model.forward(tokens[position:position + 2], logits=False)        # a pass without the head
        model.publish(2)
        model.forward(tokens[position + 2:position + 3], logits=True)
        logits.append(model.logits(0).copy())
        kv = [model.read_kv(layer, model.position - 8, 8) for layer in range(config["layers"])]
        assert model.status() == 0
        outputs.append((logits, kv))
        model.close()
    for mode in (1, 2):
        for got, want in zip(outputs[mode][0], outputs[0][0]):
            np.testing.assert_array_equal(got, want)
        for (gk, gv), (wk, wv) in zip(outputs[mode][1], outputs[0][1]):
            np.testing.assert_array_equal(gk, wk)
            np.testing.assert_array_equal(gv, wv)


def test_model_argument_errors(gf, gm):
    model, config, _ = _gpu_model(gm, "tiny-draft", 41, context=8)
    with pytest.raises(gf.GuffinError) as e:
        model.forward([config["vocab"]])                     # token outside the vocabulary
    assert e.value.status == gf.GF_ERR_INVALID
    with pytest.raises(gf.GuffinError):
        model.forward([1, 2, 3])                             # more rows than the plan's capacity
    model.prefill(np.arange(8, dtype=np.uint32))
    with pytest.raises(gf.GuffinError):
        model.forward([1])                                   # context exhausted
