"""Whole-model parity at the geometries the benchmark runs: the 270M Q8_0 drafter (512-token
prompt, 256 greedy steps) and the 12B Q4_K_M target (two-row verification at short and long
context) against the CPU oracle on the same seeded weights.  At these shapes the planner picks
other decompositions than at the tiny test geometries (K split over the warps of a CTA for
Q/K/V, eight and nine K chunks for the output and down projections, the unsplit 262144-column
head), and their fused prologues and head epilogue run here against the oracle."""
import os

import numpy as np
import pytest

from guffin_b200 import synthetic as syn
from oracle.pyoracle import OracleModel
pytestmark = pytest.mark.gpu


def rel_l2(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


@pytest.fixture(scope="module")
def gm(gf):
    from guffin_b200 import model
    return model


@pytest.fixture(scope="module")
def ge(gf):
    from guffin_b200 import engine
    return engine


@pytest.fixture()
def all_cores(oracle):
    oracle.set_threads(os.cpu_count() or 1)          # column-parallel GEMV: every column's sum is unchanged
    yield oracle
    oracle.set_threads(1)


def test_270m_greedy_256_after_512_token_prompt(gf, ge, gm, all_cores):
    """The drafter geometry of scripts/gemma3_reference_golden.py:41-42 (18 layers, hidden 640, one
    KV head, window 512, tied 262144-row Q8_0 head): 512 seeded prompt tokens, then 256 greedy
    steps on the GPU; the oracle replays the whole sequence teacher-forced and every emitted token
    must be its argmax up to the stated logit tolerance (margins are reported, ties are noise)."""
    oracle = all_cores
    config = syn.model_config("gemma3-270m")
    weights = syn.make_model_weights("gemma3-270m", 2701)
    model = gm.Model(config, weights, 512 + 256 + 8, 2)
    model.use_tensor_prefill(False)      # this test pins greedy tokens to 2e-4 of the oracle: the prompt takes the exact row path
    options = ge.H1Options(ge.sampler_options(0.0, seed=1), 0, 0, 0.7, 7, 0)
    engine = ge.H1(model, None, options)
    prompt = np.random.default_rng(31).integers(0, config["vocab"], 512).astype(np.uint32)
    engine.prefill(prompt)
    tokens = engine.generate(256)
    assert len(tokens) == 256 and model.status() == 0
    ref = OracleModel(oracle, config, weights, context=512 + 256 + 8)
    for token in prompt[:-1]:
        ref.append(token, want_logits=False)
    logits = ref.append(prompt[-1])
    worst, disagreements = 0.0, 0
    for step, token in enumerate(tokens):
        margin = float(logits.max() - logits[token])
        tolerance = 2e-4 * float(np.abs(logits).max())
        assert margin <= tolerance, (step, margin, tolerance)
        disagreements += int(token != int(logits.argmax()))
        worst = max(worst, margin)
        logits = ref.append(token)
    print(f"270M greedy-256: worst oracle margin {worst:.3e}, {disagreements} steps chose a tie within tolerance")
    # One more row on both sides: full logits agree, not only the argmax.
    model.forward([int(tokens[-1])], logits=True)
    plain = model.logits(0).copy()
    assert rel_l2(plain, logits) < 1e-3
    # The same row through the persistent decode pass kernel (its attention stays a launch of its own for an
    # f32 cache): bit-identical at this geometry too.
    model.use_pass_kernel(1)
    model.forward([int(tokens[-1])], logits=True)
    np.testing.assert_array_equal(model.logits(0), plain)
    assert model.status() == 0
    # The same prompt through the tensor-core prefill (Q8_0 weights, f32 cache): first-token logits within
    # the bf16 tolerance of the oracle's.
    model.use_pass_kernel(0)
    model.use_tensor_prefill(True)
    model.reset()
    model.prefill(prompt)
    ref.reset()
    for token in prompt[:-1]:
        ref.append(token, want_logits=False)
    error = rel_l2(model.logits(model.prefill_logits_row), ref.append(prompt[-1]))
    print(f"270M tensor prefill of 512 tokens: first-token logits rel-L2 {error:.2e}")
    assert error < 3e-2 and model.status() == 0


def _assert_same_candidates(model, gm, got_logits, want_logits, retain=40):
    """The best `retain` tokens by (logit desc, token asc) are the same set on both sides, except
    where the oracle's own logits tie within the comparison tolerance at the cut-off."""
    order = np.lexsort((np.arange(want_logits.size), -want_logits))
    want = set(int(t) for t in order[:retain])
    got = set(int(t) for t in np.lexsort((np.arange(got_logits.size), -got_logits))[:retain])
    cutoff = float(want_logits[order[retain - 1]])
    slack = 2e-4 * float(np.abs(want_logits).max())
    for token in want ^ got:
        assert abs(float(want_logits[token]) - cutoff) <= slack, (token, float(want_logits[token]), cutoff)


def test_12b_two_row_verification_matches_oracle_at_short_and_long_context(gf, gm, all_cores):
    """Gemma-3-12B Q4_K_M geometry (scripts/gemma3_target_reference.py:28-29).  (a) Three prompt
    tokens, then two width-two verification passes with a rollback between them: logits within 1e-3
    relative L2 (the tolerance of tests/engine/gemma3_target_runtime_tests.cpp:1118-1127 is looser)
    and the same candidate sets.  (b) The GPU ingests 1100 more tokens; its committed K/V rows are
    copied into the oracle, which then appends the same two tokens itself: the 1024-row window has
    slid, several attention partitions are live, and only the rows the oracle computes are compared."""
    oracle = all_cores
    config = syn.model_config("gemma3-12b")
    weights = syn.make_model_weights("gemma3-12b", 1201)
    context = 1152
    model = gm.Model(config, weights, context, 8)
    model.use_tensor_prefill(False)      # parts (a) and (b) pin the exact row path; part (c) turns the tensor path on
    ref = OracleModel(oracle, config, weights, context=context)
    tokens = np.random.default_rng(31).integers(0, config["vocab"], 1120).astype(np.uint32)

    model.prefill(tokens[:3])
    for token in tokens[:3]:
        ref.append(token, want_logits=False)
    # pass 1 on [t3, t4]; the draft row is "rejected": only row 0 is published.
    model.forward(tokens[3:5], logits=True)
    want = [ref.append(tokens[3]), ref.append(tokens[4])]
    for row in range(2):
        got = model.logits(row)
        assert rel_l2(got, want[row]) < 1e-3
        _assert_same_candidates(model, gm, got, want[row])
    model.publish(1)
    ref.truncate(4)
    # pass 2 on [t4, t5]; accepted.
    model.forward(tokens[4:6], logits=True)
    want = [ref.append(tokens[4]), ref.append(tokens[5])]
    errors = [rel_l2(model.logits(row), want[row]) for row in range(2)]
    assert max(errors) < 1e-3
    model.publish(2)
    for layer in (0, 5, 47):                         # a local, a global and the last layer: K/V rows agree
        k, v = model.read_kv(layer, 0, 6)
        for position in range(6):
            assert np.abs(k[position] - ref.key(layer, position)).max() <= 2e-3 * max(1.0, np.abs(k[position]).max())
            assert np.abs(v[position] - ref.value(layer, position)).max() <= 2e-3 * max(1.0, np.abs(v[position]).max())

    # (b) long context, reached by GPU prefill in eight-row passes.
    base = 1100
    model.prefill(tokens[6:base])                    # continues from the committed position
    assert model.position == base
    for layer in range(config["layers"]):
        k, v = model.read_kv(layer, 0, base)
        ref.set_kv(layer, 0, k, v)
    ref.seek(base)
    model.forward(tokens[base:base + 2], logits=True)
    want = [ref.append(tokens[base]), ref.append(tokens[base + 1])]
    long_errors = [rel_l2(model.logits(row), want[row]) for row in range(2)]
    assert max(long_errors) < 1e-3
    plain = [model.logits(row).copy() for row in range(2)]
    for row in range(2):
        _assert_same_candidates(model, gm, plain[row], want[row])
    # The same two rows through the persistent decode pass kernel (attention inside it, several partitions,
    # the 1024-row window): bit-identical to the kernel-per-operator schedule at this geometry.
    model.use_pass_kernel(1)
    model.forward(tokens[base:base + 2], logits=True)
    for row in range(2):
        np.testing.assert_array_equal(model.logits(row), plain[row])
    assert model.status() == 0
    # (c) The same 1101-token prefix through the tensor-core prefill (128-row bf16 GEMMs): the last token's
    # logits against the exact path's, within the stated bf16 tolerance.
    model.use_pass_kernel(0)
    model.use_tensor_prefill(True)
    model.reset()
    model.prefill(tokens[:base + 1])
    assert model.position == base + 1
    error = rel_l2(model.logits(model.prefill_logits_row), plain[0])
    print(f"12B tensor prefill of {base + 1} tokens: last-token logits rel-L2 {error:.2e} against the exact row path")
    assert error < 3e-2 and model.status() == 0
    print(f"12B verify parity: rel-L2 short context {max(errors):.2e}, at position {base} {max(long_errors):.2e}")

