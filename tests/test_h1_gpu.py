"""GPU tests of the drafter's proposal law and of the H1 draft -> verify -> accept/rollback
loop, through the C ABI: the law against the CPU oracle, every acceptance decision replayed
through the oracle's restatement of sampling.cpp, greedy losslessness, and teacher-forced
greedy agreement over 256 steps."""
import ctypes as C

import numpy as np
import pytest

from guffin_b200 import synthetic as syn
from oracle.pyoracle import OracleModel, SamplerOptions as OracleOptions, TOKEN_LOGIT

pytestmark = pytest.mark.gpu
TWO32 = float(1 << 32)


@pytest.fixture(scope="module")
def ge(gf):
    from guffin_b200 import engine
    return engine


@pytest.fixture(scope="module")
def gm(gf):
    from guffin_b200 import model
    return model


# ------------------------------------------------------------------ proposal law

def _check_law(ge, oracle, logits, options, word, history=()):
    receipt = ge.draft_sample(logits, options, word, history)
    assert receipt.status == 0
    scores = oracle.draft_process_logits(logits, options.temperature, options.repetition_penalty, history)
    k = 1 if options.temperature == 0.0 else options.top_k
    top_p, min_p = (1.0, 0.0) if options.temperature == 0.0 else (options.top_p, options.min_p)
    ids, cdf = oracle.draft_law_compact(scores, k, top_p, min_p)
    n = receipt.count
    assert n == ids.size and list(receipt.ids[:n]) == list(ids)            # same support, ascending token ids
    got = np.array(receipt.cdf[:n + 1], np.uint64)
    assert got[0] == 0 and got[-1] == 1 << 32                              # masses sum to exactly 2^32
    assert np.all(np.diff(got.astype(np.int64)) >= 0)
    mass, want = np.diff(got.astype(np.float64)) / TWO32, np.diff(cdf.astype(np.float64)) / TWO32
    assert np.abs(mass - want).max() < 1e-6                                # |dp| < 1e-6 (gemma3_draft_tests.cpp:350-438)
    assert np.array_equal(mass == 0, want == 0)                            # the same tokens were filtered out
    index = int(np.searchsorted(got, np.uint64(word), side="right") - 1)   # sampler and receipt agree on the bin
    assert receipt.token == receipt.ids[index] and receipt.word == word
    return receipt


def test_draft_law_matches_oracle(gf, ge, oracle):
    rng = np.random.default_rng(11)
    options = ge.sampler_options(0.7)
    for vocab in (262144, 2048):
        for trial in range(4):
            logits = (rng.standard_normal(vocab) * (1.0 + trial)).astype(np.float32)
            for word in (0, 1, 0x7fffffff, 0xffffffff, int(rng.integers(1 << 32))):
                _check_law(ge, oracle, logits, options, word)
    # ties at the top-k cut-off all survive
    logits = rng.standard_normal(4096).astype(np.float32)
    order = np.argsort(-logits)
    logits[order[35:60]] = logits[order[39]]
    receipt = _check_law(ge, oracle, logits, options, 123456789)
    assert receipt.count > 40
    # a peaked row: nucleus and min-p leave few tokens with mass
    logits = rng.standard_normal(4096).astype(np.float32)
    logits[77] += 12.0
    receipt = _check_law(ge, oracle, logits, options, 0xdeadbeef)
    assert receipt.token == 77
    # repetition penalty on history tokens, and a greedy drafter
    logits = (rng.standard_normal(8192) * 3).astype(np.float32)
    history = list(np.argsort(-logits)[:6].astype(np.uint32))
    _check_law(ge, oracle, logits, ge.sampler_options(0.8, repetition_penalty=1.3), 42, history)
    receipt = _check_law(ge, oracle, logits, ge.sampler_options(0.0), 99)
    assert receipt.count == 1 and receipt.token == int(np.argmax(logits))


def test_draft_law_support_overflow_is_reported(gf, ge):
    logits = np.zeros(4096, np.float32)                                    # every token ties with the top-k-th
    receipt = ge.draft_sample(logits, ge.sampler_options(0.7), 5)
    assert receipt.status == 20


# ------------------------------------------------------------------ the H1 loop

def _models(gm, context=192, target_seed=51, draft_seed=52, correlated=False):
    tc, dc = syn.model_config("tiny-target"), syn.model_config("tiny-draft")
    tw = syn.make_model_weights("tiny-target", target_seed)
    if correlated:
        # A drafter that resembles its target (independent random models almost never agree):
        # the target's weights with a flatter output norm, F32 K/V and unscaled global RoPE.
        dc = dict(tc, kv_f16=0, rope_scale_global=1.0)
        dw = dict(tw)
        dw["output_norm.weight"] = (tw["output_norm.weight"] * 0.8).astype(np.float32)
    else:
        dw = syn.make_model_weights("tiny-draft", draft_seed)
    return (gm.Model(tc, tw, context, 2), gm.Model(dc, dw, context, 2), tc, tw)


def _options(ge, temperature, seed, speculative=1, forced=0, p=0.7, record=1, penalty=1.0):
    return ge.H1Options(ge.sampler_options(temperature, seed=seed, repetition_penalty=penalty), speculative, forced, p, 7, record)


def test_h1_greedy_is_lossless(gf, ge, gm):
    """With a greedy target the speculative loop must emit exactly the ordinary decode's tokens."""
    prompt = np.random.default_rng(1).integers(0, 2048, 33).astype(np.uint32)
    target, draft, _, _ = _models(gm, correlated=True)
    spec = ge.H1(target, draft, _options(ge, 0.0, 5))
    spec.prefill(prompt)
    speculative = spec.generate(96)
    stats = spec.stats()
    target2, _, _, _ = _models(gm)
    plain = ge.H1(target2, None, _options(ge, 0.0, 5, speculative=0))
    plain.prefill(prompt)
    ordinary = plain.generate(96)
    np.testing.assert_array_equal(speculative, ordinary)
    assert stats.cycles > 20 and stats.accepted + stats.rejected + stats.fallback_cycles == stats.cycles
    assert stats.accepted > 0
    assert target.position == prompt.size + len(speculative) - 1           # every emitted token but the last is cached
    assert target.status() == 0 and draft.status() == 0


def test_h1_continues_without_the_drafter_when_its_context_fills_first(gf, ge, gm):
    """A drafter bound to a shorter context than its target stops proposing when it is full;
    generation then goes on as ordinary decoding and, greedy, still equals the plain run."""
    prompt = np.random.default_rng(2).integers(0, 2048, 24).astype(np.uint32)
    tc = syn.model_config("tiny-target")
    tw = syn.make_model_weights("tiny-target", 51)
    dc = dict(tc, kv_f16=0, rope_scale_global=1.0)
    dw = dict(tw)
    dw["output_norm.weight"] = (tw["output_norm.weight"] * 0.8).astype(np.float32)
    target, draft = gm.Model(tc, tw, 128, 2), gm.Model(dc, dw, 40, 2)
    spec = ge.H1(target, draft, _options(ge, 0.0, 5))
    spec.prefill(prompt)
    speculative = spec.generate(80)
    stats = spec.stats()
    plain = ge.H1(gm.Model(tc, tw, 128, 2), None, _options(ge, 0.0, 5, speculative=0))
    plain.prefill(prompt)
    np.testing.assert_array_equal(speculative, plain.generate(80))
    assert len(speculative) == 80 and stats.cycles > 0 and stats.ordinary_steps > 30
    assert draft.position <= 40 and target.status() == 0


@pytest.mark.parametrize("penalty", [1.0, 1.2])
def test_h1_acceptance_decisions_match_oracle(gf, ge, gm, oracle, penalty):
    """Every accept/reject decision and corrected token of a sampled run, replayed through the
    oracle's restatement of sampling.cpp with the oracle's own RNG streams."""
    seed = 1234
    prompt = np.random.default_rng(2).integers(0, 2048, 20).astype(np.uint32)
    target, draft, _, _ = _models(gm)
    engine = ge.H1(target, draft, _options(ge, 0.7, seed, penalty=penalty))
    engine.prefill(prompt)
    tokens = engine.generate(120)
    records, stats = engine.records(), engine.stats()
    assert len(records) == stats.cycles and stats.accepted > 0 and stats.rejected > 0
    options = OracleOptions(0.7, 40, 0.95, 0.05, penalty)
    target_rng = oracle.rng(seed)
    proposal_rng = oracle.proposal_rng(target_rng)
    oracle.lib.gfo_mt_next(C.byref(target_rng))                              # the first token's ordinary draw
    observed = list(prompt)
    emitted = [int(tokens[0])]
    for record in records:
        assert record.status == 0
        assert oracle.next_proposal_word(proposal_rng) == record.word
        candidates = np.zeros(record.candidate_count, TOKEN_LOGIT)
        for i in range(record.candidate_count):
            candidates[i] = (record.candidates[i].token, record.candidates[i].logit)
        window = (observed + [record.root])[-64:]
        history = list(dict.fromkeys(window)) if penalty != 1.0 else []
        rc, prepared = oracle.prepare_distribution(candidates, options, history)
        assert rc == 0 and prepared.count == record.draft.count
        q = np.array(record.draft.target_mass[:prepared.count], np.uint64)
        rc, acceptance, residual = oracle.prepare_speculative(record.proposal, record.draft.proposal_mass, q, prepared)
        assert rc == 0
        accept_draw = oracle.uniform(target_rng)
        residual_draw = oracle.uniform(target_rng) if accept_draw >= acceptance else 0.0
        rc, token, accepted = oracle.sample_speculative(record.proposal, acceptance, residual, accept_draw, residual_draw)
        assert (rc, token, accepted) == (0, record.token, bool(record.accepted))
        if accepted:
            oracle.lib.gfo_mt_next(C.byref(target_rng))                      # the next root's ordinary draw
            observed += [record.root, record.proposal]
            emitted.append(record.proposal)
        else:
            observed.append(record.root)
            emitted.append(record.token)
    # The emitted stream is roots and accepted proposals interleaved as the loop defines.
    assert emitted[:len(records)] == [int(t) for t in _expected_stream(tokens, records)][:len(records)]


def _expected_stream(tokens, records):
    """First token, then per cycle the accepted proposal or the corrected token."""
    out = [int(tokens[0])]
    for record in records:
        out.append(record.proposal if record.accepted else record.token)
    return out


def test_h1_forced_schedule_runs_the_real_law(gf, ge, gm):
    prompt = np.random.default_rng(3).integers(0, 2048, 16).astype(np.uint32)
    target, draft, _, _ = _models(gm)
    engine = ge.H1(target, draft, _options(ge, 0.7, 9, forced=1, p=0.7))
    engine.prefill(prompt)
    tokens = engine.generate(150)
    stats = engine.stats()
    assert len(tokens) == 150 and stats.cycles == len(engine.records())
    rate = stats.accepted / stats.cycles
    assert 0.5 < rate < 0.9                                                  # Bernoulli(0.7) schedule
    assert all(r.status == 0 for r in engine.records())                     # the real law ran every cycle
    assert stats.emitted_tokens == 150


def test_greedy_tokens_agree_with_teacher_forced_oracle(gf, ge, gm, oracle):
    """256 greedy steps of the drafter-shaped model; the oracle then replays the whole sequence
    and every chosen token must be the oracle's argmax up to the logit tolerance."""
    config = syn.model_config("tiny-draft")
    weights = syn.make_model_weights("tiny-draft", 61)
    model = gm.Model(config, weights, 320, 2)
    engine = ge.H1(model, None, _options(ge, 0.0, 1, speculative=0))
    prompt = np.random.default_rng(4).integers(0, config["vocab"], 48).astype(np.uint32)
    engine.prefill(prompt)
    tokens = engine.generate(256)
    assert len(tokens) == 256
    ref = OracleModel(oracle, config, weights, context=320)
    logits = None
    for token in prompt:
        logits = ref.append(token)
    worst = 0.0
    for token in tokens:
        margin = float(logits.max() - logits[token])
        tolerance = 2e-4 * float(np.abs(logits).max())
        assert margin <= tolerance, (margin, tolerance)
        worst = max(worst, margin)
        logits = ref.append(token)
    assert worst <= 1e-3
