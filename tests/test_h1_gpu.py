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
    # greedy: all the mass on the lowest id among the tied maxima (the step CDF of the reference)
    receipt = ge.draft_sample(logits, ge.sampler_options(0.0), 5)
    assert receipt.status == 0 and receipt.count == 1 and receipt.token == 0 and receipt.cdf[1] == 1 << 32


def test_selection_requests_written_on_the_device(gf, ge):
    """Request rows built on the device from the sampler's window and a chain of device-resident tokens
    equal the rows the host sampler would build (window slide, first-appearance order)."""
    from guffin_b200 import lib
    from guffin_b200.model import SelectionRequest
    rng = np.random.default_rng(8)
    for limit, held, top_k in ((64, 64, 40), (64, 10, 40), (8, 8, 1), (0, 0, 40), (64, 0, 7)):
        window = rng.integers(0, 30, held).astype(np.uint32)                   # few distinct ids: many repeats
        chain = rng.integers(0, 30, 8).astype(np.uint32)
        base = np.zeros(67, np.uint32)
        base[0], base[1], base[2] = top_k, limit, held
        base[3:3 + held] = window
        assert base.nbytes == gf.load().gf_selection_base_bytes()
        base_dev, chain_dev = lib.DeviceBuffer.from_numpy(base), lib.DeviceBuffer.from_numpy(chain)
        rows_dev = lib.DeviceBuffer(8 * C.sizeof(SelectionRequest))
        lib.check(gf.load().gf_selection_requests(base_dev.ptr, int(chain[0]), chain_dev.ptr, 8, rows_dev.ptr, None))
        rows = rows_dev.download(np.uint32).reshape(8, 66)
        for i in range(8):
            context = (list(window) + list(chain[:i + 1]))
            context = context[len(context) - limit:] if limit else []
            history = list(dict.fromkeys(int(t) for t in context))
            assert rows[i, 0] == top_k + len(history) and rows[i, 1] == len(history)
            assert list(rows[i, 2:2 + len(history)]) == history
        for b in (base_dev, chain_dev, rows_dev):
            b.free()


# ------------------------------------------------------------------ the H1 loop

def _models(gm, context=192, target_seed=51, draft_seed=52, correlated=False, rows=2, noise=0.0):
    tc, dc = syn.model_config("tiny-target"), syn.model_config("tiny-draft")
    tw = syn.make_model_weights("tiny-target", target_seed)
    if correlated:
        # A drafter that resembles its target (independent random models almost never agree):
        # the target's weights with a flatter output norm, F32 K/V and unscaled global RoPE.
        dc = dict(tc, kv_f16=0, rope_scale_global=1.0)
        dw = dict(tw)
        dw["output_norm.weight"] = (tw["output_norm.weight"] * 0.8).astype(np.float32)
        if noise:       # per-channel noise on the final norm: the drafter's best token now differs from the target's at times
            factors = 1.0 + noise * np.random.default_rng(draft_seed).standard_normal(dw["output_norm.weight"].size)
            dw["output_norm.weight"] = (dw["output_norm.weight"] * factors).astype(np.float32)
    else:
        dw = syn.make_model_weights("tiny-draft", draft_seed)
    return (gm.Model(tc, tw, context, rows), gm.Model(dc, dw, context, max(2, rows - 1)), tc, tw)


def _options(ge, temperature, seed, speculative=1, forced=0, p=0.7, record=1, penalty=1.0, horizon=1, conditional=0):
    return ge.H1Options(ge.sampler_options(temperature, seed=seed, repetition_penalty=penalty), speculative, forced, p, 7, record,
                        horizon, conditional)


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
    assert stats.cycles > 20 and stats.accepted + stats.rejected == stats.cycles and stats.fallback_cycles == 0
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


def _replay_decisions(oracle, prompt, tokens, records, seed, penalty):
    """Replays every acceptance test of a sampled run through the oracle's restatement of sampling.cpp
    with the oracle's own RNG streams; returns the token stream the decisions imply."""
    options = OracleOptions(0.7, 40, 0.95, 0.05, penalty)
    target_rng = oracle.rng(seed)
    proposal_rng = oracle.proposal_rng(target_rng)
    oracle.lib.gfo_mt_next(C.byref(target_rng))                              # the first token's ordinary draw
    observed = list(prompt)
    emitted = [int(tokens[0])]
    chain = []                                                               # rows of the running cycle accepted so far
    for record in records:
        assert record.status == 0 and record.depth == len(chain)
        assert oracle.next_proposal_word(proposal_rng) == record.word
        candidates = np.zeros(record.candidate_count, TOKEN_LOGIT)
        for i in range(record.candidate_count):
            candidates[i] = (record.candidates[i].token, record.candidates[i].logit)
        window = (observed + chain + [record.root])[-64:]
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
        chain.append(record.root)
        if accepted:
            emitted.append(record.proposal)
            if record.depth + 1 == record.horizon:                           # the whole chain held
                oracle.lib.gfo_mt_next(C.byref(target_rng))                  # the next root's ordinary draw
                observed += chain + [record.proposal]
                chain = []
                emitted.append(None)                                         # the next root: no acceptance test produced it
        else:
            emitted.append(record.token)
            observed += chain
            chain = []
    return emitted


def _check_stream(tokens, emitted):
    """The emitted tokens are the accepted proposals and corrected tokens in order, with a freely
    sampled root after every chain that held whole."""
    got = [int(t) for t in tokens]
    assert len(emitted) >= len(got) - 1
    for have, expect in zip(got, emitted):
        assert expect is None or have == expect


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
    _check_stream(tokens, _replay_decisions(oracle, prompt, tokens, records, seed, penalty))


# ------------------------------------------------------------------ horizons above one

def _assert_caches_match_replay(gm, target, draft, tc, tw, prompt, tokens, context):
    """Whatever was accepted or rolled back, the target's cache must hold exactly the rows of its own
    token sequence: compare every layer's K/V with a fresh plan fed the same tokens two at a time.
    The drafter's position must be the rows it was allowed to keep."""
    cached = target.position
    sequence = np.concatenate([prompt, tokens])[:cached].astype(np.uint32)
    fresh = gm.Model(tc, tw, context, 2)
    fresh.use_tensor_prefill(False)
    fresh.prefill(sequence)
    for layer in range(tc["layers"]):
        window = tc["sliding_window"] if fresh_layer_is_local(tc, layer) else cached
        first = max(0, cached - window)
        k0, v0 = target.read_kv(layer, first, cached - first)
        k1, v1 = fresh.read_kv(layer, first, cached - first)
        np.testing.assert_allclose(k0, k1, rtol=2e-3, atol=2e-3)            # binary16 rows: within one or two ulps
        np.testing.assert_allclose(v0, v1, rtol=2e-3, atol=2e-3)
    assert cached <= draft.position + 2 and draft.position <= cached


def fresh_layer_is_local(config, layer):
    pattern = config["sliding_pattern"]
    return (layer + 1) % 6 != 0 if pattern == 6 else layer % 2 == 0 if pattern == 2 else False


@pytest.mark.parametrize("horizon,noise", [(2, 0.0), (3, 0.5), (7, 0.5), (3, None)])
def test_chain_greedy_is_lossless(gf, ge, gm, horizon, noise):
    """A chain of `horizon` drafts verified in one pass of horizon + 1 rows: with a greedy target the
    emitted tokens are exactly the ordinary decode's, whatever is accepted or rolled back (noise:
    how far the drafter's final norm is from the target's; None = an unrelated drafter)."""
    prompt = np.random.default_rng(1).integers(0, 2048, 33).astype(np.uint32)
    target, draft, tc, tw = _models(gm, correlated=noise is not None, rows=horizon + 1, noise=noise or 0.0)
    spec = ge.H1(target, draft, _options(ge, 0.0, 5, horizon=horizon))
    spec.prefill(prompt)
    speculative = spec.generate(96)
    stats = spec.stats()
    target2, _, _, _ = _models(gm)
    plain = ge.H1(target2, None, _options(ge, 0.0, 5, speculative=0))
    plain.prefill(prompt)
    np.testing.assert_array_equal(speculative, plain.generate(96))
    assert stats.accepted + stats.rejected == stats.cycles and stats.cycles > 5
    assert stats.drafted_tokens >= stats.accepted_tokens
    if noise is not None:
        assert stats.accepted_tokens > stats.cycles                         # chains longer than one draft were kept
    assert target.position == prompt.size + len(speculative) - 1
    assert target.status() == 0 and draft.status() == 0
    _assert_caches_match_replay(gm, target, draft, tc, tw, prompt, speculative, 192)


@pytest.mark.parametrize("penalty", [1.0, 1.2])
def test_chain_acceptance_decisions_match_oracle(gf, ge, gm, oracle, penalty):
    """Horizon 3, sampled: every acceptance test along every chain replayed through the oracle
    (one proposal word per test, the target stream advanced only by the tests that ran)."""
    seed = 4321
    prompt = np.random.default_rng(5).integers(0, 2048, 20).astype(np.uint32)
    target, draft, tc, tw = _models(gm, correlated=True, rows=4, noise=0.6)
    engine = ge.H1(target, draft, _options(ge, 0.7, seed, penalty=penalty, horizon=3))
    engine.prefill(prompt)
    tokens = engine.generate(150)
    records, stats = engine.records(), engine.stats()
    assert stats.cycles > 10 and len(records) >= stats.cycles and stats.accepted_tokens > 0 and stats.rejected > 0
    assert max(r.depth for r in records) == 2                               # some chains were verified to their end
    if penalty == 1.0:
        assert any(r.depth >= 1 and not r.accepted for r in records)        # and some were cut part way
    _check_stream(tokens, _replay_decisions(oracle, prompt, tokens, records, seed, penalty))
    assert target.status() == 0 and draft.status() == 0
    _assert_caches_match_replay(gm, target, draft, tc, tw, prompt, tokens, 192)


def test_chain_forced_schedule(gf, ge, gm):
    prompt = np.random.default_rng(3).integers(0, 2048, 16).astype(np.uint32)
    target, draft, _, _ = _models(gm, context=256, rows=4)
    engine = ge.H1(target, draft, _options(ge, 0.7, 9, forced=1, p=0.7, horizon=3))
    engine.prefill(prompt)
    tokens = engine.generate(200)
    stats = engine.stats()
    assert len(tokens) == 200 and stats.emitted_tokens == 200
    rate = stats.accepted_tokens / len(engine.records())                    # Bernoulli(0.7) per acceptance test
    assert 0.55 < rate < 0.85
    assert stats.emitted_tokens > 1.8 * stats.cycles                        # 1 + 0.7 + 0.49 + 0.343 tokens per cycle expected


@pytest.mark.parametrize("horizon,penalty,forced", [(3, 1.0, 0), (4, 1.2, 0), (7, 1.0, 1), (5, 1.2, 1), (2, 1.0, 0)])
def test_conditional_tiles_emit_the_single_pass_tokens(gf, ge, gm, oracle, horizon, penalty, forced):
    """A cycle's drafts verified as a cascade of passes (the reference's conditional chain schedule: 3 = 2 + 1,
    4 = 2 + 2, 7 = 4 + 3, pairs otherwise) must reproduce the single-pass cycle test for test: the same words,
    candidates, decisions and tokens, the same caches -- only the number of target passes differs."""
    seed = 777
    prompt = np.random.default_rng(8).integers(0, 2048, 20).astype(np.uint32)
    runs = []
    for conditional in (0, 1):
        target, draft, tc, tw = _models(gm, context=256, correlated=True, rows=8, noise=0.6)
        engine = ge.H1(target, draft, _options(ge, 0.7, seed, penalty=penalty, horizon=horizon, conditional=conditional, forced=forced))
        engine.prefill(prompt)
        tokens = engine.generate(160)
        runs.append((tokens, engine.records(), engine.stats(), target, draft, tc, tw))
        assert target.status() == 0 and draft.status() == 0
    (single_tokens, single_records, single_stats, *_), (tokens, records, stats, target, draft, tc, tw) = runs
    np.testing.assert_array_equal(tokens, single_tokens)
    assert len(records) == len(single_records)
    for a, b in zip(records, single_records):
        assert (a.root, a.proposal, a.word, a.token, a.accepted, a.depth, a.horizon, a.candidate_count) == \
               (b.root, b.proposal, b.word, b.token, b.accepted, b.depth, b.horizon, b.candidate_count)
        assert bytes(a.candidates)[:8 * a.candidate_count] == bytes(b.candidates)[:8 * b.candidate_count]      # row-count invariant logits
    assert single_stats.verify_passes == single_stats.cycles
    if horizon == 2:            # one tile of two drafts and three rows: the single pass itself
        assert stats.verify_passes == stats.cycles
    else:
        assert stats.cycles < stats.verify_passes <= 2 * stats.cycles + (stats.cycles if horizon == 5 else 0)
    assert (stats.cycles, stats.accepted, stats.rejected, stats.accepted_tokens) == \
           (single_stats.cycles, single_stats.accepted, single_stats.rejected, single_stats.accepted_tokens)
    if not forced:
        _check_stream(tokens, _replay_decisions(oracle, prompt, tokens, records, seed, penalty))
    _assert_caches_match_replay(gm, target, draft, tc, tw, prompt, tokens, 256)


# ------------------------------------------------------------------ the law over the whole vocabulary

def test_full_vocabulary_law_known_answers(gf, ge):
    """The reference's own cases (tests/engine/gemma3_draft_tests.cpp:283-300): equal logits everywhere."""
    vocab = 262144
    logits = np.zeros(vocab, np.float32)
    everything = np.arange(vocab, dtype=np.uint32)
    options = ge.sampler_options(1.0, top_k=1, top_p=1.0, min_p=0.0)
    receipt, intervals = ge.draft_sample_full(logits, options, 0xffffffff, gather=everything)
    assert receipt.status == 0 and receipt.count == 0xffffffff
    mass = (intervals[:, 1] - intervals[:, 0]).astype(np.int64)
    assert np.all(mass == 16384) and int(mass.sum()) == 1 << 32             # every cut-off tie survives top-k 1
    assert receipt.token == vocab - 1 and int(intervals[-1, 0]) == (1 << 32) - 16384
    options = ge.sampler_options(1.0, top_k=1, top_p=0.5, min_p=0.0)
    receipt, intervals = ge.draft_sample_full(logits, options, 0, gather=[0, 1, vocab - 2, vocab - 1])
    mass = (intervals[:, 1] - intervals[:, 0]).astype(np.int64)
    assert receipt.status == 0 and mass[0] == 32768 and mass[2] == 0 and mass[3] == 0      # ascending-tail nucleus
    options = ge.sampler_options(1.0, top_k=1, top_p=float(np.finfo(np.float32).smallest_subnormal), min_p=0.0)
    receipt, intervals = ge.draft_sample_full(logits, options, 0, gather=[0, 1])
    mass = (intervals[:, 1] - intervals[:, 0]).astype(np.int64)
    assert receipt.status == 0 and receipt.token == 0 and mass[0] == 1 << 32 and mass[1] == 0


@pytest.mark.parametrize("vocab,top_k,top_p,min_p", [(2048, 100, 0.9, 0.02), (6144, 0, 0.8, 0.0), (262144, 200, 0.95, 0.05),
                                                     (4096, 0, 1.0, 0.0), (2048 + 256, 40, 0.95, 0.05)])
def test_full_vocabulary_law_matches_oracle(gf, ge, oracle, vocab, top_k, top_p, min_p):
    rng = np.random.default_rng(vocab + top_k)
    logits = (rng.standard_normal(vocab) * 2.0).astype(np.float32)
    if top_k == 40:
        logits[:] = rng.integers(0, 3, vocab)                               # three distinct values: > 256 ties at the cut-off
    options = ge.sampler_options(0.7, top_k=top_k, top_p=top_p, min_p=min_p)
    everything = np.arange(vocab, dtype=np.uint32)
    scores = oracle.draft_process_logits(logits, 0.7)
    status, want = oracle.draft_law_full(scores, 0.7, top_k, top_p, min_p)
    assert status == 0
    for word in (0, 0x7fffffff, 0xffffffff, int(rng.integers(1 << 32))):
        receipt, intervals = ge.draft_sample_full(logits, options, word, gather=everything)
        assert receipt.status == 0 and receipt.count == 0xffffffff and receipt.word == word
        got = np.concatenate([intervals[:, 0], intervals[-1:, 1]])
        assert np.array_equal(intervals[1:, 0], intervals[:-1, 1])          # the bins tile [0, 2^32)
        assert got[0] == 0 and got[-1] == 1 << 32 and np.all(np.diff(got.astype(np.int64)) >= 0)
        mass, expect = np.diff(got.astype(np.float64)) / TWO32, np.diff(want.astype(np.float64)) / TWO32
        assert np.abs(mass - expect).max() < 1e-6
        if top_k or top_p < 1.0 or min_p > 0.0:
            assert np.array_equal(mass == 0, expect == 0)                   # the same tokens were filtered out
        else:
            assert np.all(mass[expect > 1e-6] > 0)                          # unfiltered: only vanishing bins may close
        index = int(np.searchsorted(got, np.uint64(word), side="right") - 1)
        assert receipt.token == index


def test_flat_drafter_is_verified_through_the_full_law(gf, ge, gm, oracle):
    """A drafter whose logits all tie overflows the compact law at every proposal: each cycle then
    rebuilds the law over the whole vocabulary, verifies again, and the decisions still replay."""
    seed = 77
    prompt = np.random.default_rng(6).integers(0, 2048, 12).astype(np.uint32)
    tc, dc = syn.model_config("tiny-target"), syn.model_config("tiny-draft")
    tw, dw = syn.make_model_weights("tiny-target", 51), dict(syn.make_model_weights("tiny-draft", 52))
    dw["output_norm.weight"] = np.zeros_like(dw["output_norm.weight"])       # every logit is exactly zero
    target, draft = gm.Model(tc, tw, 128, 2), gm.Model(dc, dw, 128, 2)
    engine = ge.H1(target, draft, _options(ge, 0.7, seed))
    engine.prefill(prompt)
    tokens = engine.generate(40)
    records, stats = engine.records(), engine.stats()
    assert stats.cycles > 10 and stats.full_law_proposals == stats.cycles and stats.fallback_cycles == stats.cycles
    assert all(r.draft.proposal_mass > 0 for r in records)
    masses = {int(m) for r in records for m in r.draft.target_mass[:r.draft.count]}
    assert len(masses - {0}) == 1                                            # a uniform law over the nucleus
    _check_stream(tokens, _replay_decisions(oracle, prompt, tokens, records, seed, 1.0))


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
