"""The product's host sampler (gf_sampler_*, C++ in the CUDA library; needs no GPU) against the
decisions of the reference's sampling.cpp stored in tests/golden/ref_sampling.npz and against
the oracle restatement on fresh cases."""
import numpy as np
import pytest

from guffin_b200 import engine as ge
from oracle.pyoracle import SamplerOptions as OracleOptions, TOKEN_LOGIT
from tests.golden import make_golden as golden


def product_options(case):
    return ge.sampler_options(case["temperature"], case["top_k"], case["top_p"], case["min_p"], case["penalty"],
                              seed=case["seed"])


def test_sampler_matches_reference_fixture_bit_exact():
    want = np.load(golden.HERE / "ref_sampling.npz")
    accepted_seen = set()
    for i, case in enumerate(golden.sampling_cases()):
        sampler = ge.Sampler(product_options(case))
        sampler.observe(case["history"])
        tokens, weights, total = sampler.prepare(case["candidates"])
        assert list(tokens) == list(want[f"prep_tokens_{i}"])
        assert np.array_equal(weights, want[f"prep_weights_{i}"])            # identical doubles
        assert total == float(want[f"prep_total_{i}"])
        ref_rc, ref_token, ref_accepted, ref_draws, proposal, word = (int(v) for v in want[f"spec_{i}"])
        assert sampler.proposal_word() == word                              # proposal stream
        law_tokens, masses, cdf, bin_index = golden.draft_law_for(case, tokens, word)
        q = [masses[np.searchsorted(law_tokens, t)] for t in tokens]
        draft = ge.gathered_draft(proposal, masses[bin_index], cdf[bin_index], q)
        status, token, accepted, draws = sampler.sample_speculative(draft, case["candidates"])
        if ref_rc != 0:
            assert status != 0
            continue
        assert (status, token, accepted, draws) == (0, ref_token, bool(ref_accepted), ref_draws)
        accepted_seen.add(accepted)
        # an independent sampler with the same seed reproduces TokenSampler::sample
        fresh = ge.Sampler(product_options(case))
        fresh.observe(case["history"])
        assert fresh.sample(case["candidates"]) == int(want[f"sample_{i}"][1])
    assert accepted_seen == {True, False}


def test_proposal_words_of_a_whole_chain_match_the_reference_fixture():
    """The words a chain of drafts is sampled with are the next words of the proposal stream in order
    (the reference's preview_proposal_words for seed 42), and previewing consumes nothing."""
    want = np.load(golden.HERE / "ref_sampling.npz")["words_seed_42"]
    sampler = ge.Sampler(ge.sampler_options(0.7, seed=42))
    assert list(sampler.proposal_words(len(want))) == [int(w) for w in want]
    assert sampler.proposal_word() == int(want[0])
    assert list(sampler.proposal_words(3)) == [int(w) for w in want[:3]]


def test_sampler_streams_advance_like_the_oracle(oracle):
    """After a speculative draw both streams have moved: the next word and the next ordinary
    sample equal the oracle's restatement of the two mt19937_64 streams."""
    rng = np.random.default_rng(5)
    for trial in range(50):
        n = int(rng.integers(41, 90))
        candidates = np.zeros(n, TOKEN_LOGIT)
        candidates["token"] = rng.choice(262144, n, replace=False)
        candidates["logit"] = (rng.standard_normal(n) * 3).astype(np.float32)
        seed = 900 + trial
        sampler = ge.Sampler(ge.sampler_options(0.7, seed=seed))
        target_rng = oracle.rng(seed)
        proposal_rng = oracle.proposal_rng(target_rng)
        for step in range(3):
            word = sampler.proposal_word()
            assert word == oracle.next_proposal_word(proposal_rng)
            tokens, weights, total = sampler.prepare(candidates)
            case = dict(draft_seed=int(rng.integers(1 << 30)))
            law_tokens, masses, cdf, bin_index = golden.draft_law_for(case, tokens, word)
            q = np.array([masses[np.searchsorted(law_tokens, t)] for t in tokens], np.uint64)
            proposal = int(law_tokens[bin_index])
            draft = ge.gathered_draft(proposal, masses[bin_index], cdf[bin_index], q)
            status, token, accepted, draws = sampler.sample_speculative(draft, candidates)
            rc, prepared = oracle.prepare_distribution(candidates, OracleOptions(0.7, 40, 0.95, 0.05, 1.0))
            rc2, acceptance, residual = oracle.prepare_speculative(proposal, int(masses[bin_index]), q, prepared)
            if rc2 != 0:
                assert status != 0
                oracle.lib  # streams unchanged on failure: replay the same word next step
                proposal_rng = oracle.proposal_rng(oracle.rng(seed)) if step == 0 else proposal_rng
                break
            accept_draw = oracle.uniform(target_rng)
            residual_draw = oracle.uniform(target_rng) if accept_draw >= acceptance else 0.0
            _, want_token, want_accepted = oracle.sample_speculative(proposal, acceptance, residual, accept_draw, residual_draw)
            assert (status, token, accepted) == (0, want_token, want_accepted)


def test_sampler_rejects_bad_options_and_inputs():
    from guffin_b200 import lib
    with pytest.raises(lib.GuffinError):
        ge.Sampler(ge.sampler_options(top_k=0))
    with pytest.raises(lib.GuffinError):
        ge.Sampler(ge.sampler_options(top_p=0.0))
    sampler = ge.Sampler(ge.sampler_options(0.7, seed=1))
    few = np.zeros(3, TOKEN_LOGIT)
    few["token"] = [1, 2, 3]
    with pytest.raises(lib.GuffinError):
        sampler.sample(few)                       # fewer candidates than top_k


def test_greedy_speculative_accepts_only_the_argmax():
    candidates = np.zeros(45, TOKEN_LOGIT)
    candidates["token"] = np.arange(100, 145)
    candidates["logit"] = np.linspace(1, -1, 45, dtype=np.float32)
    sampler = ge.Sampler(ge.sampler_options(0.0, seed=3))
    word = sampler.proposal_word()
    draft = ge.gathered_draft(100, 1 << 32, 0, [1 << 32])          # drafter proposes the argmax with q = 1
    assert sampler.sample_speculative(draft, candidates) == (0, 100, True, 0)
    sampler = ge.Sampler(ge.sampler_options(0.0, seed=3))
    draft = ge.gathered_draft(101, 1 << 32, 0, [0])                # proposes another token: corrected to the argmax
    assert sampler.sample_speculative(draft, candidates) == (0, 100, False, 0)


def test_verification_schedule_is_the_reference_partition():
    """One pass of h + 1 rows, or the reference's conditional tiles: 3 = 2 + 1, 4 = 2 + 2, 7 = 4 + 3
    (make_registered_conditional_chain_schedule, src/engine/speculative_controller.cpp:596-604) and pairs for the
    lengths it does not register (src/engine/chain_chat.mm:78-86); the last tile carries the row of the token behind
    a fully accepted chain."""
    from guffin_b200 import engine as ge, lib
    for h in range(1, 8):
        assert ge.verification_schedule(h, False) == [(h, h + 1)]
    assert ge.verification_schedule(1, True) == [(1, 2)]
    assert ge.verification_schedule(2, True) == [(2, 3)]
    assert ge.verification_schedule(3, True) == [(2, 2), (1, 2)]
    assert ge.verification_schedule(4, True) == [(2, 2), (2, 3)]
    assert ge.verification_schedule(5, True) == [(2, 2), (2, 2), (1, 2)]
    assert ge.verification_schedule(6, True) == [(2, 2), (2, 2), (2, 3)]
    assert ge.verification_schedule(7, True) == [(4, 4), (3, 4)]
    for h in range(1, 8):
        for conditional in (False, True):
            tiles = ge.verification_schedule(h, conditional)
            assert sum(d for d, _ in tiles) == h and all(r == d for d, r in tiles[:-1]) and tiles[-1][1] == tiles[-1][0] + 1
    with pytest.raises(lib.GuffinError):
        ge.verification_schedule(8, True)
