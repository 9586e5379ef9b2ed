"""Independent conversation streams over one resident plan (gf_streams_*): every stream of a batched
decode step must compute what the same conversation computes alone, whatever shares its pass."""
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


@pytest.mark.parametrize("geometry,seed,rows", [("tiny-gemma2", 31, 4), ("tiny-target", 32, 4), ("tiny-draft", 33, 8)])
def test_streams_equal_single_conversations(gf, gm, oracle, geometry, seed, rows):
    """Six streams with prompts of different lengths, decoded together in groups of `rows`: each stream's
    logits at every step against the same conversation decoded alone on a second plan, and one stream
    against the CPU oracle.  The long prompts and the steps wrap the sliding layers' rings."""
    config = syn.model_config(geometry)
    weights = syn.make_model_weights(geometry, seed)
    context, steps, count = 200, 36, 6
    rng = np.random.default_rng(seed)
    prompts = [rng.integers(0, config["vocab"], n).astype(np.uint32) for n in (5, 31, 47, 90, 17, 120)]
    feeds = rng.integers(0, config["vocab"], (steps, count)).astype(np.uint32)       # the token every stream is fed at every step
    shared = gm.Model(config, weights, context, rows)
    streams = gm.Streams(shared, count)
    for s, prompt in enumerate(prompts):
        streams.prefill(s, prompt)
    batch = [[streams.logits(s)] for s in range(count)]
    for t in range(steps):
        streams.decode(feeds[t])
        for s in range(count):
            batch[s].append(streams.logits(s))
    assert [streams.position(s) for s in range(count)] == [p.size + steps for p in prompts]
    assert shared.status() == 0 and shared.position == 0                             # the plan's own cache was left alone
    single = gm.Model(config, weights, context, rows)
    for s, prompt in enumerate(prompts):
        single.reset()
        single.prefill(prompt)
        alone = [single.logits(single.prefill_logits_row)]
        for t in range(steps):
            single.forward(feeds[t, s:s + 1], logits=True)
            single.publish(1)
            alone.append(single.logits(0))
        for t, (got, want) in enumerate(zip(batch[s], alone)):
            assert rel_l2(got, want) < 2e-5, (s, t)
            assert int(np.argmax(got)) == int(np.argmax(want))
    # the plan still decodes on its own afterwards, and agrees with the oracle like stream 1 did
    ref = OracleModel(oracle, config, weights, context=context)
    for token in prompts[1]:
        last = ref.append(token)
    if prompts[1].size <= 64:                                                        # the exact row path ingested it
        assert rel_l2(batch[1][0], last) < 2e-4
        for t in range(8):
            assert rel_l2(batch[1][t + 1], ref.append(feeds[t, 1])) < 2e-4
    greedy = streams.greedy()
    assert [int(g) for g in greedy] == [int(np.argmax(batch[s][-1])) for s in range(count)]
    assert streams.kv_bytes_per_step() > 0


def test_stream_results_do_not_depend_on_their_neighbours(gf, gm):
    """The same conversation in slot 0 of a set of one, and in slot 2 of a set of three with other
    conversations beside it: identical logits bit for bit (rows 1 to 4 share one arithmetic)."""
    config = syn.model_config("tiny-gemma2")
    weights = syn.make_model_weights("tiny-gemma2", 41)
    rng = np.random.default_rng(41)
    prompts = [rng.integers(0, config["vocab"], n).astype(np.uint32) for n in (23, 9, 40)]
    feeds = rng.integers(0, config["vocab"], (12, 3)).astype(np.uint32)
    plan = gm.Model(config, weights, 96, 4)
    three, one = gm.Streams(plan, 3), gm.Streams(plan, 1)
    for s in range(3):
        three.prefill(s, prompts[s])
    one.prefill(0, prompts[2])
    np.testing.assert_array_equal(three.logits(2), one.logits(0))
    for t in range(12):
        three.decode(feeds[t])
        one.decode(feeds[t, 2:3])
        np.testing.assert_array_equal(three.logits(2), one.logits(0))
    assert plan.status() == 0


@pytest.mark.parametrize("geometry,seed", [("tiny-gemma2", 51), ("tiny-target", 52)])
def test_tensor_core_step_tracks_the_exact_step(gf, gm, geometry, seed):
    """Mode 1 runs all streams of a set through one pass of bf16 tensor-core GEMMs.  Fed the same tokens
    as a set in the exact mode, its logits stay within the bf16 tolerance of the prompt path at every
    step, every stream advances, and the cache rows it publishes are the exact ones within that tolerance."""
    config = syn.model_config(geometry)
    weights = syn.make_model_weights(geometry, seed)
    rng = np.random.default_rng(seed)
    count, steps = 7, 20
    prompts = [rng.integers(0, config["vocab"], n).astype(np.uint32) for n in (9, 30, 14, 41, 3, 22, 35)]
    feeds = rng.integers(0, config["vocab"], (steps, count)).astype(np.uint32)
    plan = gm.Model(config, weights, 96, 4)
    exact, wide = gm.Streams(plan, count), gm.Streams(plan, count)
    wide.set_mode(1)
    for s, prompt in enumerate(prompts):
        exact.prefill(s, prompt)
        wide.prefill(s, prompt)
        np.testing.assert_array_equal(exact.logits(s), wide.logits(s))              # ingestion is shared code
    worst = 0.0
    for t in range(steps):
        exact.decode(feeds[t])
        wide.decode(feeds[t])
        for s in range(count):
            worst = max(worst, rel_l2(wide.logits(s), exact.logits(s)))
    assert worst < 3e-2, worst
    assert [wide.position(s) for s in range(count)] == [p.size + steps for p in prompts]
    assert plan.status() == 0
    greedy_exact, greedy_wide = exact.greedy(), wide.greedy()
    assert np.mean(greedy_exact == greedy_wide) >= 0.7                                # near-ties may flip under bf16
