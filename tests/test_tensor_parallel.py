"""The optional tensor-parallel mode (guffin_b200.tensor_parallel): weight sharding and candidate merging on
the CPU against the oracle; on a GPU, two shards of a model on one device (each driven by its own host thread,
partial sums summed in rank order) against the unsharded plan."""
import threading

import numpy as np
import pytest

from guffin_b200 import synthetic as syn
from guffin_b200 import tensor_parallel as tp


def test_shard_config_and_errors():
    config = syn.model_config("gemma3-12b")
    local = tp.shard_config(config, 2)
    assert (local["heads"], local["kv_heads"], local["ffn"], local["vocab"], local["hidden"]) == (8, 4, 7680, 131072, 3840)
    with pytest.raises(ValueError):
        tp.shard_config(syn.model_config("gemma3-270m"), 2)          # one KV head does not split
    with pytest.raises(ValueError):
        tp.shard_config(config, 3)


@pytest.mark.parametrize("dtype", [syn.Q4_K, syn.Q6_K, syn.Q8_0])
def test_shards_of_a_matrix_against_the_oracle(dtype):
    """Column shards reproduce their columns of the full product bit for bit; row shards sum to it."""
    from oracle.pyoracle import Oracle
    oracle = Oracle()
    rng = np.random.default_rng(5)
    k, n, size = 1024, 48, 2
    native = syn.make_weight(rng, dtype, k, n)
    x = rng.standard_normal((2, k)).astype(np.float32)
    full = oracle.matmul(dtype, x, native, k, n)
    columns = [oracle.matmul(dtype, x, tp._columns((dtype, k, n, native), r, size)[3], k, n // size) for r in range(size)]
    assert np.array_equal(np.concatenate(columns, axis=1), full)
    partial = [oracle.matmul(dtype, np.ascontiguousarray(x[:, r * k // size:(r + 1) * k // size]),
                             tp._rows((dtype, k, n, native), r, size)[3], k // size, n) for r in range(size)]
    total = partial[0].astype(np.float64) + partial[1]
    assert np.linalg.norm(total - full) <= 1e-6 * np.linalg.norm(full)


def test_shard_weights_names_and_shapes():
    config = syn.model_config("tiny-target")
    weights = syn.make_model_weights("tiny-target", 3)
    shard = dict(tp.shard_weights(weights, 1, 2))
    assert shard["blk.0.attn_q.weight"][1:3] == (512, 512) and shard["blk.0.attn_k.weight"][1:3] == (512, 256)
    assert shard["blk.0.attn_output.weight"][1:3] == (512, 512) and shard["blk.0.ffn_down.weight"][1:3] == (512, 512)
    assert shard["blk.0.ffn_gate.weight"][1:3] == (512, 512)
    assert shard["token_embd.weight"][2] == config["vocab"] and shard["output.weight"][2] == config["vocab"] // 2
    assert np.array_equal(shard["blk.0.attn_norm.weight"], weights["blk.0.attn_norm.weight"])


def test_merge_candidates_is_the_full_top_k():
    rng = np.random.default_rng(2)
    logits = rng.standard_normal(4096).astype(np.float32)
    logits[100] = logits[3000] = logits.max() + 1.0                   # a tie across the two shards
    pair = np.dtype([("token", np.uint32), ("logit", np.float32)])
    lists = []
    for rank in range(2):
        part = logits[rank * 2048:(rank + 1) * 2048]
        order = np.lexsort((np.arange(2048), -part.astype(np.float64)))[:64]
        lists.append(np.array([(o + rank * 2048, part[o]) for o in order], pair))
    merged = tp.merge_candidates(lists, 64)
    order = np.lexsort((np.arange(4096), -logits.astype(np.float64)))[:64]
    assert np.array_equal(merged["token"], order.astype(np.uint32)) and merged["token"][0] == 100 and merged["token"][1] == 3000


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["tiny-target", "tiny-gemma2"])
def test_two_shards_on_one_device_match_the_unsharded_plan(name):
    from guffin_b200 import model as gm
    config = syn.model_config(name)
    weights = syn.make_model_weights(name, 11)
    rng = np.random.default_rng(4)
    prompt = rng.integers(0, config["vocab"], 21).astype(np.uint32)
    steps = [rng.integers(0, config["vocab"], 2).astype(np.uint32) for _ in range(3)]
    request = gm.SelectionRequest(retain=64, history_count=0)

    full = gm.Model(config, weights, 64, 8)
    full.prefill(prompt)
    want = [(full.logits(full.prefill_logits_row), None)]
    for tokens in steps:
        full.forward(tokens)
        picked = full.select([request, request])
        want.append((np.stack([full.logits(0), full.logits(1)]), [p.pairs() for p in picked]))
        full.publish(1)
    want_kv = full.read_kv(1, 0, full.position)

    size = 2
    reducer = tp.ThreadReducer(size, 8 * config["hidden"])
    shards = [tp.Shard(config, weights, 64, rank, size, reducer.hook(rank), row_capacity=8) for rank in range(size)]
    for shard in shards:
        shard.model.use_graph(False)
    got = [[] for _ in range(size)]
    errors = []

    def drive(rank):
        try:
            model = shards[rank].model
            model.prefill(prompt)
            got[rank].append((model.logits(model.prefill_logits_row), None))
            for tokens in steps:
                model.forward(tokens)
                picked = model.select([request, request])
                got[rank].append((np.stack([model.logits(0), model.logits(1)]), [shards[rank].global_candidates(p) for p in picked]))
                model.publish(1)
            assert model.status() == 0
        except Exception as error:          # a failed shard must not leave the other at the barrier
            reducer.barrier.abort()
            errors.append(error)

    threads = [threading.Thread(target=drive, args=(rank,)) for rank in range(size)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not errors, errors
    assert reducer.calls == 2 * config["layers"] * (3 + len(steps))           # 21 prompt tokens = 3 passes of up to 8 rows
    for step, (logits, candidates) in enumerate(want):
        merged = np.concatenate([got[r][step][0] for r in range(size)], axis=-1)
        assert np.linalg.norm(merged - logits) <= 2e-5 * np.linalg.norm(logits), step
        if candidates is not None:
            for row in range(2):
                both = tp.merge_candidates([got[r][step][1][row] for r in range(size)], 64)
                assert np.array_equal(both["token"][:8], candidates[row]["token"][:8])
                assert np.allclose(both["logit"], candidates[row]["logit"], rtol=1e-4, atol=1e-5)
    # each shard's KV ring holds its own heads of the unsharded ring
    kv_width = config["kv_heads"] * config["head_dim"] // size
    for rank in range(size):
        k, v = shards[rank].model.read_kv(1, 0, shards[rank].model.position)
        assert np.allclose(k, want_kv[0][:, rank * kv_width:(rank + 1) * kv_width], rtol=2e-3, atol=2e-3)
        assert np.allclose(v, want_kv[1][:, rank * kv_width:(rank + 1) * kv_width], rtol=2e-3, atol=2e-3)


@pytest.mark.gpu
def test_single_shard_exchange_is_the_plain_plan():
    """One shard of one: the exchange-carrying launches (parts read through the arena, nothing to wait for) must
    give the plain plan's bits."""
    from guffin_b200 import model as gm
    config = syn.model_config("tiny-target")
    weights = syn.make_model_weights("tiny-target", 11)
    rng = np.random.default_rng(4)
    prompt = rng.integers(0, config["vocab"], 21).astype(np.uint32)
    pair = rng.integers(0, config["vocab"], 2).astype(np.uint32)
    plain = gm.Model(config, weights, 64, 8)
    shard = tp.Shard(config, weights, 64, 0, 1, row_capacity=8)
    shard.connect([shard.arena])
    for graph in (False, True):
        results = []
        for model in (plain, shard.model):
            model.reset()
            model.use_graph(graph)
            model.prefill(prompt)
            first = model.logits(model.prefill_logits_row)
            model.forward(pair)
            results.append((first, model.logits(0), model.logits(1)))
            model.publish(2)
            assert model.status() == 0
        for want, got in zip(*results):
            assert np.array_equal(want, got)
    k0, v0 = plain.read_kv(3, 0, plain.position)
    k1, v1 = shard.model.read_kv(3, 0, shard.model.position)
    assert np.array_equal(k0, k1) and np.array_equal(v0, v1)


@pytest.mark.gpu
def test_single_shard_prompt_chunks_are_the_plain_plan():
    """The tensor-core prompt path of a shard (a chunk's O and down products summed over the shards in one launch),
    one shard of one: the same bits as the plain plan's chunks."""
    from guffin_b200 import model as gm
    config = syn.model_config("tiny-target")
    weights = syn.make_model_weights("tiny-target", 11)
    prompt = np.random.default_rng(6).integers(0, config["vocab"], 150).astype(np.uint32)
    plain = gm.Model(config, weights, 256, 8)
    shard = tp.Shard(config, weights, 256, 0, 1, row_capacity=8)
    shard.connect([shard.arena])
    results = []
    for model in (plain, shard.model):
        model.prefill(prompt)
        results.append((model.logits(model.prefill_logits_row), model.read_kv(5, 0, model.position),       # the global layer: every row
                        model.read_kv(6, model.position - 8, 8)))                                            # a sliding layer: the rows still in its ring
        assert model.status() == 0
    assert np.array_equal(results[0][0], results[1][0])
    for layer in (1, 2):
        assert np.array_equal(results[0][layer][0], results[1][layer][0]) and np.array_equal(results[0][layer][1], results[1][layer][1])


def _two_devices():
    from guffin_b200 import lib
    return lib.device_count() >= 2


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["tiny-target", "tiny-gemma2"])
def test_two_shards_on_two_devices_exchange_inside_the_launches(name):
    """Two shards in one process, one GPU each, every shard driven by its own host thread; the partial sums
    cross NVLink inside the projection launches.  Checked against the unsharded plan."""
    from guffin_b200 import lib, model as gm
    if not _two_devices():
        pytest.skip("needs two GPUs")
    L = lib.load()
    config = syn.model_config(name)
    weights = syn.make_model_weights(name, 11)
    rng = np.random.default_rng(4)
    prompt = rng.integers(0, config["vocab"], 21).astype(np.uint32)
    steps = [rng.integers(0, config["vocab"], 2).astype(np.uint32) for _ in range(6)]
    lib.check(L.gf_set_device(0))
    full = gm.Model(config, weights, 256, 8)
    full.prefill(prompt)
    want = [full.logits(full.prefill_logits_row)[None, :]]
    for tokens in steps:
        full.forward(tokens)
        want.append(np.stack([full.logits(0), full.logits(1)]))
        full.publish(1)
    want_kv = full.read_kv(1, 0, full.position)

    size = 2
    shards = []
    for rank in range(size):
        lib.check(L.gf_set_device(rank))
        shards.append(tp.Shard(config, weights, 256, rank, size, row_capacity=8))
    arenas = [shard.arena for shard in shards]
    for rank in range(size):
        lib.check(L.gf_set_device(rank))
        shards[rank].connect(arenas)
        lib.check(L.gf_model_shard_set_wait_limit(shards[rank].model.handle, 1 << 20))      # about a second per wait
    lib.check(L.gf_set_device(0))
    got = [[] for _ in range(size)]
    kv = [None] * size
    errors = []

    def drive(rank):
        try:
            lib.check(L.gf_set_device(rank))
            model = shards[rank].model
            model.prefill(prompt)
            got[rank].append(model.logits(model.prefill_logits_row)[None, :])
            for tokens in steps:
                model.forward(tokens)
                got[rank].append(np.stack([model.logits(0), model.logits(1)]))
                model.publish(1)
            kv[rank] = model.read_kv(1, 0, model.position)
            assert model.status() == 0
            model.synchronize()
        except Exception as error:
            errors.append(error)

    threads = [threading.Thread(target=drive, args=(rank,)) for rank in range(size)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not errors, errors
    for step, logits in enumerate(want):
        merged = np.concatenate([got[r][step] for r in range(size)], axis=-1)
        assert np.linalg.norm(merged - logits) <= 2e-5 * np.linalg.norm(logits), step
    kv_width = config["kv_heads"] * config["head_dim"] // size
    for rank in range(size):
        assert np.allclose(kv[rank][0], want_kv[0][:, rank * kv_width:(rank + 1) * kv_width], rtol=2e-3, atol=2e-3)
        assert np.allclose(kv[rank][1], want_kv[1][:, rank * kv_width:(rank + 1) * kv_width], rtol=2e-3, atol=2e-3)

    # A prompt long enough for the tensor-core path: each chunk's O and down products cross NVLink in one launch.
    long_prompt = np.random.default_rng(9).integers(0, config["vocab"], 200).astype(np.uint32)
    full.reset()
    full.prefill(long_prompt)
    want_long = full.logits(full.prefill_logits_row)
    global_layer = 5 if config["sliding_pattern"] == 6 else 1                 # a layer whose ring keeps every row
    want_long_kv = full.read_kv(global_layer, 0, full.position)
    got_long, kv_long = [None] * size, [None] * size

    def ingest(rank):
        try:
            lib.check(L.gf_set_device(rank))
            model = shards[rank].model
            model.reset()
            model.prefill(long_prompt)
            got_long[rank] = model.logits(model.prefill_logits_row)
            kv_long[rank] = model.read_kv(global_layer, 0, model.position)
            assert model.status() == 0
        except Exception as error:
            errors.append(error)

    threads = [threading.Thread(target=ingest, args=(rank,)) for rank in range(size)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=300)
    assert not errors, errors
    merged = np.concatenate(got_long)
    assert np.linalg.norm(merged - want_long) <= 3e-2 * np.linalg.norm(want_long)            # bf16 operands on both sides
    for rank in range(size):
        ours, theirs = kv_long[rank][0], want_long_kv[0][:, rank * kv_width:(rank + 1) * kv_width]
        assert np.linalg.norm(ours - theirs) <= 3e-2 * np.linalg.norm(theirs)


@pytest.mark.gpu
def test_a_silent_peer_costs_a_timeout_not_a_hang():
    """One shard of two whose peer never runs: its arena is a zeroed buffer nothing writes.  Every poll for the
    peer's values runs out after its (shortened) limit, the pass completes, the status call reports
    GF_ERR_TIMEOUT, the poisoned plan refuses further passes, and a reset makes it usable again."""
    from guffin_b200 import lib, model as gm
    L = lib.load()
    config = syn.model_config("tiny-target")
    weights = syn.make_model_weights("tiny-target", 11)
    shard = tp.Shard(config, weights, 64, 0, 2)
    silent = lib.DeviceBuffer(L.gf_model_shard_arena_bytes(shard.model.handle))
    silent.zero()
    shard.connect([shard.arena, silent.ptr])
    lib.check(L.gf_model_shard_set_wait_limit(shard.model.handle, 500))
    model = shard.model
    model.use_graph(False)
    tokens = np.array([5, 9], np.uint32)
    model.forward(tokens)                                   # enqueues; every wait for the peer gives up on the device
    with pytest.raises(lib.GuffinError) as error:
        model.status()
    assert error.value.status == lib.GF_ERR_TIMEOUT
    with pytest.raises(lib.GuffinError) as error:
        model.forward(tokens)
    assert error.value.status == lib.GF_ERR_STATE
    model.reset()
    model.forward(tokens)                                   # usable again (and times out again: the peer is still silent)
    with pytest.raises(lib.GuffinError) as error:
        model.status()
    assert error.value.status == lib.GF_ERR_TIMEOUT


@pytest.mark.gpu
def test_single_shard_global_selection_and_engine_are_the_plain_ones():
    """Global selection on one shard of one: the gathered and merged rows are the plain selection's (history tokens
    included), and an H1 engine on the shard emits the plain engine's tokens."""
    from guffin_b200 import engine as ge, model as gm
    config = syn.model_config("tiny-target")
    weights = syn.make_model_weights("tiny-target", 11)
    prompt = np.random.default_rng(4).integers(0, config["vocab"], 21).astype(np.uint32)
    plain = gm.Model(config, weights, 160, 2)
    shard = tp.Shard(config, weights, 160, 0, 1)
    shard.connect([shard.arena])
    shard.global_selection()
    requests = [gm.SelectionRequest(retain=40, history_count=0), gm.SelectionRequest(retain=43, history_count=3)]
    requests[1].history[0], requests[1].history[1], requests[1].history[2] = 7, 2000, 512
    rows = []
    for model in (plain, shard.model):
        model.prefill(prompt)
        model.forward(np.array([3, 9], np.uint32))
        for repeat in range(3):          # consecutive gathers alternate their slots
            picked = model.select(requests)
        rows.append([p.pairs() for p in picked])
        assert [p.status for p in picked] == [0, 0]
    for want, got in zip(*rows):
        assert np.array_equal(want["token"], got["token"]) and np.array_equal(want["logit"], got["logit"])

    dc = dict(config, kv_f16=0, rope_scale_global=1.0)
    dw = dict(weights)
    dw["output_norm.weight"] = (weights["output_norm.weight"] * 0.8).astype(np.float32)
    emitted = []
    for sharded in (False, True):
        if sharded:
            target_shard = tp.Shard(config, weights, 160, 0, 1)
            target_shard.connect([target_shard.arena])
            target_shard.global_selection()
            target = target_shard.model
        else:
            target = gm.Model(config, weights, 160, 2)
        draft = gm.Model(dc, dw, 160, 2)
        engine = ge.H1(target, draft, ge.H1Options(ge.sampler_options(0.7, seed=5), 1, 0, 0.7, 7, 0, 1))
        engine.prefill(prompt)
        emitted.append(engine.generate(80))
        assert engine.stats().accepted > 0 and target.status() == 0
    np.testing.assert_array_equal(emitted[0], emitted[1])


@pytest.mark.gpu
def test_h1_engines_on_two_shards_run_in_step():
    """One H1 engine per shard (two GPUs, one process, a host thread each; every shard has its own replica of the
    drafter and the same seeds): the merged candidate rows are the same on both shards, so both engines emit the
    same tokens, and a greedy run emits the unsharded engine's."""
    from guffin_b200 import engine as ge, lib, model as gm
    if not _two_devices():
        pytest.skip("needs two GPUs")
    L = lib.load()
    config = syn.model_config("tiny-target")
    weights = syn.make_model_weights("tiny-target", 11)
    dc = dict(config, kv_f16=0, rope_scale_global=1.0)
    dw = dict(weights)
    dw["output_norm.weight"] = (weights["output_norm.weight"] * 0.8).astype(np.float32)
    prompt = np.random.default_rng(4).integers(0, config["vocab"], 90).astype(np.uint32)     # long enough for the chunk path
    size = 2
    for temperature in (0.0, 0.7):
        lib.check(L.gf_set_device(0))
        single = ge.H1(gm.Model(config, weights, 256, 2), gm.Model(dc, dw, 256, 2), ge.H1Options(ge.sampler_options(temperature, seed=5), 1, 0, 0.7, 7, 0, 1))
        single.prefill(prompt)
        want = single.generate(64)
        shards, drafts = [], []
        for rank in range(size):
            lib.check(L.gf_set_device(rank))
            shards.append(tp.Shard(config, weights, 256, rank, size))
            drafts.append(gm.Model(dc, dw, 256, 2))
        arenas = [shard.arena for shard in shards]
        for rank in range(size):
            lib.check(L.gf_set_device(rank))
            shards[rank].connect(arenas)
            shards[rank].global_selection()
            lib.check(L.gf_model_shard_set_wait_limit(shards[rank].model.handle, 1 << 20))
        lib.check(L.gf_set_device(0))
        emitted, stats, errors = [None] * size, [None] * size, []

        def drive(rank):
            try:
                lib.check(L.gf_set_device(rank))
                engine = ge.H1(shards[rank].model, drafts[rank], ge.H1Options(ge.sampler_options(temperature, seed=5), 1, 0, 0.7, 7, 0, 1))
                engine.prefill(prompt)
                emitted[rank] = engine.generate(64)
                stats[rank] = engine.stats()
                assert shards[rank].model.status() == 0
            except Exception as error:
                errors.append(error)

        threads = [threading.Thread(target=drive, args=(rank,)) for rank in range(size)]
        for t in threads:
            t.start()
        for t in threads:
            t.join(timeout=300)
        assert not errors, errors
        np.testing.assert_array_equal(emitted[0], emitted[1])
        assert stats[0].cycles == stats[1].cycles and stats[0].accepted == stats[1].accepted and stats[0].accepted > 0
        if temperature == 0.0:
            np.testing.assert_array_equal(emitted[0], want)


def test_shards_of_a_binary16_table_and_of_a_matrix_bound_through_a_transform():
    """The Gemma 2 file forms: an F16 head / embedding table is cut by vocabulary row, and a Q6_K matrix that the
    plan requantises at load keeps its marker, so every shard transforms its own slice (the transforms work block by
    block and column by column, so they commute with the cuts)."""
    rng = np.random.default_rng(1)
    k, vocab = 512, 64
    table = rng.standard_normal((vocab, k)).astype(np.float16)
    down = syn.make_weight(rng, syn.Q6_K, 1024, 32)
    weights = {"token_embd.weight": (1, k, vocab, table.view(np.uint8).reshape(-1)),
               "blk.0.ffn_down.weight": (syn.Q6_K, 1024, 32, down, "requantize"),
               "output_norm.weight": np.ones(k, np.float32)}
    for rank in range(2):
        shard = dict(tp.shard_weights(weights, rank, 2))
        assert shard["token_embd.weight"][2] == vocab                                   # the gather table stays whole
        head = shard["output.weight"]                                                   # cut from the tied table
        assert head[:3] == (1, k, vocab // 2)
        assert np.array_equal(head[3].view(np.float16).reshape(vocab // 2, k), table[rank * vocab // 2:(rank + 1) * vocab // 2])
        cut = shard["blk.0.ffn_down.weight"]
        assert cut[:3] == (syn.Q6_K, 512, 32) and cut[4] == "requantize"
        blocks = down.reshape(32, 4, 210)
        assert np.array_equal(cut[3].reshape(32, 2, 210), blocks[:, 2 * rank:2 * rank + 2])
