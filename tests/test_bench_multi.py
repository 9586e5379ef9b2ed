"""The multi-stream aggregation of bench.py with two gloo ranks on CPU: tokens add up over
ranks, the time is the slowest rank's; and the reference arm's non-zero ranks stay silent."""
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_stream_aggregation_with_two_gloo_ranks(tmp_path):
    script = tmp_path / "ranks.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys, json
        sys.path.insert(0, {ROOT!r})
        import torch.distributed as dist
        import bench
        dist.init_process_group("gloo")
        rank = dist.get_rank()
        out = bench.aggregate_streams(dist, 100.0 + rank, 90.0 + rank, 10.0 * (rank + 1), 0.5 * (rank + 1))
        print(json.dumps({{"rank": rank, "out": list(out)}}))
        dist.destroy_process_group()
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outputs = [p.communicate(timeout=120) for p in procs]
    assert all(p.returncode == 0 for p in procs), outputs
    import json
    for stdout, _ in outputs:
        result = json.loads(stdout.strip().splitlines()[-1])
        assert result["out"] == [201.0, 181.0, 20.0, 1.0]      # sums of tokens, max of times


def test_single_process_aggregation_is_identity():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.aggregate_streams(None, 5.0, 4.0, 3.0, 2.0) == (5.0, 4.0, 3.0, 2.0)


def test_tensor_parallel_host_logic_with_two_gloo_ranks(tmp_path):
    """Two CPU ranks each cut their shard out of the same seeded matrices (guffin_b200.tensor_parallel), multiply
    with the CPU checker, sum the row shards' partial products in rank order and merge the column shards'
    candidate lists: the results are the unsharded product and its top candidates."""
    script = tmp_path / "tp_ranks.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys, json
        sys.path.insert(0, {ROOT!r})
        import numpy as np
        import torch, torch.distributed as dist
        from guffin_b200 import synthetic as syn, tensor_parallel as tp
        from oracle.pyoracle import Oracle
        dist.init_process_group("gloo")
        rank, size = dist.get_rank(), dist.get_world_size()
        oracle = Oracle()
        rng = np.random.default_rng(3)
        k, n, vocab = 1024, 64, 512
        down = syn.make_weight(rng, syn.Q4_K, k, n)               # split by input row
        head = syn.make_weight(rng, syn.Q6_K, n * 4, vocab)       # split by output column
        x = rng.standard_normal((2, k)).astype(np.float32)
        hidden = rng.standard_normal((2, n * 4)).astype(np.float32)
        part = oracle.matmul(syn.Q4_K, np.ascontiguousarray(x[:, rank * k // size:(rank + 1) * k // size]),
                             tp._rows((syn.Q4_K, k, n, down), rank, size)[3], k // size, n)
        parts = [torch.zeros(2, n) for _ in range(size)]
        dist.all_gather(parts, torch.from_numpy(part))
        total = parts[0].numpy().copy()
        for other in parts[1:]:
            total = total + other.numpy()                          # rank order on every rank: the same bits everywhere
        full = oracle.matmul(syn.Q4_K, x, down, k, n)
        logits = oracle.matmul(syn.Q6_K, hidden, tp._columns((syn.Q6_K, n * 4, vocab, head), rank, size)[3], n * 4, vocab // size)
        pair = np.dtype([("token", np.uint32), ("logit", np.float32)])
        order = np.lexsort((np.arange(vocab // size), -logits[0].astype(np.float64)))[:16]
        mine = np.array([(o + rank * (vocab // size), logits[0][o]) for o in order], pair)
        lists = [None] * size
        dist.all_gather_object(lists, mine)
        merged = tp.merge_candidates(lists, 16)
        whole = oracle.matmul(syn.Q6_K, hidden, head, n * 4, vocab)[0]
        want = np.lexsort((np.arange(vocab), -whole.astype(np.float64)))[:16]
        print(json.dumps({{"rank": rank, "sum_ok": bool(np.linalg.norm(total - full) <= 1e-6 * np.linalg.norm(full)),
                          "digest": float(total.astype(np.float64).sum()), "tokens_ok": bool(np.array_equal(merged["token"], want)),
                          "logits_ok": bool(np.array_equal(merged["logit"], whole[want]))}}))
        dist.destroy_process_group()
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE="2")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r), LOCAL_RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outputs = [p.communicate(timeout=300) for p in procs]
    assert all(p.returncode == 0 for p in procs), outputs
    import json
    results = [json.loads(stdout.strip().splitlines()[-1]) for stdout, _ in outputs]
    assert all(r["sum_ok"] and r["tokens_ok"] and r["logits_ok"] for r in results), results
    assert results[0]["digest"] == results[1]["digest"]           # both ranks hold the same sum, bit for bit
