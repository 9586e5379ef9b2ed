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
