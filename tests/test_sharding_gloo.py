"""CPU, world size 2 over gloo: the host logic of the multi-GPU path (sequence sharding, gather
of the ids to rank 0, max of the per-rank times). The token path itself has no collective."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from mini_llm_cuda_b200.sharding import shard_range

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_range_covers_everything_once():
    for n in (0, 1, 7, 256, 257):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                a, b = shard_range(n, world, r)
                assert 0 <= a <= b <= n and (b - a) - n // world in (0, 1)
                seen += list(range(a, b))
            assert seen == list(range(n))
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    import torch.distributed as dist
    sys.path.insert(0, os.environ["MLB_ROOT"])
    from mini_llm_cuda_b200.sharding import shard_range, gather_tokens, max_over_ranks
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    n_total, T = 7, 5                                  # ragged: 4 + 3 sequences
    a, b = shard_range(n_total, world, rank)
    # stand-in for decode: the ids of sequence i are a pure function of i
    local = np.array([[1000 * i + t for t in range(T)] for i in range(a, b)], dtype=np.int32).reshape(b - a, T)
    full = gather_tokens(local, n_total)
    slowest = max_over_ranks(10.0 + rank)
    dist.barrier()
    if rank == 0:
        want = np.array([[1000 * i + t for t in range(T)] for i in range(n_total)], dtype=np.int32)
        assert np.array_equal(full, want), full
        assert slowest == 10.0 + world - 1
        print("GLOO_OK", full.shape)
    else:
        assert full is None and slowest == 10.0 + world - 1
    dist.destroy_process_group()
""")


def test_two_ranks_gather_and_max(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MLB_ROOT=ROOT, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)],
                       capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "GLOO_OK (7, 5)" in r.stdout
