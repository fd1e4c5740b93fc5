"""CPU: replica routing and the world_size-2 combination of replica counters over gloo."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

import numpy as np

from mtlqwen_b200 import replicas

ROOT = Path(__file__).resolve().parents[1]


def test_route_keeps_shared_prefixes_together_and_balances():
  rng = np.random.default_rng(0)
  shared = [int(t) for t in rng.integers(0, 1000, 2048)]
  prompts = [shared + [int(t) for t in rng.integers(0, 1000, 64 + i)] for i in range(8)]
  prompts += [[int(t) for t in rng.integers(0, 1000, 600)] for _ in range(8)]
  assignment = replicas.route(prompts, 2)
  assert sorted(sum(assignment, [])) == list(range(16))
  owner = [r for r, streams in enumerate(assignment) if 0 in streams][0]
  assert all(i in assignment[owner] for i in range(8))  # the shared-prefix group stays on one replica
  assert [len(a) for a in assignment] == [8, 8]
  assert len(replicas.route(prompts, 1)[0]) == 16


def test_route_cuts_a_prefix_group_that_exceeds_the_fair_share():
  """64 streams with one shared 2048-token prefix (the multi-replica benchmark configuration): every replica gets
  64 / N of them and computes the prefix once, instead of one replica getting all."""
  rng = np.random.default_rng(1)
  shared = [int(t) for t in rng.integers(0, 1000, 2048)]
  prompts = [shared + [int(t) for t in rng.integers(0, 1000, 64 + i)] for i in range(64)]
  for world in (1, 2, 4, 8):
    assignment = replicas.route(prompts, world)
    assert sorted(sum(assignment, [])) == list(range(64))
    assert [len(a) for a in assignment] == [64 // world] * world
  uneven = replicas.route(prompts[:10], 4)
  assert sorted(len(a) for a in uneven) == [1, 3, 3, 3]


def test_combine_over_two_gloo_ranks(tmp_path):
  script = tmp_path / "rank.py"
  script.write_text(textwrap.dedent(f"""
    import os, sys
    sys.path.insert(0, {str(ROOT)!r})
    import torch.distributed as dist
    from mtlqwen_b200 import replicas
    dist.init_process_group("gloo")
    rank = dist.get_rank()
    tokens, seconds = replicas.combine(dist, 100 * (rank + 1), 2.0 + rank)
    assert (tokens, seconds) == (300.0, 3.0), (tokens, seconds)
    dist.barrier()
    if rank == 0:
      print("combined", tokens / seconds)
  """))
  env = dict(os.environ, MASTER_ADDR="127.0.0.1")
  result = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                           "--master-port", "29611", str(script)], capture_output=True, text=True, env=env, timeout=240)
  assert result.returncode == 0, result.stderr[-2000:]
  assert "combined 100.0" in result.stdout
