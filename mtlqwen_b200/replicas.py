"""Independent engine replicas, one per GPU: the only multi-GPU mode of this path.

An 8-sequence batch over one 5.5 GB model does not shard, so scaling out means N engines that share nothing.
Request streams are routed once and never migrate; streams that share their first 512-token block go to the
same replica so its prefix-checkpoint cache (512-token granularity, runtime/engine.cpp:70-83 in the reference) is
hit. No collective touches the data path; `torch.distributed` (gloo) is used only to line the replicas up for a
measurement and to combine their counters.
"""
import hashlib

import numpy as np


def route(prompts, world):
  """Assigns each token-id prompt to a replica. Streams with the same first 512 tokens stay together, so that the
  replica's prefix cache is hit, as long as that does not give one replica more than its fair share
  ceil(streams / world): a larger group is cut into pieces of that size and each replica that gets a piece computes
  the shared prefix once. Pieces are dealt out largest-first onto the least-loaded replica."""
  groups = {}
  for index, prompt in enumerate(prompts):
    head = np.asarray(prompt[:512], dtype=np.int32).tobytes()
    groups.setdefault(hashlib.blake2b(head, digest_size=8).digest(), []).append(index)
  share = max(1, -(-len(prompts) // world))
  pieces = []
  for key in sorted(groups):
    members = groups[key]
    pieces += [members[at:at + share] for at in range(0, len(members), share)]
  load, assignment = [0] * world, [[] for _ in range(world)]
  for piece in sorted(pieces, key=lambda p: (-len(p), p[0])):
    target = min(range(world), key=lambda r: (load[r], r))
    assignment[target] += piece
    load[target] += len(piece)
  return assignment


def combine(dist, tokens, seconds):
  """Whole-job throughput of replicas that each produced `tokens` in `seconds`: sum of the tokens over the
  slowest replica's time. `dist` is an initialised torch.distributed module or None for a single process."""
  if dist is None:
    return float(tokens), float(seconds)
  import torch
  total = torch.tensor([float(tokens)], dtype=torch.float64)
  slowest = torch.tensor([float(seconds)], dtype=torch.float64)
  dist.all_reduce(total, op=dist.ReduceOp.SUM)
  dist.all_reduce(slowest, op=dist.ReduceOp.MAX)
  return float(total.item()), float(slowest.item())
