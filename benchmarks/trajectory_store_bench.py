"""Throughput of the trajectory stores: steps appended per second by several episode writers, time until the data
is durable (`flush`), and full read-back (the reference keeps a harness for the same question under
tunix/experimental/trajectory/benchmarks/run_benchmark.py and commits no results).

  python -m benchmarks.trajectory_store_bench --store file --episodes 64 --turns 8 --tokens 512 --threads 8
  python -m benchmarks.trajectory_store_bench --store memory

Prints one JSON line. Runs on the CPU; nothing here touches a GPU.
"""
from __future__ import annotations

import argparse
import json
import tempfile
import threading
import time

import numpy as np

from tunix_b200.experimental.trajectory import converter, file_store, in_memory_store, trajectory as tl
from tunix_b200.rl.agentic.agents import agent_types


def make_episode(turns: int, tokens: int, seed: int) -> agent_types.Trajectory:
  rng = np.random.default_rng(seed)
  steps = []
  for t in range(turns):
    steps.append(agent_types.Step(
        model_response="r" * 64, action=agent_types.Action(action={"name": "act", "arguments": {"turn": t}}),
        observation="o" * 64, reward=float(t == turns - 1), done=t == turns - 1,
        assistant_tokens=rng.integers(0, 50000, tokens), assistant_masks=np.ones(tokens, np.int32),
        logprobs=-rng.random(tokens).astype(np.float32), env_tokens=rng.integers(0, 50000, 32),
        env_masks=np.zeros(32, np.int32)))
  return agent_types.Trajectory(task={"prompts": ["p" * 256]}, steps=steps, reward=1.0,
                                status=agent_types.TrajectoryStatus.SUCCEEDED)


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--store", choices=["file", "memory"], default="file")
  ap.add_argument("--episodes", type=int, default=64)
  ap.add_argument("--turns", type=int, default=8)
  ap.add_argument("--tokens", type=int, default=512)
  ap.add_argument("--threads", type=int, default=8)
  args = ap.parse_args()

  tmp = tempfile.TemporaryDirectory() if args.store == "file" else None
  if tmp is not None:
    store = file_store.FileTrajectoryStore(tmp.name, trajectory_cls=tl.TunixTrajectory)
  else:
    store = in_memory_store.InMemoryTrajectoryStore(trajectory_cls=tl.TunixTrajectory)
  episodes = [make_episode(args.turns, args.tokens, i) for i in range(args.episodes)]

  def write(ids) -> None:
    for i in ids:
      md = converter.create_trajectory_metadata(f"traj-{i}", agent=tl.Agent(name="bench"))
      for step in converter.EpisodeWriter().episode(episodes[i]):
        store.add_step(step, md)
      store.update_metadata(md.model_copy(update={"status": "SUCCEEDED", "total_reward": 1.0}))

  t0 = time.perf_counter()
  workers = [threading.Thread(target=write, args=(range(k, args.episodes, args.threads),)) for k in range(args.threads)]
  for w in workers:
    w.start()
  for w in workers:
    w.join()
  t_append = time.perf_counter() - t0
  store.flush()
  t_durable = time.perf_counter() - t0
  t1 = time.perf_counter()
  back = store.get_trajectories([f"traj-{i}" for i in range(args.episodes)])
  t_read = time.perf_counter() - t1
  n_steps = args.episodes * (2 * args.turns + 1)
  assert len(back) == args.episodes and all(len(t.steps) == 2 * args.turns + 1 for t in back)
  print(json.dumps({"store": args.store, "episodes": args.episodes, "steps": n_steps, "writer_threads": args.threads,
                    "append_steps_per_s": round(n_steps / t_append, 1), "durable_steps_per_s": round(n_steps / t_durable, 1),
                    "read_steps_per_s": round(n_steps / t_read, 1), "tokens_per_agent_step": args.tokens}))
  if hasattr(store, "close"):
    store.close()
  if tmp is not None:
    tmp.cleanup()


if __name__ == "__main__":
  main()
