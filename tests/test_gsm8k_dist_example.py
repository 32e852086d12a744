"""The distributed GSM8K GRPO example: its GSM8K pieces, and the whole system - control plane, trainer node, rollout
node, inference node - found through discovery, driven over remote execution, weights moved through host-staged
endpoints, with the tiny model on the CPU."""
import json
import socket
import threading

import pytest
import torch

from tunix_b200.experimental.distributed.runtime import main as rt_main
from tunix_b200.experimental.examples.math_gsm8k_dist import (gsm8k, models, node_common, run_gsm8k_dist_grpo as control,
                                                               run_inference_node, run_rollout_node, run_trainer_node)
from tunix_b200.experimental.rl.agentic import registry

PKG = "tunix_b200.experimental.examples.math_gsm8k_dist"


def free_port() -> int:
  with socket.socket() as s:
    s.bind(("127.0.0.1", 0))
    return s.getsockname()[1]


def test_answers_are_read_from_the_answer_format_only():
  assert gsm8k.extract_answer("<reasoning>48 + 24</reasoning><answer>\\boxed{72}</answer>") == "72"
  assert gsm8k.extract_answer("first \\boxed{7}, no wait \\boxed{ 1,072.0 }") == "1072"
  assert gsm8k.extract_answer("<answer> it is -3.5 dollars </answer>") == "-3.5"
  assert gsm8k.extract_answer("I think 72 is right") is None and gsm8k.extract_answer("\\boxed{none}") is None
  assert gsm8k.gold_of("48/2 = 24 ... #### 72") == "72" and gsm8k.gold_of("1,000") == "1000"

  class Item:
    def __init__(self, text, gold="72", n=10):
      self.metadata, self.completion_tokens = {"completion_text": text, "gold_answer": gold}, list(range(n))
  answer, contains, length = (gsm8k.make_reward_fn(m) for m in ("answer", "contains", "length"))
  assert answer(Item("\\boxed{72}")) == pytest.approx(1.1) and answer(Item("\\boxed{71}")) == pytest.approx(0.1)
  assert answer(Item("72")) == 0.0 and contains(Item("so 72 clips")) == 1.0 and contains(Item("71")) == 0.0
  assert length(Item("", n=1)) > length(Item("", n=50))
  with pytest.raises(ValueError, match="unknown reward mode"):
    gsm8k.make_reward_fn("vibes")


def test_tasks_come_from_a_file_or_a_generator_and_carry_the_gold_answer(tmp_path):
  tasks = gsm8k.load_tasks(None, 5, seed=3)
  assert tasks == gsm8k.load_tasks(None, 5, seed=3) and len(tasks) == 5 and all(gold.isdigit() for _, gold in tasks)
  path = tmp_path / "train.jsonl"
  path.write_text("\n".join(json.dumps({"question": f"q{i}?", "answer": f"work #### {i * 7}"}) for i in range(4)))
  assert gsm8k.load_tasks(str(path), 3) == [("q0?", "0"), ("q1?", "7"), ("q2?", "14")]
  rows = gsm8k.prompt_items(tasks[:2], {"temperature": 0.7}, agentic=True)
  assert rows[0]["prompt_id"] == "gsm8k_00000" and "Problem: " in rows[0]["prompt"] and rows[0]["max_turns"] == 1
  assert rows[1]["metadata"]["gold_answer"] == tasks[1][1] and rows[1]["metadata"]["env_config"]["env_type"] == "gsm8kenv"
  assert "env_config" not in gsm8k.prompt_items(tasks[:1], {})[0]["metadata"]


def test_environment_and_agent_are_registered_and_score_one_step():
  assert registry.ENV_REGISTRY.get(gsm8k.GSM8K_ENV_NAME) is gsm8k.GSM8KEnv
  assert registry.AGENT_REGISTRY.get(gsm8k.GSM8K_AGENT_NAME) is gsm8k.GSM8KAgent
  env = gsm8k.GSM8KEnv(prompt="2 + 2?", gold_answer="4", group_id="g", pair_index=1)
  obs, _ = env.reset()
  assert obs == {"prompts": "2 + 2?"}
  agent = gsm8k.GSM8KAgent()
  action = agent.update_from_model("the answer is 4")
  out = env.step(action)
  assert out[1] == 1.0 and out[2] is True and out[0]["gold_answer"] == "4"
  assert agent.trajectory.steps[-1].model_response == "the answer is 4"
  wrong = gsm8k.GSM8KEnv(prompt="2 + 2?", gold_answer="4")
  wrong.reset()
  assert wrong.step("five")[1] == 0.0


def test_every_node_builds_the_same_tiny_model():
  a, b = models.build_model("tiny", seed=0, device="cpu"), models.build_model("tiny", seed=0, device="cpu")
  assert all(torch.equal(p, q) for p, q in zip(a.parameters(), b.parameters()))
  tok = models.build_tokenizer("tiny")
  assert tok.decode(tok.encode("2 + 2 = 4")) == "2 + 2 = 4" and max(tok.encode("~")) < models.TINY_VOCAB
  assert models.pad_and_eos(tok) == (0, 2)
  with pytest.raises(ValueError, match="--tokenizer"):
    models.build_tokenizer("qwen3-0.6b")
  unit = run_trainer_node  # the node modules import without side effects
  assert unit.main and run_rollout_node.main and run_inference_node.main
  info = node_common.parse_announcement(node_common.announcement("actor", "t0", 5))
  assert info == {"role": "actor", "worker_id": "t0", "rpc_port": 5}


@pytest.mark.timeout(300)
def test_the_whole_system_trains_and_syncs_weights_over_the_wire(monkeypatch):
  node_common.stop.clear()
  disc = free_port()
  captured = {}
  built = {}
  original_run, original_rollout = control.run, run_rollout_node.build_worker

  def recording_run(ctx, args):
    captured["history"] = original_run(ctx, args)
    return captured["history"]

  def recording_rollout(args):
    out = original_rollout(args)
    built["rollout_model"] = out[2]._model
    built["before"] = {n: p.detach().clone() for n, p in out[2]._model.named_parameters()}
    return out
  monkeypatch.setattr(control, "run", recording_run)
  monkeypatch.setattr(run_rollout_node, "build_worker", recording_rollout)
  node = lambda name, did, *flags: ["--process", f"--process_main={PKG}.{name}.main", f"--discovery_id={did}",   # noqa: E731
                                    f"--discovery_addrs=control:{disc}", "--port=0", *flags]
  try:
    rt_main.main(["prog",
                  "--process", f"--process_main={PKG}.run_gsm8k_dist_grpo.main", "--discovery_id=control",
                  f"--discovery_port={disc}", "--steps=2", "--num_generations=2", "--mini_batch_size=2",
                  "--num_prompts=6", "--max_prompt_length=160", "--max_response_length=8", "--reward=length",
                  "--wait_s=120", "--beta=0.04",
                  *node("run_trainer_node", "trainer", "--lr=1e-2"),
                  *node("run_rollout_node", "rollout", "--max_seq_len=192", "--page_size=16", "--max_batch=8"),
                  *node("run_inference_node", "inference")])
  finally:
    node_common.stop.clear()
  history = captured["history"]
  assert [r.policy_version for r in history] == [1, 2] and all(r.num_rollouts == 4 for r in history)
  moved = [n for n, p in built["rollout_model"].named_parameters() if not torch.equal(p, built["before"][n])]
  assert moved, "the rollout node's model never received new weights"
