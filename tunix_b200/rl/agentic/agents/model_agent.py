"""Single-turn agent: the model's response is the action (tunix/rl/agentic/agents/model_agent.py:22-49)."""
from __future__ import annotations

import copy

from . import agent_types, base_agent


class ModelAgent(base_agent.ConversationAgentBase):
  def update_from_model(self, response: str, **kwargs) -> agent_types.Action:
    self.chat_completions.append({"role": "assistant", "content": response})
    self.trajectory.steps.append(agent_types.Step(chat_completions=copy.deepcopy(self.chat_completions),
                                                  action=agent_types.Action(action=response),
                                                  model_response=response))
    return agent_types.Action(action=response)
