"""Enums naming the training mode and the model roles of an RL cluster
(same members as tunix/common/datatypes.py:20-37)."""
import enum


class Mode(enum.Enum):
  TRAIN = "train"
  EVAL = "eval"

  def __str__(self):
    return self.value


class Role(enum.Enum):
  ACTOR = "actor"
  CRITIC = "critic"
  REFERENCE = "reference"
  REWARD = "reward"
  ROLLOUT = "rollout"

  def __str__(self):
    return self.value
