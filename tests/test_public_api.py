"""The top-level package exports the reference's public names (tunix/__init__.py:28-67)."""
import subprocess
import sys

import pytest

import tunix_b200

REFERENCE_NAMES = """CacheConfig ClusterConfig RLTrainingConfig RolloutConfig TrainingConfig Role DistillationTrainer
DistillationTrainingConfig Sampler Tokenizer TokenizerAdapter PerfMetricsExport PerfMetricsConfig PerfSpanQuery
AgenticGRPOConfig AgenticGRPOLearner GRPOConfig GrpoConfig GRPOLearner GrpoLearner RewardFn PPOConfig PpoConfig
PPOLearner PpoLearner MetricsBuffer RLCluster RLEngine CheckpointManager DPOTrainer DpoTrainer DPOTrainingConfig
DpoTrainingConfig ORPOTrainer OrpoTrainer ORPOTrainingConfig OrpoTrainingConfig MetricsLogger MetricsLoggerOptions
PeftTrainer""".split()


@pytest.mark.parametrize("name", REFERENCE_NAMES)
def test_name_resolves(name):
  obj = getattr(tunix_b200, name)
  assert obj is not None
  assert name in tunix_b200.__all__


def test_aliases_point_at_one_object():
  assert tunix_b200.GrpoLearner is tunix_b200.GRPOLearner
  assert tunix_b200.DpoTrainer is tunix_b200.DPOTrainer
  assert tunix_b200.AgenticGRPOLearner is not tunix_b200.GRPOLearner


def test_unknown_name_raises_attribute_error():
  with pytest.raises(AttributeError):
    tunix_b200.NoSuchThing


def test_import_is_lazy():
  code = "import sys, tunix_b200; assert 'torch' not in sys.modules; from tunix_b200 import Role; print(Role)"
  r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True)
  assert r.returncode == 0, r.stderr
