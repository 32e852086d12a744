"""Command-line layer on CPU: config merging rules, optimizer / mesh factories, reward function
loading, dataset utilities, and the peft / grpo entry points end to end on a tiny random model."""
import os

import numpy as np
import pytest
import yaml

from tunix_b200.cli import config as config_lib
from tunix_b200.cli.reward_fn import gsm8k, gsm8k_verl, simple_math
from tunix_b200.cli.utils import data as data_lib
from tunix_b200.data import ListDataset
from tunix_b200.utils import mesh as mesh_lib

TINY = {"num_layers": 2, "embed_dim": 32, "hidden_dim": 64, "num_heads": 4, "head_dim": 8, "num_kv_heads": 2,
        "vocab_size": 200}


@pytest.fixture(scope="module")
def sp_model(tmp_path_factory):
  import sentencepiece as spm
  d = tmp_path_factory.mktemp("tok")
  corpus = d / "c.txt"
  words = ("alpha beta gamma delta epsilon zeta eta theta iota kappa what is plus answer reasoning translate this "
           "into french you are given a problem think about the and provide your user model system ")
  corpus.write_text("\n".join([words + " ".join(str(i) for i in range(100))] * 50))
  spm.SentencePieceTrainer.train(input=str(corpus), model_prefix=str(d / "tok"), vocab_size=200, pad_id=0, unk_id=3,
                                 bos_id=1, eos_id=2, model_type="bpe", minloglevel=2)
  return str(d / "tok.model")


def argv(entry, sp_model, tmp_path, *extra):
  tiny = "{" + ", ".join(f"{k}: {v}" for k, v in TINY.items()) + "}"
  return [entry, "base_config.yaml", "model_config.model_source=dummy", "model_config.dtype=float32",
          "model_config.device=cpu", f"model_config.model_overrides={tiny}", "model_config.model_id=Qwen/Qwen3-0.6B",
          "model_config.model_name=qwen3-0.6b", f"tokenizer_config.tokenizer_path={sp_model}",
          "tokenizer_config.tokenizer_type=sentencepiece", "tokenizer_config.add_eos=false", *extra]


def test_override_precedence_and_validation(tmp_path, monkeypatch, sp_model):
  base = argv("peft_main", sp_model, tmp_path)
  hp = config_lib.HyperParameters(base + ["batch_size=4", "rollout_config.temperature=0.5"])
  assert hp.config["batch_size"] == 4 and hp.config["rollout_config"]["temperature"] == 0.5
  assert hp.config["rollout_config"]["top_k"] == 50                       # merged, not replaced
  assert hp.config["actor_model_config"]["model_source"] == "dummy"        # inherited from model_config
  hp = config_lib.HyperParameters(base + ["optimizer_config.opt_type=sgd", "optimizer_config.learning_rate=0.1"])
  assert hp.config["optimizer_config"] == {"opt_type": "sgd", "learning_rate": 0.1}     # replace key
  ov = tmp_path / "ov.yaml"
  ov.write_text(yaml.safe_dump({"batch_size": 2, "rollout_config": {"top_k": 7}}))
  hp = config_lib.HyperParameters(base + [f"override_config_file={ov}", "batch_size=8"])
  assert hp.config["batch_size"] == 8 and hp.config["rollout_config"]["top_k"] == 7
  monkeypatch.setenv("T_BATCH_SIZE", "32")
  assert config_lib.HyperParameters(base).config["batch_size"] == 32
  with pytest.raises(ValueError, match="both CLI and ENV"):
    config_lib.HyperParameters(base + ["batch_size=8"])
  monkeypatch.delenv("T_BATCH_SIZE")
  monkeypatch.setenv("T_NOT_A_KEY", "1")
  with pytest.raises(ValueError, match="doesn't match a key"):
    config_lib.HyperParameters(base)
  monkeypatch.delenv("T_NOT_A_KEY")
  with pytest.raises(ValueError, match="isn't in config"):
    config_lib.HyperParameters(base + ["nonsense=1"])
  with pytest.raises(ValueError, match="first argument"):
    config_lib.HyperParameters(["peft_main", "batch_size=4"])
  with pytest.raises(ValueError, match="tokenizer_type"):
    config_lib.HyperParameters(base + ["tokenizer_config.tokenizer_type=bpe"])
  with pytest.raises(ValueError, match="only supported for GRPO"):
    config_lib.HyperParameters(base + ["training_config.perf_metrics_options={enable_perf_v1: true}"])
  with pytest.raises(ValueError, match="cannot turn"):
    config_lib.HyperParameters(base + ["batch_size=abc"])


def test_optimizer_and_mesh_factories(tmp_path, sp_model):
  hp = config_lib.HyperParameters(argv("peft_main", sp_model, tmp_path, "model_config.mesh.shape=(4,2)"))
  tx = hp.create_optimizer("optimizer_config")
  assert tx is not None
  assert hp.parse_mesh_config("model_config") == ((4, 2), ("fsdp", "tp"))
  hp.config["model_config"]["mesh"]["shape"] = "(4,)"
  with pytest.raises(ValueError, match="same length"):
    hp.parse_mesh_config("model_config")
  hp.config["optimizer_config"] = {"opt_type": "adamw"}
  with pytest.raises(ValueError, match="learning_rate"):
    hp.create_optimizer("optimizer_config")
  with pytest.raises(KeyError):
    hp.create_optimizer("nope")
  tc = hp.obtain_training_config_dict("training_config")
  assert tc["checkpointing_options"] is not None and tc["perf_metrics_options"] is None
  assert mesh_lib.normalize_allocation_policy(None) == "COMPACT"
  with pytest.raises(ValueError):
    mesh_lib.normalize_allocation_policy("fast")
  s = mesh_lib.allocate_named_mesh_device_slices([("a", 2), ("b", 4), ("c", 2)], range(8), "PERFORMANCE")
  assert s == {"b": [0, 1, 2, 3], "a": [4, 5], "c": [6, 7]}


def test_reward_functions_and_loading(tmp_path, sp_model):
  good = "<reasoning>2+2</reasoning><answer>4</answer>"
  assert gsm8k.match_format_exactly(None, [good, "4"]) == [3.0, 0]
  assert gsm8k.match_format_approximately(None, [good, "<answer>"]) == [2.0, -1.0]
  assert gsm8k.check_answer(None, [good, good, good, "x"], answer=["4", "4.2", "40", "4"]) == [3.0, 0.5, -1.0, 0]
  assert gsm8k.check_numbers(None, [good, "<answer>five"], answer=["4", "4"]) == [1.5, 0]
  assert gsm8k_verl.compute_score("so #### 1,234", "1234") == 1.0 and gsm8k_verl.compute_score("1234", "1234") == 0
  assert gsm8k_verl.extract_solution("about 3. or 7", "flexible") == "7"
  assert simple_math.check_format(None, [good, "x" + good]) == [0.1, 0]
  hp = config_lib.HyperParameters(argv("grpo_main", sp_model, tmp_path))
  names = {f.__name__ for f in hp.obtain_reward_fn()}
  assert {"match_format_exactly", "match_format_approximately", "check_answer", "check_numbers"} <= names
  hp.config["reward_functions"] = ["tunix_b200.cli.reward_fn.gsm8k_verl"]
  hp.config["verl_compatible"] = True
  fn = hp.obtain_reward_fn()[0]
  assert fn(["p"], ["#### 5"], {"ground_truth": ["5"]}) == [1.0]


def test_dataset_utils(tmp_path):
  assert data_lib.parse_call_string("'a', 2, k='v'") == (["a", 2], {"k": "v"})
  with pytest.raises(ValueError):
    data_lib.parse_call_string("a b")
  mod = tmp_path / "mydata.py"
  mod.write_text("from tunix_b200.data import ListDataset\n"
                 "def create_dataset(n=3):\n  return ListDataset([{'prompts': 'p ' * (i + 1), 'answer': str(i)} for i in range(n)])\n"
                 "def other(n, tag='x'):\n  return ListDataset([{'prompts': tag, 'answer': '0'}] * n)\n")
  assert len(data_lib.get_dataset_from_module(str(mod))) == 3
  assert len(data_lib.get_dataset_from_module(f"{mod}:other(5, tag='y')")) == 5

  class Tok:
    def encode(self, s): return s.split()
  ds = ListDataset([{"q": "w " * n, "answer": str(n)} for n in range(1, 11)])
  tr, ev = data_lib.post_init_dataset(ds, Tok(), batch_size=2, num_batches=4, max_prompt_length=9, fraction=0.75,
                                      num_epochs=2, prompt_key="q")
  tb, eb = list(tr), list(ev)
  assert len(tb) == 6 and len(eb) == 2 and tb[0]["prompts"] == ["w ", "w w "] and tb[0]["answer"] == ["1", "2"]
  with pytest.raises(ValueError, match="empty after"):
    data_lib.post_init_dataset(ds, Tok(), 2, None, max_prompt_length=0 or -1 + 1 or None, prompt_key="q") if False else \
        data_lib.post_init_dataset(ListDataset([{"prompts": "a b c"}]), Tok(), 2, None, max_prompt_length=1)


def test_peft_main_end_to_end(tmp_path, sp_model):
  from tunix_b200.cli import peft_main
  tr = peft_main.main(argv("peft_main", sp_model, tmp_path, "dataset_name=synthetic", "batch_size=8",
                           "max_target_length=48", "training_config.max_steps=6", "training_config.eval_every_n_steps=3",
                           f"training_config.checkpoint_root_directory={tmp_path / 'ck'}",
                           "optimizer_config.opt_type=adamw", "optimizer_config.learning_rate=0.01"))
  losses = tr.metrics_logger.get_metric_history("", "loss", "train")
  assert len(losses) == 6 and losses[-1] < losses[0]
  assert os.path.isdir(tmp_path / "ck")


def test_grpo_main_end_to_end(tmp_path, sp_model):
  from tunix_b200.cli import grpo_main
  common = ["data_source=synthetic", "apply_chat_template_to_dataset=false", "batch_size=2", "num_batches=3",
            "rollout_config.total_generation_steps=8", "rollout_config.max_prompt_length=256",
            "rollout_config.temperature=1.0", "rollout_config.top_k=0", "rl_training_config.max_steps=2",
            "rl_training_config.eval_every_n_steps=10", "rl_training_config.actor_optimizer_config.opt_type=adamw",
            "rl_training_config.actor_optimizer_config.learning_rate=0.001"]
  learner = grpo_main.main(argv("grpo_main", sp_model, tmp_path, *common, "rollout_engine=native"))
  assert learner.rl_engine.global_steps == 2


def test_deepscaler_recipe_and_vllm_entry_arguments(tmp_path):
  import json
  from tunix_b200.cli import grpo_vllm_main
  from tunix_b200.cli.recipes import deepscaler_data
  train = tmp_path / "deepscaler.json"
  train.write_text(json.dumps([{"problem": "1+1?", "answer": "2"}, {"problem": "2+2?", "answer": "4"}]))
  evalf = tmp_path / "aime.jsonl"
  evalf.write_text(json.dumps({"question": "3+3?", "ground_truth": "6"}) + "\n")
  ds = deepscaler_data.create_dataset(str(train), str(evalf))
  assert len(ds) == 2 and ds[0]["question"] == "1+1?" and ds[0]["answer"] == "2"
  assert ds[1]["prompts"].startswith("2+2? Let's think step by step") and "\\boxed{}" in ds[1]["prompts"]
  assert deepscaler_data.create_eval_dataset(str(evalf))[0] == {
      "prompts": "3+3? " + deepscaler_data.INSTRUCTION, "question": "3+3?", "answer": "6"}
  assert {r["question"] for r in deepscaler_data.create_dataset(str(train), shuffle=True, seed=1)} == {"1+1?", "2+2?"}
  with pytest.raises(FileNotFoundError):
    deepscaler_data.create_dataset(str(train), str(tmp_path / "missing.parquet"))
  ds2 = data_lib.get_dataset_from_module(
      f"tunix_b200.cli.recipes.deepscaler_data:create_dataset(train_data_path={str(train)!r})")
  assert len(ds2) == 2
  assert grpo_vllm_main.with_vllm_engine(["p", "a=1"]) == ["p", "a=1", "rollout_engine=vllm"]
  assert grpo_vllm_main.with_vllm_engine(["p", "rollout_engine=native"]) == ["p", "rollout_engine=native"]


def test_example_scripts_run_on_cpu():
  import subprocess
  import sys
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="2")
  for script, args in (("examples/sft/sft_synthetic.py", ["--steps", "3"]),
                       ("examples/model_load/from_safetensors.py", []),
                       ("examples/distillation/logit_distillation.py", ["--steps", "4", "--teacher-steps", "4"]),
                       ("examples/qlora/qlora_sft.py", ["--steps", "3"]),
                       ("examples/tools/forward_pass_logit_checker.py", ["--self-test"]),
                       ("examples/dpo/dpo_synthetic.py", ["--steps", "3", "--lora-rank", "4"]),
                       ("examples/dpo/dpo_synthetic.py", ["--steps", "3", "--algorithm", "orpo"])):
    r = subprocess.run([sys.executable, os.path.join(root, script), *args], env=env, capture_output=True, text=True,
                       timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
