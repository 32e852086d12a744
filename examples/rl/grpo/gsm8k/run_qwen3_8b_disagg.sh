#!/bin/bash
# Qwen3-8B GRPO on one 8 x B200 node: FSDP trainer over all 8 GPUs, rollout replicas tensor-parallel over pairs
# of GPUs (TP 2 x DP 4), weights re-laid-out from the trainer's flat buffer into every replica after each step by
# one copy-kernel launch per rank (the layout of examples/rl/grpo/gsm8k/run_qwen3_8b_disagg.sh in the reference:
# rollout tensor_parallel_size 2, data_parallel_size 4).
#
#   bash examples/rl/grpo/gsm8k/run_qwen3_8b_disagg.sh            # synthetic prompts, random-init weights
#   ROLLOUT_TP=8 bash examples/rl/grpo/gsm8k/run_qwen3_8b_disagg.sh
#
# Prints one JSON line: rollout, scoring, training and weight-sync times per step and tokens/s for the whole job.
set -euo pipefail
cd "$(dirname "$0")/../../../.."
NGPU=${NGPU:-8}
ROLLOUT_TP=${ROLLOUT_TP:-2}
STEPS=${STEPS:-3}
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 \
  --master-port "${MASTER_PORT:-29555}" bench.py --gpus "$NGPU" --workload grpo --model qwen3_8b \
  --rollout-tp "$ROLLOUT_TP" --steps "$STEPS" --warmup 1 \
  --grpo-prompts 64 --grpo-generations 8 --grpo-prompt-len 256 --grpo-new-tokens 768
