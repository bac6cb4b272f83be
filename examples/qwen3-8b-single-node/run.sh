#!/usr/bin/env bash
# Online DSpark training of a Qwen3-8B-shaped Draft on one node: 4 Target GPUs prefill, 4 Draft GPUs train.
# Usage: examples/qwen3-8b-single-node/run.sh [OUTPUT_DIR] [STEPS]
set -euo pipefail
OUT=${1:-outputs/qwen3_8b_single_node}
STEPS=${2:-50}
CLI="python -m aspec_b200.cli"
RECIPE=aspec_b200/recipes/qwen3_8b_dspark_1layer.yaml

python -m aspec_b200.build
$CLI doctor --gpu
# 1. the plan: what will run, on which GPUs, with which kernels; nothing starts
$CLI --config "$RECIPE" --dry-run output_dir="$OUT" training.num_train_steps="$STEPS" > /dev/null
# 2. train (synthetic corpus unless ASPEC_TRAIN_DATA is set)
$CLI --config "$RECIPE" output_dir="$OUT" training.num_train_steps="$STEPS" training.save_interval="$STEPS" \
     inference.inference_num_gpus=4 training.training_num_gpus_per_node=4
# 3. what happened, checked against what was planned
$CLI --report "$OUT"
# 4. export the last checkpoint to the native serving layout and propose blocks with it on held-out rows
LAST=$(cat "$OUT/checkpoints/latest_checkpointed_iteration.txt")
$CLI export --input-dir "$OUT/checkpoints/iter_$(printf %07d "$LAST")" --output-dir "$OUT/asset" --format aspec
$CLI evaluate --asset-dir "$OUT/asset" --synthetic 32
