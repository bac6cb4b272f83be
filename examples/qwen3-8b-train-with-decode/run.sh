#!/usr/bin/env bash
# Train with decode on one node: 6 Target GPUs continue the prompts of the corpus themselves (sampled decoding with
# cached keys / values; blocks of the live Draft are verified after every weight sync), 2 Draft GPUs train on what was
# written.
# Usage: examples/qwen3-8b-train-with-decode/run.sh [OUTPUT_DIR] [STEPS]
set -euo pipefail
OUT=${1:-outputs/qwen3_8b_train_with_decode}
STEPS=${2:-100}
CLI="python -m aspec_b200.cli"
RECIPE=aspec_b200/recipes/qwen3_8b_dspark_train_with_decode.yaml

python -m aspec_b200.build
$CLI doctor --gpu
$CLI --config "$RECIPE" --dry-run output_dir="$OUT" training.num_train_steps="$STEPS" > /dev/null
$CLI --config "$RECIPE" output_dir="$OUT" training.num_train_steps="$STEPS" training.save_interval="$STEPS"
# decode/generated_tokens, decode/tokens_per_target_pass and decode/accepted_draft_tokens_per_round are logged per update
$CLI --report "$OUT"
