#!/usr/bin/env bash
# DSA Draft in three stages.  Each stage starts from the previous stage's weights (a weights-only transition: fresh
# optimizer, masters re-derived), because the set of trainable parameters changes between stages:
#   dense           the Draft trains with full attention; the indexer is idle
#   indexer_warmup  everything but the indexer is frozen; the indexer learns the attention distribution (KL)
#   sparse          attention reads only the indexer's top-k keys; Draft and indexer train together
# Usage: examples/qwen3-8b-dsa/run.sh [OUTPUT_ROOT] [STEPS_PER_STAGE]
set -euo pipefail
ROOT=${1:-outputs/qwen3_8b_dsa}
STEPS=${2:-30}
CLI="python -m aspec_b200.cli"
RECIPE=aspec_b200/recipes/qwen3_8b_dsa_sparse_dspark.yaml
PREV=""
for STAGE in dense indexer_warmup sparse; do
  OUT="$ROOT/$STAGE"
  EXTRA=()
  if [ -n "$PREV" ]; then
    EXTRA=(training.load_path="$PREV/checkpoints" training.continual_training=true)
  fi
  $CLI --config "$RECIPE" output_dir="$OUT" training.num_train_steps="$STEPS" training.save_interval="$STEPS" \
       model.draft_overrides.dsa_training_stage="$STAGE" "${EXTRA[@]}"
  $CLI --report "$OUT"
  PREV="$OUT"
done
