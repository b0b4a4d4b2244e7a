#!/bin/bash
# SDXL UNet at 1024 x 1024 (128 x 128 latents): two stages x four replicas, micro-batch 4 x 8.
WORLD_SIZE=${WORLD_SIZE:-8}
DP_MESH=${DP_MESH:-2,-4}
cd "$(dirname "$0")/.." || exit 1
python mp_launch.py --world_size "$WORLD_SIZE" --dp_mesh="$DP_MESH" examples/train_sdxl.py \
  --resolution 1024 \
  --train_batch_size 4 \
  --batch_cnt 8 \
  --proportion_empty_prompts 0.2 \
  --learning_rate 1e-06 \
  --mixed_precision bf16 \
  "$@"
