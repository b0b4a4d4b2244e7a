#!/bin/bash
# ViT-g/14 on the GPUs of one node: micro-batch 24 x 8 micro-batches per replica, fp16.
# The mesh is the launcher's: leave --dp_mesh out for one pipeline over all ranks, or name it,
# e.g. DP_MESH="-8,1" for eight replicas, "-2,4" for two pipelines of four stages.
WORLD_SIZE=${WORLD_SIZE:-8}
DP_MESH=${DP_MESH:--${WORLD_SIZE},1}
cd "$(dirname "$0")/.." || exit 1
python mp_launch.py --world_size "$WORLD_SIZE" --dp_mesh="$DP_MESH" examples/train_vit.py \
  --batch_size 24 \
  --batch_cnt 8 \
  --mixed_precision fp16 \
  --cuda_graphs \
  "$@"
