#!/bin/bash
# Llama-2-7B, 2048-token samples, one sample per micro-batch, 16 micro-batches; a looped pipeline
# of 16 stages on 8 ranks.  With DP_MESH="-2,4" and --use_fsdp the matrices of every stage stay
# sharded over the two replicas between optimizer steps.
WORLD_SIZE=${WORLD_SIZE:-8}
DP_MESH=${DP_MESH:-${WORLD_SIZE}}
cd "$(dirname "$0")/.." || exit 1
python mp_launch.py --world_size "$WORLD_SIZE" --dp_mesh="$DP_MESH" examples/train_llama.py \
  --block_size 2048 \
  --per_device_train_batch_size 1 \
  --batch_cnt 16 \
  --loop_cnt 2 \
  --mixed_precision bf16 \
  "$@"
