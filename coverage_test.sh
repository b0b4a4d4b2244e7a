#!/bin/bash
# Model-coverage sweep: every model below goes through capture, planning, partitioning and two
# pipeline stages, and its losses are compared with the un-pipelined module (--check_valid).
# The reference's sweep runs TorchBench models; these are the ones that can be built offline
# (torchvision, HuggingFace configs with random weights, this package's own models).
#
#   ./coverage_test.sh            # 2 GPUs
#   CPU=1 ./coverage_test.sh      # 2 CPU ranks (gloo)
#   WORLD_SIZE=4 ./coverage_test.sh hf_Bert tv:resnet50      # chosen models only

declare -a MODELS=(
    toy
    tv:alexnet
    tv:densenet121
    tv:mnasnet1_0
    tv:mobilenet_v2
    tv:resnet18
    tv:resnet50
    tv:resnext50_32x4d
    tv:shufflenet_v2_x1_0
    tv:squeezenet1_1
    tv:vgg16
    tv:vit_b_16
    hf_Albert
    hf_Bert
    hf_Bert_large
    hf_DistilBert
    hf_GPT2
    hf_GPT2_large
    hf_Roberta
    vit_tiny
    llama_tiny
    unet_tiny
)
if [ "$#" -gt 0 ]; then MODELS=("$@"); fi

WORLD_SIZE=${WORLD_SIZE:-2}
PORT=${MASTER_PORT:-26100}
EXTRA=()
if [ -n "$CPU" ]; then EXTRA+=(--cpu); fi
cd "$(dirname "$0")" || exit 1

pass=0; fail=0; failed=()
for val in "${MODELS[@]}"; do
    PORT=$((PORT + 1))
    if python mp_launch.py --world_size "$WORLD_SIZE" --master_port "$PORT" "${EXTRA[@]}" \
        benchmark_mp.py --batch_size=1 --batch_cnt=2 --valid_steps=2 \
        --model="$val" --loop_cnt=1 --prefetch_fwd=0 --no_bench_optimizer --check_valid \
        > "/tmp/coverage_${val//[:\/]/_}.log" 2>&1; then
        echo "PASS $val"; pass=$((pass + 1))
    else
        echo "FAIL $val (see /tmp/coverage_${val//[:\/]/_}.log)"; fail=$((fail + 1)); failed+=("$val")
    fi
done
echo "passed $pass, failed $fail ${failed[*]}"
[ "$fail" -eq 0 ]
