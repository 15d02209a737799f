#!/bin/bash
# Wan 2.1 14B text-to-video with the step-cache and CFG-cache shortcuts on, all GPUs of the node as one context group.
#   bash end_to_end/gpu/run_wan_fast_inference.sh MODEL_DIR=/models/Wan2.1-T2V-14B-Diffusers OUTPUT_DIR=/tmp/wan [GPUS=8]
set -euo pipefail
for ARGUMENT in "$@"; do
  IFS='=' read -r KEY VALUE <<< "$ARGUMENT"
  export "$KEY"="$VALUE"
done
: "${MODEL_DIR:?}" "${OUTPUT_DIR:?}"
GPUS="${GPUS:-$(nvidia-smi -L | wc -l)}"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port "${PORT:-29512}" \
  -m maxdiffusion_b200.generate_wan maxdiffusion_b200/configs/base_wan_14b.yml \
  pretrained_model_name_or_path="$MODEL_DIR" output_dir="$OUTPUT_DIR" run_name="${RUN_NAME:-wan-fast}" \
  height=720 width=1280 num_frames=81 num_inference_steps=50 attention=flash ici_context_parallelism="$GPUS" \
  context_strategy=ulysses use_cfg_cache=True use_magcache=True log_config=false
