#!/bin/bash
# SDXL finetuning smoke: trains STEPS steps and asserts that the mean of the last 10 losses is below LOSS_THRESHOLD.
#   bash end_to_end/gpu/test_sdxl_training_loss.sh MODEL_DIR=/models/sdxl-base DATASET=/data/pokemon_sdxl \
#        OUTPUT_DIR=/tmp/out RUN_NAME=sdxl-loss STEPS=200 LOSS_THRESHOLD=0.15 [GPUS=8]
set -euo pipefail
for ARGUMENT in "$@"; do
  IFS='=' read -r KEY VALUE <<< "$ARGUMENT"
  export "$KEY"="$VALUE"
done
: "${MODEL_DIR:?}" "${DATASET:?}" "${OUTPUT_DIR:?}" "${RUN_NAME:?}" "${STEPS:?}" "${LOSS_THRESHOLD:?}"
GPUS="${GPUS:-$(nvidia-smi -L | wc -l)}"
METRICS="${OUTPUT_DIR}/${RUN_NAME}/metrics.txt"
rm -f "$METRICS"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port "${PORT:-29511}" \
  -m maxdiffusion_b200.train_sdxl maxdiffusion_b200/configs/base_xl.yml \
  pretrained_model_name_or_path="$MODEL_DIR" dataset_name="$DATASET" dataset_type=hf resolution=1024 per_device_batch_size=1 \
  weights_dtype=bfloat16 activations_dtype=bfloat16 max_train_steps="$STEPS" write_metrics=True metrics_file="$METRICS" \
  run_name="$RUN_NAME" output_dir="$OUTPUT_DIR" log_config=false
python end_to_end/gpu/eval_assert.py final_loss "$METRICS" "$LOSS_THRESHOLD"
