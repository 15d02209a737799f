#!/bin/bash
# Launches COMMAND (a `python -m maxdiffusion_b200.<entry> <config> key=value …` line without the leading `python`)
# as one process per GPU on every node of a multi-node job. Run the same line on each node with its own NODE_RANK.
#   NNODES=2 NODE_RANK=0 COORDINATOR_ADDRESS=10.0.0.1 COORDINATOR_PORT=29500 GPUS_PER_NODE=8 \
#   COMMAND="-m maxdiffusion_b200.train_wan maxdiffusion_b200/configs/base_wan_14b.yml dcn_data_parallelism=2" \
#   bash gpu_multi_process_run.sh
set -euo pipefail
: "${NNODES:?Must set NNODES}"
: "${NODE_RANK:?Must set NODE_RANK}"
: "${COORDINATOR_ADDRESS:?Must set COORDINATOR_ADDRESS}"
: "${COORDINATOR_PORT:?Must set COORDINATOR_PORT}"
: "${GPUS_PER_NODE:?Must set GPUS_PER_NODE}"
: "${COMMAND:?Must set COMMAND}"

# NVLink / NVSwitch inside the node, the fabric NCCL detects between nodes. Only library defaults are steered here;
# nothing that outlasts the job (clocks, persistence mode) is touched.
export NCCL_DEBUG="${NCCL_DEBUG:-WARN}"
export NCCL_NVLS_ENABLE="${NCCL_NVLS_ENABLE:-1}"
export CUDA_DEVICE_MAX_CONNECTIONS="${CUDA_DEVICE_MAX_CONNECTIONS:-8}"
export TORCH_NCCL_ASYNC_ERROR_HANDLING="${TORCH_NCCL_ASYNC_ERROR_HANDLING:-1}"
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-8}"

echo "node ${NODE_RANK}/${NNODES}: ${GPUS_PER_NODE} ranks, coordinator ${COORDINATOR_ADDRESS}:${COORDINATOR_PORT}"
# shellcheck disable=SC2086
# MAX_RESTARTS > 0: when a rank fails (its own exception, or a peer's seen through the health monitor) every rank is
# torn down and started again; the trainers resume from the latest checkpoint.
exec python -m torch.distributed.run --nnodes="$NNODES" --node-rank="$NODE_RANK" --nproc-per-node="$GPUS_PER_NODE" \
  --master-addr "$COORDINATOR_ADDRESS" --master-port "$COORDINATOR_PORT" --max-restarts "${MAX_RESTARTS:-0}" $COMMAND
