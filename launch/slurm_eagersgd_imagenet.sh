#!/bin/bash
# ImageNet ResNet-50 with solo eager-SGD on one 8-GPU B200 node per task group.
# The reference runs 64 single-GPU nodes with a warm-up epoch and nine 10-epoch jobs, copying
# rank 0's checkpoint over the others between jobs (test_scripts_imagenet/daint_eagersgd_imagenet.sh,
# synchm.sh); here one job covers the run and replicas are re-synchronised in place every 10 epochs.
#SBATCH --job-name=eagersgd_imagenet
#SBATCH --nodes=1
#SBATCH --ntasks-per-node=8
#SBATCH --gpus-per-node=8
#SBATCH --time=06:00:00
set -euo pipefail
export MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
export MASTER_PORT=${MASTER_PORT:-29500}
MODEL_DIR=${MODEL_DIR:-$SCRATCH/eagersgd_resnet50}
python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr $MASTER_ADDR --master-port $MASTER_PORT \
  -m eagersgd_b200.train.resnet_main --dataset imagenet -solo -rs 50 -rv 1 -bs 128 -te 90 -ebe 10 \
  --resync_epochs 10 --imbalance sleep --imbalance_seconds 0.32 --model_dir "$MODEL_DIR" ${DATA_DIR:+--data_dir "$DATA_DIR"} \
  ${DATA_DIR:---synthetic}
