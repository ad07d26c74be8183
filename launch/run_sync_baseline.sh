#!/bin/bash
# Synchronous NCCL data-parallel baseline with the same model, data and injected imbalance
# (the reference's Horovod job: test_scripts_imagenet/daint_hvd_imagenet.sh).
set -euo pipefail
N=${1:-8}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 --master-port 29501 \
  -m eagersgd_b200.train.resnet_main --dataset imagenet -hvd -rs 50 -rv 1 -bs 128 -te 90 --synthetic \
  --imbalance sleep --imbalance_seconds 0.32
