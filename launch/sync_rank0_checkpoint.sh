#!/bin/bash
# Between two jobs of a chained run: every rank's checkpoint directory becomes a copy of rank 0's
# (the reference's test_scripts_imagenet/synchm.sh).  Usage: sync_rank0_checkpoint.sh <model_dir> [world]
set -euo pipefail
python -m eagersgd_b200.ckpt.sync_dirs "$1" ${2:+--world "$2"}
