"""Command-line flags of the training mains.

Same names (long and short) as the reference's absl flag groups
(official/utils/flags/_base.py:28-141, _performance.py:46-141, _benchmark.py:26-99 and the
ResNet / eager-SGD flags in resnet_run_loop_solo_imagenet_300.py:693-758), on argparse.
"""
from __future__ import annotations

import argparse

# The reference's half-precision choice is fp16 with a static loss scale of 128 (official/utils/flags/
# _performance.py:30-43).  The kernels here compute in bfloat16, which needs no loss scaling; float16 is
# not offered because the partial-allreduce and tensor-core kernels read 16-bit data as bfloat16.
DTYPE_MAP = {"bf16": ("bfloat16", 1.0), "fp32": ("float32", 1.0)}


def define_base(p: argparse.ArgumentParser):
    g = p.add_argument_group("base")
    g.add_argument("--data_dir", "-dd", default=None)
    g.add_argument("--model_dir", "-md", default="/tmp/eagersgd_model")
    g.add_argument("--clean", action="store_true")
    g.add_argument("--train_epochs", "-te", type=float, default=90)
    g.add_argument("--epochs_between_evals", "-ebe", type=int, default=1)
    g.add_argument("--stop_threshold", "-st", type=float, default=None)
    g.add_argument("--batch_size", "-bs", type=int, default=128, help="per-rank batch size")
    g.add_argument("--max_train_steps", "-mts", type=int, default=None)
    g.add_argument("--export_dir", "-ed", default=None)
    g.add_argument("--hooks", "-hk", default="LoggingTensorHook,ExamplesPerSecondHook")


def define_performance(p):
    g = p.add_argument_group("performance")
    g.add_argument("--dtype", "-dt", default="bf16", choices=sorted(DTYPE_MAP))
    g.add_argument("--loss_scale", "-ls", type=float, default=None)
    g.add_argument("--use_synthetic_data", "-synth", "--synthetic", action="store_true")
    g.add_argument("--num_parallel_calls", "-npc", type=int, default=4)
    g.add_argument("--cuda_graph", action="store_true")


def define_benchmark(p):
    g = p.add_argument_group("benchmark")
    g.add_argument("--benchmark_logger_type", "-blt", default="BaseBenchmarkLogger",
                   choices=["BaseBenchmarkLogger", "BenchmarkFileLogger"])
    g.add_argument("--benchmark_log_dir", "-bld", default=None)
    g.add_argument("--benchmark_test_id", "-bti", default=None)


def define_resnet(p, default_size=50, sizes=(18, 34, 50, 101, 152, 200)):
    g = p.add_argument_group("resnet / eager-SGD")
    g.add_argument("--resnet_size", "-rs", type=int, default=default_size)
    g.add_argument("--resnet_version", "-rv", type=int, default=1, choices=[1, 2])
    g.add_argument("--fine_tune", "-ft", action="store_true")
    g.add_argument("--pretrained_model_checkpoint_path", "-pmcp", default=None)
    g.add_argument("--eval_only", action="store_true")
    g.add_argument("--mode", default="solo", choices=["solo", "majority", "sync", "ddp"])
    g.add_argument("--solodance", "-solo", action="store_true", help="same as --mode solo")
    g.add_argument("--horovod", "-hvd", action="store_true", help="same as --mode ddp (synchronous NCCL baseline)")
    g.add_argument("--limiter", type=int, default=32)
    g.add_argument("--bucket_mb", type=float, default=25.0)
    g.add_argument("--accumulate", action="store_true",
                   help="fold a gradient that no round picked up into the rank's next one (default: it is superseded, "
                        "as in the reference)")
    g.add_argument("--baseseed", "-bse", type=int, default=1234,
                   help="seed of the replicas' initial weights, of the data order and of the injected delays")
    g.add_argument("--shuffleaug", "-saug", type=int, default=1,
                   help="groups of this many consecutive ranks read the same samples in the same order (each with its own "
                        "augmentation); the data are divided among world / shuffleaug groups")
    g.add_argument("--regime", "-fr", type=int, default=0, choices=[0, 1, 2],
                   help="ImageNet learning-rate boundaries: 0 = 30/60/80/90 epochs, 1 = 30/35/39/40, 2 = 15/20/22/30")
    g.add_argument("--lrmult", type=float, default=1.0)
    g.add_argument("--disablewarmup", action="store_true")
    g.add_argument("--start_epoch", type=int, default=0)
    g.add_argument("--lars", action="store_true")
    g.add_argument("--poly_rate", type=float, default=0.0)
    g.add_argument("--train_acc_steps", type=int, default=10)
    g.add_argument("--resync_epochs", type=int, default=10, help="re-synchronise replicas from rank 0 every N epochs")
    g.add_argument("--weight_decay", type=float, default=None,
                   help="L2 coefficient (default: the reference's value for the data set, 1e-4)")
    g.add_argument("--imbalance", default="none",
                   choices=["none", "sleep", "random_rank", "exponential", "constant"])
    g.add_argument("--imbalance_seconds", type=float, default=0.32)
    g.add_argument("--batchaug", type=int, default=1)
    g.add_argument("--virtual_batch_size", type=int, default=None)


def build_parser(description: str, default_size: int = 50) -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description=description)
    define_base(p)
    define_performance(p)
    define_benchmark(p)
    define_resnet(p, default_size)
    return p


def resolve(args):
    if args.solodance:
        args.mode = "solo"
    if args.horovod:
        args.mode = "ddp"
    dtype, default_scale = DTYPE_MAP[args.dtype]
    args.torch_dtype = dtype
    if args.loss_scale is None:
        args.loss_scale = default_scale
    return args
