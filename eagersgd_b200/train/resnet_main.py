"""ResNet training main: ImageNet and CIFAR-10 with eager-SGD (solo / majority), synchronous
partial allreduce, or the synchronous NCCL baseline.

    python -m eagersgd_b200.train.resnet_main --dataset imagenet -solo -rs 50 -rv 1 -bs 128 --synthetic
    torchrun --nproc-per-node 8 -m eagersgd_b200.train.resnet_main --dataset cifar10 --mode majority -rs 32 --synthetic

One program covers what the reference spreads over imagenet_main_eagersgd.py, imagenet_main_hvd.py,
cifar10_main.py and the run loops resnet_run_loop_{solo_imagenet_300,hvd_imagenet_300,hvd_cifar10}.py:
identical replicas from a shared seed (:510-513), per-rank model directories (:551-556), the seeded
imbalance injector (:288-298), learning-rate schedule with warm-up (:164-217), momentum or LARS
(:366-374), loss scaling (:398-416), rank-0 logging of loss / Prec@1 / Prec@5 (:582-623), train /
evaluate cycles (:662-684) and the export at the end (:686-690).  Replicas are re-synchronised from
rank 0 every ``--resync_epochs`` epochs, which the reference does by copying checkpoint directories
between launches (test_scripts_imagenet/synchm.sh).
"""
from __future__ import annotations

import contextlib
import os
import sys
import time

import numpy as np
import torch

from .model_helpers import past_stop_threshold
from .. import ckpt
from ..data import (OrderedSampler, ReplicateBatch, ShuffleSampler, SyntheticImageDataset, cifar10_transforms, load_cifar10,
                    partition)
from ..models.resnet import cifar_resnet, imagenet_resnet
from ..optim.lars import LARS, poly_rate_schedule
from ..parallel.group import init as init_group, finalize
from . import flags as F
from .imbalance import ConstantRanks, ExponentialDelays, FixedRanksSleep, NoImbalance, RandomRankFactor
from .logger import (BaseBenchmarkLogger, ExamplesPerSecondHook, ProfilerHook, benchmark_context, config_benchmark_logger,
                     parse_hooks, training_log_line)
from .metrics import topk_accuracy
from .schedule import cifar10_schedule, imagenet_schedule
from .step import TrainStep

DATASETS = {
    # weight decay 1e-4 in both programs (imagenet_main_eagersgd.py:358, cifar10_main.py:242); the ImageNet objective
    # leaves the batch-norm variables out of the L2 term, the CIFAR-10 one includes every variable (cifar10_main.py:244-250)
    # defaults when the flags are not given: ResNet-50 for 90 epochs with an evaluation after each (the reference runs them
    # as 1 + 9 x 10 in chained jobs, daint_eagersgd_imagenet.sh:34-44); ResNet-32 for 190 epochs, evaluated every 10
    # (cifar10_main.py:274-279)
    "imagenet": dict(train=1281167, val=50000, classes=1001, shape=(3, 224, 224), wd=1e-4, decay_norm=False, default_size=50,
                     train_epochs=90, epochs_between_evals=1),
    "cifar10": dict(train=50000, val=10000, classes=10, shape=(3, 32, 32), wd=1e-4, decay_norm=True, default_size=32,
                    train_epochs=190, epochs_between_evals=10),
}


def build_model(args, info):
    if args.dataset == "imagenet":
        return imagenet_resnet(args.resnet_size, args.resnet_version, info["classes"])
    return cifar_resnet(args.resnet_size, args.resnet_version, info["classes"])


def build_data(args, info, group):
    if args.use_synthetic_data or args.data_dir is None:
        n_train = args.synthetic_train_size or info["train"]
        train = SyntheticImageDataset(n_train, info["shape"], info["classes"], seed=1)
        val = SyntheticImageDataset(min(info["val"], 4 * args.batch_size), info["shape"], info["classes"], seed=2)
    elif args.dataset == "cifar10":
        train, val = load_cifar10(args.data_dir)
    else:
        # <data_dir>/{train,val}/<wnid>/*.JPEG, or the shards build_shards() packs from it
        from ..data.imagenet import ImageNetFolder, ShardedImageDataset
        if any(f.startswith("train-") and f.endswith(".npz") for f in os.listdir(args.data_dir)):
            train = ShardedImageDataset(args.data_dir, "train", seed=args.baseseed)
            val = ShardedImageDataset(args.data_dir, "val", seed=args.baseseed)
        else:
            train = ImageNetFolder(args.data_dir, "train", seed=args.baseseed)
            val = ImageNetFolder(args.data_dir, "val", seed=args.baseseed)
        info["train"], info["val"] = len(train), len(val)
        train.num_parallel_calls = val.num_parallel_calls = max(int(args.num_parallel_calls), 1)
        train.batchaug = max(int(args.batchaug), 1)      # copies are made before the random crop and flip
    # dataset.take(n // num_workers) in the reference (:94-96); with --shuffleaug M the workers are groups of M
    # consecutive ranks that share a part of the data and a shuffle seed (:82-88, :494-507)
    m = max(int(getattr(args, "shuffleaug", 1)), 1)
    workers = max(group.world // m, 1)
    shard = partition(train, min(group.rank // m, workers - 1), workers)
    seed = args.baseseed + 17 + (group.rank // m if m > 1 else 0)
    train_sampler, val_sampler = ShuffleSampler(shard, args.batch_size, seed=seed), OrderedSampler(val, args.batch_size)
    train_sampler.replicates = getattr(train, "batchaug", 1) > 1      # the data set hands out the copies itself
    if args.dataset == "cifar10" and not (args.use_synthetic_data or args.data_dir is None):
        # pad + random crop + flip + per-image standardisation; copies for batch augmentation are made before them
        for t in cifar10_transforms(True, seed=args.baseseed + 1000 * (group.rank + 1), batchaug=args.batchaug):
            train_sampler.add_input_transformation(t)
        for t in cifar10_transforms(False):
            val_sampler.add_input_transformation(t)
        train_sampler.replicates = True
    return train_sampler, val_sampler


def make_injector(args, group, step_time):
    w = group.world
    return {"none": lambda: NoImbalance(w),
            "sleep": lambda: FixedRanksSleep(w, args.imbalance_seconds, 2, seed=args.baseseed + 5),
            "random_rank": lambda: RandomRankFactor(w, step_time, 1.5, seed=args.baseseed + 5),
            "exponential": lambda: ExponentialDelays(w, step_time, 0.5, 2, seed=args.baseseed + 5),
            "constant": lambda: ConstantRanks(w, (0, 1), args.imbalance_seconds)}[args.imbalance]()


def evaluate(step: TrainStep, sampler, device):
    model = step.model
    model.eval()
    sampler.reset()
    top1 = top5 = n = 0.0
    with torch.no_grad():
        for batch in sampler:
            x = torch.as_tensor(batch["x"]).to(device)
            y = torch.as_tensor(batch["y"]).to(device)
            if device.type == "cuda":
                x = x.to(step.compute_dtype).contiguous(memory_format=torch.channels_last)
            a1, a5 = topk_accuracy(model(x), y, (1, min(5, model.fc.out_features)))
            top1 += a1 * len(y)
            top5 += a5 * len(y)
            n += len(y)
    model.train()
    return top1 / max(n, 1), top5 / max(n, 1)


def main(argv=None):
    p = F.build_parser(__doc__.split("\n")[0])
    p.add_argument("--dataset", default="imagenet", choices=sorted(DATASETS))
    p.add_argument("--synthetic_train_size", type=int, default=None, help="samples per epoch of synthetic data")
    p.set_defaults(resnet_size=None, train_epochs=None, epochs_between_evals=None)      # filled in per data set below
    args = F.resolve(p.parse_args(argv))
    info = DATASETS[args.dataset]
    if args.resnet_size is None:
        args.resnet_size = info["default_size"]
    if args.train_epochs is None:
        args.train_epochs = info["train_epochs"]
    if args.epochs_between_evals is None:
        args.epochs_between_evals = info["epochs_between_evals"]
    group = init_group()
    device = group.device
    torch.manual_seed(args.baseseed)      # identical initial replicas without a broadcast
    np.random.seed(args.baseseed)
    if args.clean and group.rank == 0:
        ckpt.clean(args.model_dir)
    group.barrier()

    model = build_model(args, info)
    if args.virtual_batch_size:                  # ghost batch norm (resnet_model.py:45-60)
        from ..models.resnet import BatchNormAct
        for m in model.modules():
            if isinstance(m, BatchNormAct):
                m.virtual_batch_size = int(args.virtual_batch_size)
    if args.fine_tune:                           # only the dense layer learns (run loop :404-416)
        for name, p_ in model.named_parameters():
            p_.requires_grad_(name.startswith("fc."))
    hooks = parse_hooks(args.hooks)
    global_batch = args.batch_size * group.world
    # an epoch is one pass of the groups of ranks that read different data (all ranks unless --shuffleaug)
    epoch_batch = args.batch_size * max(group.world // max(int(args.shuffleaug), 1), 1)
    steps_per_epoch = max((args.synthetic_train_size or info["train"]) // epoch_batch, 1)
    if args.dataset == "imagenet":
        lr_fn = imagenet_schedule(global_batch, info["train"], warmup=not args.disablewarmup, start_epoch=args.start_epoch,
                                  regime=args.regime)
    else:
        lr_fn = cifar10_schedule(global_batch, info["train"])
    wd = info["wd"] if args.weight_decay is None else args.weight_decay
    step = TrainStep(model, group, impl="ddp" if args.mode == "ddp" else "ours", mode=args.mode if args.mode != "ddp" else "sync",
                     limiter=args.limiter, bucket_mb=args.bucket_mb, lr=lr_fn(0) * args.lrmult, momentum=0.9,
                     weight_decay=wd, compute_dtype=getattr(torch, args.torch_dtype),
                     inner_optimizer=(lambda ps, **kw: LARS(ps, lr=kw["lr"], momentum=0.9, weight_decay=wd))
                     if args.lars else None, loss_scale=args.loss_scale, accumulate=args.accumulate,
                     decay_norm_params=info["decay_norm"])
    if args.pretrained_model_checkpoint_path:
        ckpt.import_tf_layout(step.model, args.pretrained_model_checkpoint_path, exclude=("dense",))
        if hasattr(step.opt, "refresh_master_from_params"):
            step.opt.refresh_master_from_params()    # the fp32 masters follow the imported weights
    global_step = ckpt.load(step.model, step.opt if hasattr(step.opt, "state_dict") else None, args.model_dir, group.rank)

    train_sampler, val_sampler = build_data(args, info, group)
    steps_per_epoch = max((args.synthetic_train_size or info["train"]) // epoch_batch, 1)   # a data set read from disk knows its size
    if args.benchmark_logger_type == "BenchmarkFileLogger" and not args.benchmark_log_dir:
        args.benchmark_logger_type = "BaseBenchmarkLogger"           # nowhere to write files to
    logger = config_benchmark_logger(args)                           # also what get_benchmark_logger() returns from now on
    if group.rank == 0:
        logger.log_run_info("resnet%d" % args.resnet_size, args.dataset, vars(args), args.benchmark_test_id)
    eps_hook = ExamplesPerSecondHook(global_batch, every_n_steps=max(args.train_acc_steps, 1), warm_steps=5,
                                     metric_logger=logger if group.rank == 0 else _Quiet())
    profiler = ProfilerHook(os.path.join(args.model_dir, str(group.rank))) if "ProfilerHook" in hooks else None
    replicate = ReplicateBatch(args.batchaug) if args.batchaug and args.batchaug > 1 and not train_sampler.replicates else None
    injector = None
    t_step = None
    captured = False

    def to_device(batch):
        x = torch.as_tensor(batch["x"]).pin_memory() if device.type == "cuda" else torch.as_tensor(batch["x"])
        y = torch.as_tensor(batch["y"])
        x = x.to(device, non_blocking=True)
        if device.type == "cuda":
            x = x.to(step.compute_dtype).contiguous(memory_format=torch.channels_last)
        return x, y.to(device, non_blocking=True)

    with benchmark_context(logger):
        epochs = int(np.ceil(args.train_epochs))
        for epoch in range(args.start_epoch, args.start_epoch + epochs):
            if args.eval_only:
                break
            train_sampler.reset()
            for batch in train_sampler:
                if args.max_train_steps is not None and global_step >= args.max_train_steps:
                    break
                lr = (poly_rate_schedule(global_step / steps_per_epoch, args.poly_rate, global_batch, epochs)
                      if args.lars else lr_fn(global_step)) * args.lrmult
                step.set_lr(lr)
                if injector is not None:
                    injector.apply(group.rank, device)
                t0 = time.perf_counter()
                if replicate is not None:            # batch augmentation: every sample several times per step
                    batch = replicate(batch)
                x, y = to_device(batch)
                if args.cuda_graph and not captured and device.type == "cuda" and args.mode != "ddp" \
                        and getattr(step.opt, "fused", False) and len(y) == args.batch_size * max(args.batchaug, 1):
                    step.capture(x, y)               # the whole step becomes one graph launch from here on
                    captured = True
                with (profiler.step(global_step) if profiler is not None else contextlib.nullcontext()):
                    loss = step.run_device(x, y)
                global_step += 1
                if "ExamplesPerSecondHook" in hooks:
                    eps_hook.after_step()
                if "LoggingTensorHook" in hooks and global_step % max(args.train_acc_steps, 1) == 0:
                    lv = float(loss)        # synchronises: only every train_acc_steps
                    if group.rank == 0:
                        with torch.no_grad():
                            step.model.eval()
                            a1, a5 = topk_accuracy(step.model(x), y, (1, min(5, info["classes"])))
                            step.model.train()
                        print(training_log_line(epoch, global_step, steps_per_epoch, lr, lv, a1, a5), flush=True)
                if injector is None and global_step == 5:   # calibrate the delay on undisturbed steps
                    if device.type == "cuda":
                        torch.cuda.synchronize()
                    t_step = time.perf_counter() - t0
                    injector = make_injector(args, group, max(t_step, 1e-3))
            if (epoch + 1) % args.epochs_between_evals == 0:
                a1, a5 = evaluate(step, val_sampler, device)
                if group.rank == 0:
                    logger.log_evaluation_result({"accuracy": a1, "accuracy_top_5": a5, "global_step": global_step})
                if past_stop_threshold(args.stop_threshold, a1):
                    break
            if args.resync_epochs and (epoch + 1) % args.resync_epochs == 0:
                ckpt.resync_from_rank0(step.model, step.opt if hasattr(step.opt, "resync_from_rank0") else None, group)
            ckpt.save(step.model, step.opt if hasattr(step.opt, "state_dict") else None, args.model_dir, group.rank,
                      global_step)
            if args.max_train_steps is not None and global_step >= args.max_train_steps:
                break
        if hasattr(step.opt, "flush"):
            step.opt.flush()
        if args.eval_only:
            a1, a5 = evaluate(step, val_sampler, device)
            if group.rank == 0:
                logger.log_evaluation_result({"accuracy": a1, "accuracy_top_5": a5, "global_step": global_step})
        if args.export_dir and group.rank == 0:
            ckpt.export_tf_layout(step.model, os.path.join(args.export_dir, "model.npz"),
                                  step.opt if hasattr(step.opt, "master_params") else None, global_step)
            # and the servable form: the inference graph with its weights as one .onnx file
            from ..graph import from_torch_resnet, save_onnx
            try:
                import copy
                frozen = copy.deepcopy(step.model).float().cpu().eval()
                save_onnx(from_torch_resnet(frozen), os.path.join(args.export_dir, "model.onnx"))
            except (TypeError, ValueError, AttributeError) as e:    # a model the graph builder does not cover
                print("no .onnx export for this model: %s" % e)
    stats = step.stats()
    if group.rank == 0 and stats:
        print("eager-SGD counters:", stats)
    step.close()
    finalize()
    return 0


class _Quiet(BaseBenchmarkLogger):
    def log_metric(self, *a, **k):
        pass


if __name__ == "__main__":
    sys.exit(main())
