#!/usr/bin/env python
"""Headline benchmark: ResNet-50 v1.5 training throughput (images/s) under seeded,
injected load imbalance, bf16 compute with fp32 master weights, batch 256 per GPU,
solo-allreduce eager-SGD with ~25 MB gradient buckets.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 20 --warmup 5

Rank 0 prints one JSON line.  After the headline run the same process measures, on the same GPUs and with
the same seeded delays, this framework without imbalance, its own synchronous mode and a plain PyTorch
DistributedDataParallel / NCCL step (``same_box`` in the JSON line; ``--no-baselines`` skips them), and
reports the delay it injected per step, so that a reader can split step time into compute, injected delay
and collective.  ``--impl ddp`` makes the PyTorch arm the headline; ``--impl reference`` reports whether the
unmodified reference can run here and runs the part of it that can (its communication library).
"""
from __future__ import annotations

import argparse
import json
import os
import random
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "ddp"])
    ap.add_argument("--mode", default=None, choices=["solo", "majority", "sync"],
                    help="default: solo for resnet50, majority for resnet32 and lstm")
    ap.add_argument("--model", default="resnet50", choices=["resnet50", "resnet32", "lstm"])
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch (default: 256 / 128)")
    ap.add_argument("--limiter", type=int, default=32)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--imbalance", default="auto", choices=["auto", "none"],
                    help="auto (N > 1): resnet50: 2 random ranks/step delayed by Exp(0.5 x step time); resnet32: one "
                         "random rank delayed by 1.5 x step time; lstm: none injected (sequence lengths differ per rank)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--max-frames", type=int, default=1800, help="lstm: longest sequence kept by the sampler")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of one CUDA graph")
    ap.add_argument("--no-baselines", action="store_true",
                    help="skip the comparison arms measured after the headline run on the same GPUs (same model, same "
                         "injected delays): this framework without imbalance, its synchronous mode, and PyTorch DDP / NCCL")
    ap.add_argument("--baseline-steps", type=int, default=None, help="timed steps of each comparison arm (default: --steps)")
    ap.add_argument("--accumulate", action="store_true",
                    help="fold gradients that no round picked up into the next publish instead of dropping them")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                for n, v in zip(names, r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def reference_arm(args):
    """The reference's training path is TensorFlow 1.x + Horovod + mpi4py + an MPI library (the custom op
    links tensorflow_framework; its vendored Deep500 package installs but cannot be imported), so the
    headline metric has no reference value on this machine.  What of the reference does run here is its
    communication library: fflib2, built unmodified against a shared-memory MPI subset, driven by its own
    SGD-loop timing programs (evaluation/ssgd.c, rsgd.c, randomsgd.c).  Their figures ride along in
    ``fflib2_sgd_loops``; ``python -m eagersgd_b200.parallel.bench_allreduce`` is this framework's
    counterpart of those loops."""
    if int(os.environ.get("RANK", "0")) != 0:
        return 0
    missing = []
    for mod in ("tensorflow", "horovod", "mpi4py", "onnx"):
        try:
            __import__(mod)
        except Exception:
            missing.append(mod)
    why = ("reference training path cannot run here: missing " + ", ".join(missing or ["the Piz Daint SLURM setup"]) +
           "; the repository root is not an installable project and its vendored deep500 package fails at import; "
           "no network")
    out = {"impl": "reference", "unavailable": why}
    try:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import run_reference
        ranks = sorted({2, max(2, min(args.gpus, 8))})
        out["fflib2_sgd_loops"] = run_reference.run(ranks=ranks, counts=(1024, 262144, 6553600), iters=12)
    except Exception as e:  # noqa
        out["fflib2_sgd_loops"] = {"unavailable": repr(e)[:200]}
    print(json.dumps(out))
    return 0


def build_model(args, impl, classes):
    """The model of the named config: this framework's modules, or plain torch.nn ones for the DDP arm."""
    if impl == "ddp":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import torch_resnet as T
        if args.model == "resnet50":
            return T.TorchResNet50(classes)
        if args.model == "resnet32":
            return T.TorchResNetCifar(32, classes)
        return T.TorchLSTMClassifier(2048, 2048, 2, classes)
    from eagersgd_b200.models.lstm import LSTMClassifier
    from eagersgd_b200.models.resnet import cifar_resnet, imagenet_resnet
    if args.model == "resnet50":
        return imagenet_resnet(50, 1, classes)
    if args.model == "resnet32":
        return cifar_resnet(32, 1, classes)
    return LSTMClassifier(2048, 2048, 2, classes)


def make_batches(args, rank, n_steps):
    """Synthetic data of the named shape in pinned host memory."""
    import torch
    g = torch.Generator().manual_seed(100 + rank)
    host = []
    if args.model in ("resnet50", "resnet32"):
        batch, res, classes = (args.batch or 256, 224, 1000) if args.model == "resnet50" else (args.batch or 128, 32, 10)
        for _ in range(3):
            x = torch.randn(batch, 3, res, res, generator=g).to(torch.bfloat16)
            x = x.contiguous(memory_format=torch.channels_last).pin_memory()
            host.append((x, torch.randint(0, classes, (batch,), generator=g).pin_memory()))
        return host, batch, classes, {"image": [res, res, 3], "classes": classes, "seq_len": None}
    # 2-layer LSTM (hidden 2048) on 2048-d frame features; per-sample length from a clipped log-normal over
    # 30..1800 frames, length-bucketed batches, left-padded: the per-rank sequence length IS the imbalance
    from eagersgd_b200.data import BucketSampler, SyntheticSequenceDataset
    batch, classes = args.batch or 16, 101
    ds = SyntheticSequenceDataset(2048, 8, classes, seed=7 + rank)      # lengths / labels only; features below
    sampler = BucketSampler(ds, batch, ds.lengths, num_buckets=30, max_length=args.max_frames, seed=rank)
    lengths = []
    for _ in range(n_steps):
        b = sampler()
        if b is None:
            sampler.reset()
            b = sampler()
        lengths.append(int(b["x"].shape[1]))
        x = torch.randn(batch, lengths[-1], 2048, generator=g).to(torch.bfloat16).pin_memory()
        host.append((x, torch.as_tensor(b["y"]).pin_memory()))
    return host, batch, classes, {"feature_dim": 2048, "classes": classes,
                                  "seq_len": "log-normal 30..%d, this rank: min %d max %d"
                                  % (args.max_frames, min(lengths), max(lengths))}


def run_arm(args, group, host_batches, batch, classes, impl, mode, inject, steps, with_e2e, base_step_s=None):
    """Build one training arm, warm it up, time ``steps`` steps on the device (and, with ``with_e2e``, end to
    end from pinned host memory), tear it down.  Returns a dict of what was measured."""
    import torch
    import torch.distributed as dist
    from eagersgd_b200.parallel import _native as N
    rank, world, dev = group.rank, group.world, group.device
    torch.manual_seed(1234)  # identical replicas through a shared seed
    model = build_model(args, impl, classes)
    if impl == "ddp":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        from ddp_step import DDPStep
        step = DDPStep(model, group, bucket_mb=args.bucket_mb, lr=0.01, momentum=0.9, weight_decay=1e-4,
                       channels_last=args.model != "lstm")
    else:
        from eagersgd_b200.train.step import TrainStep
        step = TrainStep(model, group, impl="ours", mode=mode, limiter=args.limiter, bucket_mb=args.bucket_mb,
                         lr=0.01, momentum=0.9, weight_decay=1e-4, accumulate=args.accumulate)
    nb = len(host_batches)
    dev_batches = [(x.to(dev, non_blocking=True), y.to(dev, non_blocking=True)) for x, y in host_batches]
    torch.cuda.synchronize()

    def sync_all():
        torch.cuda.synchronize()
        group.barrier()
        torch.cuda.synchronize()

    use_graph = not args.no_graph and args.model != "lstm"   # the sequence length varies from step to step
    if use_graph:
        step.capture(*dev_batches[0])
    warm = max(args.warmup, 3)
    # ---- warm-up (untimed); its last two steps give the undisturbed step time ----
    t_w = None
    for i in range(warm):
        if i == warm - 2:
            sync_all()
            t_w = time.perf_counter()
        step.run_device(*dev_batches[i % nb])
    torch.cuda.synchronize()
    own = torch.tensor([(time.perf_counter() - t_w) / 2.0], device=dev)
    if world > 1:
        dist.all_reduce(own, op=dist.ReduceOp.MAX)
    if base_step_s is None:
        base_step_s = float(own.item())      # every arm injects delays scaled by the headline arm's step time
    delay_rng = random.Random(4242)          # same stream on every rank and in every arm
    injected = []

    def delay_for_step():
        if not inject:
            return 0.0
        if args.model == "resnet32":         # one random rank is delayed by 1.5 x its step time
            return 1.5 * base_step_s if delay_rng.randrange(world) == rank else 0.0
        d = 0.0                              # two random ranks, each delayed by Exp(mean 0.5 x step time)
        for victim in (delay_rng.randrange(world), delay_rng.randrange(world)):
            e = delay_rng.expovariate(1.0 / (0.5 * base_step_s))
            if victim == rank:
                d += e
        return min(d, 5.0 * base_step_s)

    def timed(fn, batches, stream_api=False):
        delay_rng.seed(4242)                 # the device-timed and the end-to-end loop see the same delays
        sampler = ClockSampler(dev.index)
        launches0 = N.launch_count()
        sync_all()
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        last, total_delay = None, 0.0
        if stream_api:
            # the public end-to-end loop: pinned host batches in, one python float per step out; it overlaps the
            # next batch's host-to-device copy and the previous loss's read-back with the running step
            def before(i):
                nonlocal total_delay
                d = delay_for_step()
                if d > 0:
                    step.inject_delay(d)
                    total_delay += d
            for last in fn((batches[(warm + i) % nb] for i in range(steps)), before_step=before):
                pass
        else:
            for i in range(steps):
                d = delay_for_step()
                if d > 0:
                    step.inject_delay(d)
                    total_delay += d
                last = fn(*batches[(warm + i) % nb])
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        group.barrier()
        clocks = sampler.stop()
        dl = torch.tensor([total_delay * 1e3 / steps], device=dev)      # ms per step injected on this rank
        dmax, dsum = dl.clone(), dl.clone()
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dist.all_reduce(dmax, op=dist.ReduceOp.MAX)
            dist.all_reduce(dsum)
        injected.append({"max_over_ranks": float(dmax.item()), "mean_over_ranks": float(dsum.item()) / world})
        launched = N.launch_count() - launches0 + steps * getattr(step, "graph_kernel_launches", 0)
        return float(ms.item()), clocks, launched, last

    ms_dev, clocks, launches, _ = timed(step.run_device, dev_batches)
    out = {"impl": impl, "mode": mode if impl == "ours" else "nccl-allreduce", "value": world * batch * steps / (ms_dev / 1e3),
           "ms_per_step": ms_dev / steps, "steps": steps, "cuda_graph": bool(use_graph and (impl == "ours" or world == 1)),
           "undisturbed_ms_per_step": float(own.item()) * 1e3, "base_step_s": base_step_s,
           "injected_ms_per_step": injected[0], "clocks": clocks, "gpu_launches": launches, "e2e": None}
    if with_e2e:
        ms_e2e, _, _, last_loss = timed(step.run_host_stream, host_batches, stream_api=True)
        out["e2e"] = {"value": world * batch * steps / (ms_e2e / 1e3), "ms_per_step": ms_e2e / steps,
                      "h2d_bytes_per_step": int(sum(x.numel() * 2 + y.numel() * 8 for x, y in host_batches) / nb),
                      "d2h_bytes_per_step": 4, "last_loss": last_loss, "injected_ms_per_step": injected[1]}
    out["eager_stats"] = step.stats()
    step.close()
    del step, model, dev_batches
    torch.cuda.empty_cache()
    return out


def main():
    args = parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import torch

    import eagersgd_b200 as es

    # NCCL announces its version on stdout at the first collective: keep stdout for the one JSON line
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    group = es.init()
    group.barrier()
    rank, world = group.rank, group.world
    assert world == args.gpus, "launch with torchrun --nproc-per-node %d (WORLD_SIZE=%d)" % (args.gpus, world)
    torch.backends.cudnn.benchmark = True
    if args.mode is None:
        args.mode = "solo" if args.model == "resnet50" else "majority"
    unit = "sequences/s" if args.model == "lstm" else "images/s"
    name = {"resnet50": "ResNet-50 v1.5", "resnet32": "ResNet-32 (CIFAR)",
            "lstm": "2-layer LSTM classifier (hidden 2048)"}[args.model]
    bsteps = args.baseline_steps or args.steps
    host_batches, batch, classes, shape_cfg = make_batches(args, rank, max(args.steps, bsteps) + max(args.warmup, 3))
    inject = args.imbalance == "auto" and world > 1 and args.model != "lstm"

    head = run_arm(args, group, host_batches, batch, classes, args.impl, args.mode, inject, args.steps, not args.no_e2e)
    same_box = None
    if not args.no_baselines:
        # comparison arms on the same GPUs, same data, same seeded delays (scaled by the headline arm's step time)
        same_box = {}
        arms = []
        if inject:
            arms.append(("no_imbalance", args.impl, args.mode, False))
        if args.impl == "ours":
            if world > 1 and args.mode != "sync":
                arms.append(("sync_ours", "ours", "sync", inject))
            arms.append(("ddp_nccl", "ddp", None, inject))
        for key, impl, mode, inj in arms:
            try:
                r = run_arm(args, group, host_batches, batch, classes, impl, mode, inj, bsteps, False, head["base_step_s"])
                same_box[key] = {k: r[k] for k in ("value", "ms_per_step", "steps", "cuda_graph", "injected_ms_per_step",
                                                   "undisturbed_ms_per_step")}
                same_box[key]["headline_over_this"] = head["value"] / r["value"]
            except Exception as e:  # noqa
                same_box[key] = {"error": repr(e)[:300]}
    sys.stdout.flush()
    os.dup2(saved_stdout, 1)
    os.close(saved_stdout)

    if rank == 0:
        e2e = head["e2e"]
        if e2e is not None:
            e2e = dict(e2e, unit=unit)
        out = {
            "metric": "train_%s_per_sec_under_%s_imbalance" % (unit.split("/")[0],
                                                                "natural" if args.model == "lstm" else "injected"),
            "impl": args.impl,
            "value": head["value"], "unit": unit, "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": head["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic N(0,1) inputs, uniform labels, random-init weights",
            "config": {"model": name, "global_batch": batch * world, "per_gpu_batch": batch, **shape_cfg,
                       "parallelism": "dp%d" % world,
                       "collective": args.mode + "-allreduce" if args.impl == "ours" else "nccl-allreduce",
                       "bucket_mb": args.bucket_mb, "limiter": args.limiter, "cuda_graph": head["cuda_graph"],
                       "optimizer": "momentum SGD 0.9, wd 1e-4, fp32 master weights",
                       "imbalance": (("one random rank/step delayed by 1.5 x %.1f ms" if args.model == "resnet32" else
                                      "2 random ranks/step delayed by Exp(mean 0.5 x %.1f ms)")
                                     % (head["base_step_s"] * 1e3))
                       if inject else "natural (per-rank sequence lengths)" if args.model == "lstm"
                       else "none (single rank)" if world == 1 else "none",
                       "l2": "per-step working set (activations + 51 MB gradients) exceeds the 126 MB L2"},
            "clocks": head["clocks"], "e2e": e2e, "gpu_launches": head["gpu_launches"],
            "undisturbed_ms_per_step": head["undisturbed_ms_per_step"],
            "injected_ms_per_step": head["injected_ms_per_step"],
            "same_box": same_box, "eager_stats": head["eager_stats"],
        }
        print(json.dumps(out))
    es.finalize()
    return 0


if __name__ == "__main__":
    sys.exit(main())
