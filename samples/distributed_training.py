"""Hyperplane regression with a selectable distributed scheme.

    torchrun --nproc-per-node 4 samples/distributed_training.py --scheme solo --sleep-ms 50

Schemes: local, solo, majority, sync (partial allreduce), dsgd (allreduce of gradients), pssgd
(parameter server), mavg (model averaging), dpsgd (ring neighbours), hvd (fused allreduce) — the
selector of the reference sample (deep500 samples/distributed_training.py:54-70) plus the eager modes.
Each step one seeded-random rank sleeps, which is the load imbalance eager-SGD tolerates.
"""
import argparse
import os
import random
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import eagersgd_b200 as es  # noqa: E402
from eagersgd_b200.models.hyperplane import HyperplaneData, HyperplaneRegressor  # noqa: E402
from eagersgd_b200.optim import base, distributed as D  # noqa: E402
from eagersgd_b200.train.executor import GraphExecutor, mse_loss  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--scheme", default="solo")
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--dim", type=int, default=4096)
    ap.add_argument("--sleep-ms", type=float, default=50.0)
    args = ap.parse_args()
    group = es.init(backend="gloo")
    torch.manual_seed(0)
    model = HyperplaneRegressor(args.dim)
    data = HyperplaneData(args.dim, noise_std=0.1, seed=3, rank=group.rank)
    sleeper = random.Random(1234)
    t0 = time.time()
    if args.scheme in ("solo", "majority", "sync", "local"):
        inner = torch.optim.SGD(model.parameters(), lr=0.01)
        opt = {"solo": es.SoloAllreduceOptimizer, "majority": es.MajorityAllreduceOptimizer,
               "sync": es.SyncAllreduceOptimizer}.get(args.scheme, lambda o, g: o)(inner, group)
        for _ in range(args.steps):
            if sleeper.randrange(group.world) == group.rank:
                time.sleep(args.sleep_ms / 1e3)
            x, y = data.batch(64)
            opt.zero_grad()
            torch.nn.functional.mse_loss(model(x), y).backward()
            opt.step()
        if hasattr(opt, "flush"):
            opt.flush()
    else:
        ex = GraphExecutor(model, lambda o, b: mse_loss(o, b))
        cls = {"dsgd": D.ConsistentDecentralized, "pssgd": D.ConsistentParameterServer, "mavg": D.ModelAverageDecentralized,
               "dpsgd": D.ConsistentNeighbors, "hvd": D.HorovodStyleOptimizer}[args.scheme]
        opt = cls(base.GradientDescent(ex, learning_rate=0.01), group)
        for _ in range(args.steps):
            if sleeper.randrange(group.world) == group.rank:
                time.sleep(args.sleep_ms / 1e3)
            x, y = data.batch(64)
            opt.step({"x": x, "y": y})
    group.barrier()
    err = (model.linear.weight.detach().view(-1) - data.w_star).norm() / data.w_star.norm()
    if hasattr(opt, "close"):
        opt.close()
    if group.rank == 0:
        print("scheme %s: %d steps in %.2f s (%.1f steps/s), relative error %.4f"
              % (args.scheme, args.steps, time.time() - t0, args.steps / (time.time() - t0), err))
    es.finalize()


if __name__ == "__main__":
    main()
