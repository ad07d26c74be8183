"""Minimum end-to-end slice on CPU: hyperplane regression, 4 gloo ranks, one
random rank sleeping per step, solo / majority / sync wrappers around torch SGD."""
import random
import time

import pytest
import torch

from mp_util import run_ranks


def _train(rank, world, mode, steps, dim, sleep_s):
    import eagersgd_b200 as es
    from eagersgd_b200.models.hyperplane import HyperplaneData, HyperplaneRegressor

    group = es.init(backend="gloo")
    torch.manual_seed(0)  # identical initial replicas via a shared seed, as in the reference
    model = HyperplaneRegressor(dim)
    data = HyperplaneData(dim, noise_std=0.1, seed=3, rank=rank)
    inner = torch.optim.SGD(model.parameters(), lr=0.01)
    cls = {"solo": es.SoloAllreduceOptimizer, "majority": es.MajorityAllreduceOptimizer,
           "sync": es.SyncAllreduceOptimizer}[mode]
    opt = cls(inner, group, limiter=8) if mode == "solo" else cls(inner, group)
    sleeper = random.Random(1234)  # same stream on all ranks: they agree on who sleeps
    t0 = time.time()
    for k in range(steps):
        if sleeper.randrange(world) == rank:
            time.sleep(sleep_s)
        x, y = data.batch(64)
        opt.zero_grad()
        loss = torch.nn.functional.mse_loss(model(x), y)
        loss.backward()
        opt.step()
    elapsed = time.time() - t0
    opt.flush()
    group.barrier()
    err = (model.linear.weight.detach().view(-1) - data.w_star).norm().item() / data.w_star.norm().item()
    st = opt.stats()
    opt.close()
    es.finalize()
    return err, elapsed, st, model.linear.weight.detach().view(-1)[:8].tolist()


@pytest.mark.parametrize("mode", ["sync", "solo", "majority"])
def test_hyperplane_converges(mode):
    res = run_ranks(_train, 4, (mode, 150, 256, 0.005))
    for err, _, st, _ in res:
        assert err < 0.2, (mode, err)
        assert st["status"] == 0
    if mode == "sync":
        for r in res[1:]:
            assert r[3] == pytest.approx(res[0][3], rel=1e-5)


def test_solo_faster_than_sync_under_imbalance():
    sync = run_ranks(_train, 4, ("sync", 40, 256, 0.03))
    solo = run_ranks(_train, 4, ("solo", 40, 256, 0.03))
    t_sync = max(r[1] for r in sync)
    t_solo = max(r[1] for r in solo)
    assert t_solo < t_sync, (t_solo, t_sync)
