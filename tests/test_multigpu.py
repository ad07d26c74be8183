"""Partial allreduce across real GPUs: one process per GPU, CUDA-IPC peer arenas.

Closed-form and oracle checks at the world size the box offers (2, 4 or 8), the
three imbalance regimes of the reference's evaluation programs (balanced,
randomly imbalanced, constantly imbalanced: fflib2 evaluation/ssgd_synch_send.c:
66-189) with assertable invariants, and failure detection without faulting a GPU
(a rank that does not join a synchronous round makes the others' bounded wait
run out with a status word).
"""
import os
import random

import pytest
import torch

from mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _world():
    return min(torch.cuda.device_count(), 8)


def _setup(rank, world):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import eagersgd_b200 as es
    torch.cuda.set_device(rank)
    return es, es.init()


def _channel(group, count, mode, limiter, average, slot_dtype=torch.float32, timeout_s=5.0, grace_us=0.0,
             fused=False):
    from eagersgd_b200.parallel.nvlink_channel import NvlinkChannel, create_arenas
    dev = group.device
    arena, bases = create_arenas(count, slot_dtype, group.rank, group.world, group.exchange)
    grad = torch.zeros(count, device=dev)
    out = torch.zeros(count, device=dev)
    ch = NvlinkChannel(count, group.rank, group.world, bases, dev, grad, slot_dtype=slot_dtype, mode=mode,
                       limiter=limiter, average=average, out=out, timeout_s=timeout_s, grace_us=grace_us)
    return arena, ch, grad, out


def _sync_closed_form(rank, world, slot_bf16):
    es, group = _setup(rank, world)
    count = 1 << 20
    arena, ch, grad, out = _channel(group, count, "sync", -1, "sum",
                                    torch.bfloat16 if slot_bf16 else torch.float32)
    ok = True
    for k in range(1, 6):
        grad.fill_(float(rank + 1 + k))
        ch.step()
        torch.cuda.synchronize()
        expect = float(sum(r + 1 + k for r in range(world)))
        ok = ok and bool(torch.all(out == expect))
    st = ch.stats()
    group.barrier()
    arena.free()
    es.finalize()
    return ok, st


@pytest.mark.parametrize("slot_bf16", [False, True])
def test_sync_closed_form(slot_bf16):
    for ok, st in run_ranks(_sync_closed_form, _world(), (slot_bf16,)):
        assert ok and st["status"] == 0 and st["participated"] == 5


def _eager_regimes(rank, world, mode):
    es, group = _setup(rank, world)
    from eagersgd_b200.parallel import _native as N
    count = 1 << 18
    arena, ch, grad, out = _channel(group, count, mode, 7, "sum")
    applied = torch.zeros(count, dtype=torch.float64, device=group.device)
    rng = random.Random(77)  # shared stream: every rank knows who is delayed
    torn = False
    steps = 0
    stream = torch.cuda.current_stream()
    for phase in ("balanced", "random", "constant"):
        for _ in range(16):
            steps += 1
            victims = {"balanced": [], "random": [rng.randrange(world)], "constant": [0]}[phase]
            if rank in victims:
                N.cuda().esgd_spin(2_000_000, stream.cuda_stream)  # 2 ms late
            grad.fill_(float((rank + 1) * 100 + steps))
            ch.step()
            torch.cuda.synchronize()
            torn = torn or not bool(torch.all(out == out[0]))
            applied += out.double()
    group.barrier()  # every round any rank opened has completed
    ch.flush()
    torch.cuda.synchronize()
    applied += out.double()
    st = ch.stats()
    total = applied[0].item()
    group.barrier()
    arena.free()
    es.finalize()
    return torn, total, st, steps


@pytest.mark.parametrize("mode", ["solo", "majority"])
def test_eager_three_regimes(mode):
    world = _world()
    res = run_ranks(_eager_regimes, world, (mode,))
    steps = res[0][3]
    published = sum((r + 1) * 100 + k for r in range(world) for k in range(1, steps + 1))
    for torn, total, st, _ in res:
        assert not torn
        assert st["status"] == 0
        assert total == res[0][1]          # replicas accumulated the same updates
        assert 0 < total <= published      # nothing duplicated
        assert st["sync_rounds"] == steps // 8


def _wrapper_sync_equals_big_batch(rank, world):
    es, group = _setup(rank, world)
    dev = group.device
    torch.manual_seed(5)
    model = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 4)).to(dev)
    ref = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 4)).to(dev)
    ref.load_state_dict(model.state_dict())
    opt = es.SyncAllreduceOptimizer(torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9), group)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)
    g = torch.Generator().manual_seed(9)
    for k in range(5):
        xs = torch.randn(world, 8, 32, generator=g).to(dev)
        ys = torch.randn(world, 8, 4, generator=g).to(dev)
        opt.zero_grad()
        torch.nn.functional.mse_loss(model(xs[rank]), ys[rank]).backward()
        opt.step()
        ropt.zero_grad()
        torch.nn.functional.mse_loss(ref(xs.view(-1, 32)), ys.view(-1, 4)).backward()
        ropt.step()
    torch.cuda.synchronize()
    err = max((a - b).abs().max().item() for a, b in zip(model.parameters(), ref.parameters()))
    st = opt.stats()
    opt.close()
    es.finalize()
    return err, st


def test_sync_wrapper_equals_large_batch_sgd():
    for err, st in run_ranks(_wrapper_sync_equals_big_batch, _world()):
        assert err < 1e-5 and st["status"] == 0


def _absent_rank(rank, world):
    es, group = _setup(rank, world)
    arena, ch, grad, out = _channel(group, 4096, "sync", -1, "sum", timeout_s=1.0)
    grad.fill_(1.0)
    ch.step()                      # first round: everyone joins
    torch.cuda.synchronize()
    ok_first = bool(torch.all(out == float(world)))
    group.barrier()
    status = 0
    if rank != world - 1:          # the last rank does not join the second round (it stays alive and idle)
        ch.step()
        torch.cuda.synchronize()
        status = ch.stats()["status"]
    alive = float((torch.ones(8, device=group.device) * 3).sum().item())
    group.barrier()
    arena.free()
    es.finalize()
    return ok_first, status, alive


def test_missing_rank_is_detected_by_bounded_wait():
    world = _world()
    res = run_ranks(_absent_rank, world)
    for r, (ok_first, status, alive) in enumerate(res):
        assert ok_first and alive == 24.0
        if r != world - 1:
            assert status != 0     # arrival or round timeout, reported instead of hanging


def _two_shot_vs_nccl(rank, world, slot_bf16):
    """Random gradients through the two-shot data phase (reduce-scatter and gather, both by peer loads)
    against NCCL's allreduce of the same tensors, plus the one-shot form of the same channel."""
    es, group = _setup(rank, world)
    import torch.distributed as dist
    from eagersgd_b200.parallel.nvlink_channel import NvlinkChannel, create_arenas
    dev = group.device
    count = (1 << 20) + 8 * 3
    sdt = torch.bfloat16 if slot_bf16 else torch.float32
    outs, arenas, stats, flags = [], [], [], []
    torch.manual_seed(100 + rank)
    grads = [torch.randn(count, device=dev) for _ in range(3)]
    if slot_bf16:
        grads = [g.to(torch.bfloat16).float() for g in grads]
    for tsm in (None, 1 << 18):
        arena, bases = create_arenas(count, sdt, group.rank, group.world, group.exchange)
        grad = torch.zeros(count, device=dev)
        out = torch.zeros(count, device=dev)
        ch = NvlinkChannel(count, group.rank, group.world, bases, dev, grad, slot_dtype=sdt, mode="sync", limiter=-1,
                           average="world", out=out, timeout_s=5.0, grace_us=0.0, two_shot_min=tsm)
        res = []
        for g in grads:
            grad.copy_(g)
            ch.step()
            torch.cuda.synchronize()
            res.append(out.clone())
        outs.append(res)
        stats.append(ch.stats()["status"])
        flags.append(ch.two_shot)
        group.barrier()
        arenas.append(arena)
    err = 0.0
    for k, g in enumerate(grads):
        ref = g.clone()
        dist.all_reduce(ref)
        ref /= world
        err = max(err, (outs[1][k] - ref).abs().max().item())
    same = all(torch.equal(a, b) for a, b in zip(outs[0], outs[1]))
    group.barrier()
    for a in arenas:
        a.free()
    es.finalize()
    return err, same, stats, flags


@pytest.mark.parametrize("slot_bf16", [False, True])
def test_two_shot_matches_nccl_and_one_shot(slot_bf16):
    for err, same, stats, flags in run_ranks(_two_shot_vs_nccl, _world(), (slot_bf16,)):
        assert flags == [0, 1]
        assert stats == [0, 0]
        assert same, "two-shot and one-shot reductions differ"
        assert err < (2e-2 if slot_bf16 else 2e-6)      # the result is rounded to the slot's element type


def _multicast_round(rank, world, slot_bf16):
    """Rounds in which every rank is on time, reduced inside the NVSwitch (multimem.ld_reduce / multimem.st on a
    multicast mapping of symmetric memory), against NCCL's allreduce of the same tensors.  No rank leaves this
    job early, so multicast stays on here."""
    os.environ.pop("NCCL_NVLS_ENABLE", None)
    os.environ["ESGD_MULTICAST"] = "1"
    import eagersgd_b200 as es
    import torch.distributed as dist
    from eagersgd_b200.parallel.nvlink_channel import NvlinkChannel, create_arenas
    torch.cuda.set_device(rank)
    group = es.init()
    dev = group.device
    count = (1 << 19) + 8 * 5
    sdt = torch.bfloat16 if slot_bf16 else torch.float32
    arena, bases = create_arenas(count, sdt, group.rank, group.world, group.exchange)
    grad = torch.zeros(count, device=dev)
    out = torch.zeros(count, device=dev)
    ch = NvlinkChannel(count, group.rank, group.world, bases, dev, grad, slot_dtype=sdt, mode="sync", limiter=-1,
                       average="world", out=out, timeout_s=5.0, mc_base=arena.mc_base, two_shot_min=1 << 16)
    torch.manual_seed(200 + rank)
    err, same = 0.0, True
    for k in range(4):
        g = torch.randn(count, device=dev)
        if slot_bf16:
            g = g.to(torch.bfloat16).float()
        grad.copy_(g)
        ch.step()
        torch.cuda.synchronize()
        ref = g.clone()
        dist.all_reduce(ref)
        ref /= world
        err = max(err, (out - ref).abs().max().item())
        lo, hi = out.clone(), out.clone()          # every rank must hold the very same bits
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        same = same and bool(torch.equal(lo, hi))
    st = ch.stats()["status"]
    used = ch.multicast
    group.barrier()
    arena.free()
    es.finalize()
    return err, same, st, used


@pytest.mark.parametrize("slot_bf16", [False, True])
def test_full_rounds_over_the_switch_match_nccl(slot_bf16):
    res = run_ranks(_multicast_round, _world(), (slot_bf16,))
    if not all(r[3] for r in res):
        pytest.skip("no NVLink multicast mapping on this machine")
    for err, same, st, used in res:
        assert st == 0 and same
        assert err < (2e-2 if slot_bf16 else 2e-6)


def _train_resnet32(rank, world, mode, accumulate, steps):
    """ResNet-32 on a learnable synthetic task (every class has a fixed random low-frequency template, an image
    is half its class template plus unit noise), one random rank per step delayed by 1.5 x the step time:
    returns the loss curve of this rank and the optimizer's counters."""
    es, group = _setup(rank, world)
    from eagersgd_b200.models.resnet import cifar_resnet
    from eagersgd_b200.train.imbalance import RandomRankFactor
    from eagersgd_b200.train.step import TrainStep
    dev = group.device
    torch.manual_seed(11)                                   # same initial replica and same teacher everywhere
    model = cifar_resnet(32, 1, 10)
    teacher = torch.randn(10, 3, 4, 4).repeat_interleave(8, 2).repeat_interleave(8, 3).to(dev)   # low-frequency templates
    step = TrainStep(model, group, mode=mode, limiter=8, bucket_mb=1.0, lr=0.1, momentum=0.9, weight_decay=1e-4,
                     accumulate=accumulate)
    g = torch.Generator(device=dev).manual_seed(1000 + rank)     # every rank sees its own data
    inj = RandomRankFactor(world, 0.005, 1.5, seed=77)
    losses = []
    for k in range(steps):
        y = torch.randint(0, 10, (128,), device=dev, generator=g)
        x = torch.randn(128, 3, 32, 32, device=dev, generator=g) + 0.5 * teacher[y]
        xb = x.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
        d = inj.delays()[rank]
        if d > 0 and mode is not None:
            step.inject_delay(d)
        losses.append(step.run_device(xb, y))
    torch.cuda.synchronize()
    curve = [float(l) for l in losses]
    st = step.stats()
    group.barrier()
    step.close()
    es.finalize()
    return curve, st


def test_eager_training_converges_like_synchronous_sgd():
    """Solo and majority eager-SGD under injected imbalance reach the loss of synchronous SGD on the same task
    (the reference's claim, README.md:4-6), no gradient is dropped when unconsumed gradients are folded into
    the next publish, and no rank falls further behind than the limiter allows."""
    world, steps = _world(), 300
    tail = lambda c: sum(c[-30:]) / 30.0
    curves, final = {}, {}
    for mode in ("sync", "solo", "majority"):
        res = run_ranks(_train_resnet32, world, (mode, mode != "sync", steps), timeout=600)
        curves[mode] = [sum(r[0][k] for r in res) / world for k in range(steps)]      # mean over ranks per step
        final[mode] = tail(curves[mode])
        for curve, st in res:
            assert st["status"] == 0
            assert st["dropped_grads"] == 0
            assert st["staleness"] <= 8 + 1
    out_dir = os.environ.get("ESGD_CURVES_DIR")
    if out_dir:
        import json
        with open(os.path.join(out_dir, "convergence_resnet32_%dgpu.json" % world), "w") as f:
            json.dump({"world": world, "steps": steps, "final": final,
                       "curves": {m: [round(v, 4) for v in c[::5]] for m, c in curves.items()}}, f)
    assert final["sync"] < 0.7 * curves["sync"][0], final            # the task is learnable and was learnt
    for mode in ("solo", "majority"):
        assert final[mode] <= 1.10 * final["sync"] + 0.02, final


def _peer_collectives(rank, world):
    """Every classic collective on this package's kernels, against closed forms; then the same calls through
    the Group API with the native path switched on."""
    os.environ["ESGD_NATIVE_COLLECTIVES"] = "1"
    es, group = _setup(rank, world)
    dev = group.device
    pc = group.peer_collectives(stage_mb=1.0)
    n = 300_001                                    # odd byte counts and more than one stage of 1 MiB (fp32: 1.2 MB)
    res = {}
    t = torch.full((n,), float(rank), device=dev) + torch.arange(n, device=dev) % 7
    ref = (torch.arange(n, device=dev) % 7).float()
    # broadcast from the last rank
    b = t.clone()
    pc.bcast(b, world - 1)
    res["bcast"] = bool(torch.equal(b, ref + (world - 1)))
    # all-gather and gather (uint8 payload of odd length)
    u = (torch.arange(1001, device=dev) % 251).to(torch.uint8) + rank
    ag = pc.allgather(u)
    res["allgather"] = all(bool(torch.equal(ag[j], (torch.arange(1001, device=dev) % 251).to(torch.uint8) + j))
                           for j in range(world))
    g = pc.gather(t, 1 % world)
    res["gather"] = (g is None) if rank != 1 % world else all(bool(torch.equal(g[j], ref + j)) for j in range(world))
    # all-reduce: bits equal on every rank and equal to the rank-ordered fp32 sum
    a = (torch.randn(1 << 18, device=dev, generator=torch.Generator(dev).manual_seed(rank)))
    parts = pc.allgather(a)
    expect = torch.zeros_like(a)
    for j in range(world):
        expect += parts[j]
    s = a.clone()
    pc.allreduce(s)
    res["allreduce_f32"] = bool(torch.equal(s, expect))
    h = a.to(torch.bfloat16)
    hp = pc.allgather(h)
    eh = torch.zeros_like(a)
    for j in range(world):
        eh += hp[j].float()
    pc.allreduce(h)
    res["allreduce_bf16"] = bool(torch.equal(h, eh.to(torch.bfloat16)))
    # ring of sends: rank r sends to r+1, receives from r-1 (even ranks send first)
    x = torch.full((4097,), float(rank), device=dev)
    y = torch.empty_like(x)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    pc.send(x, nxt)                                # a send returns once the stage holds the data: no deadlock
    pc.recv(y, prv)
    res["sendrecv"] = bool(torch.all(y == float(prv)))
    # whichever rank sends first: all send one word to rank 0
    if rank == 0:
        seen = sorted(int(pc.recv_any(y[:4]) ) for _ in range(world - 1))
        res["recv_any"] = seen == list(range(1, world))
    else:
        pc.send(x[:4], 0)
        res["recv_any"] = True
    # ring-neighbour sum
    z = torch.full((1024,), float(rank + 1), device=dev)
    pc.reduce_from_neighbours(z)
    res["neighbours"] = bool(torch.all(z == float(rank + 1 + prv + 1 + nxt + 1)))
    pc.barrier()
    pc.check()
    # the Group API on the native path
    w = torch.full((64,), float(rank), device=dev)
    group.bcast(w, 0)
    v = torch.ones(64, device=dev)
    group.allreduce(v)
    res["group_api"] = bool(torch.all(w == 0)) and bool(torch.all(v == world))
    torch.cuda.synchronize()
    import eagersgd_b200.parallel._native as N
    res["launches"] = N.launch_count() > 20
    group.barrier()
    es.finalize()
    return res


def test_classic_collectives_on_peer_memory():
    world = _world()
    if world < 2:
        pytest.skip("needs 2 GPUs")
    for r, res in enumerate(run_ranks(_peer_collectives, world, timeout=240)):
        assert all(res.values()), (r, res)


def _partial_allreduce_object(rank, world):
    """The stand-alone collective object across GPUs: synchronous closed form, then solo with a late rank."""
    es, group = _setup(rank, world)
    dev = group.device
    t = torch.zeros(1 << 16, device=dev)
    ok = True
    with es.PartialAllreduce(t, group, mode="sync", average="sum") as ar:
        for k in range(1, 4):
            t.fill_(float(rank + k))
            ar.post()
            info = ar.wait()
            ok = ok and bool(torch.all(t == float(sum(r + k for r in range(world))))) and info["contributors"] == world
    x = torch.ones(1000, device=dev, dtype=torch.bfloat16) * (rank + 1)     # not a multiple of eight: padded inside
    out = torch.zeros(1000, device=dev, dtype=torch.bfloat16)
    with es.PartialAllreduce(x, group, mode="solo", limiter=3, average="world", out=out, timeout_s=10.0) as solo:
        for k in range(8):
            if rank == world - 1:
                torch.cuda._sleep(20_000_000)               # this rank's stream is late every step
            solo.post()
            solo.wait()
        st = solo.flush()
    ok = ok and st["status"] == 0 and st["steps"] == 8 and st["forced_sync"] >= 1 and bool(torch.isfinite(out.float()).all())
    es.finalize()
    return ok, st


def test_partial_allreduce_object_across_gpus():
    world = _world()
    if world < 2:
        pytest.skip("needs 2 GPUs")
    for ok, st in run_ranks(_partial_allreduce_object, world, timeout=240):
        assert ok, st
