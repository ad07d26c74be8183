"""NVLink partial-allreduce kernels on one GPU.

Multi-rank behaviour is exercised by ``EmulatedWorld``: all ranks of a channel
live on one device and are stepped by a single cooperative launch (one block per
rank), because separate launches that wait on one another are not guaranteed to
run concurrently on one GPU.  Oracles: closed-form sums (fflib2
evaluation/allreduce.c:34-38) and a plain PyTorch fp32 momentum SGD.
"""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("slot_dtype", [torch.float32, torch.bfloat16])
def test_sync_closed_form(world, slot_dtype):
    from eagersgd_b200.parallel.nvlink_channel import EmulatedWorld
    count = 4096 + 64
    w = EmulatedWorld(world, count, _dev(), slot_dtype=slot_dtype, mode="sync", limiter=-1, average="sum",
                      timeout_s=2.0)
    try:
        for k in range(1, 6):
            for r in range(world):
                w.grads[r].fill_(float(r + 1 + k))
            w.step()
            torch.cuda.synchronize()
            expect = float(sum(r + 1 + k for r in range(world)))
            for r in range(world):
                assert torch.all(w.outs[r] == expect), (world, k, r, w.outs[r][:4])
        for c in w.channels:
            st = c.stats()
            assert st["status"] == 0 and st["participated"] == 5 and st["local_step"] == 5
    finally:
        w.close()


@pytest.mark.parametrize("mode", ["solo", "majority"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_eager_modes_replicas_agree(mode, world):
    """Random late arrivals: results are never torn and all ranks accumulate the same total."""
    from eagersgd_b200.parallel.nvlink_channel import EmulatedWorld
    count = 2048
    w = EmulatedWorld(world, count, _dev(), slot_dtype=torch.float32, mode=mode, limiter=5, average="sum",
                      timeout_s=2.0, grace_us=0.0)
    rng = random.Random(world * 7 + len(mode))
    applied = [torch.zeros(count, dtype=torch.float64, device=_dev()) for _ in range(world)]
    try:
        steps = 30
        for k in range(1, steps + 1):
            for r in range(world):
                w.grads[r].fill_(float((r + 1) * 100 + k))
            delays = [rng.choice([0, 0, 20, 200]) for _ in range(world)]
            w.step(delays_us=delays)
            torch.cuda.synchronize()
            for r in range(world):
                o = w.outs[r]
                assert torch.all(o == o[0]), "torn result"
                applied[r] += o.double()
        w.step(flush=True)
        torch.cuda.synchronize()
        for r in range(world):
            applied[r] += w.outs[r].double()
        for r in range(1, world):
            assert torch.equal(applied[r], applied[0])
        published = sum((r + 1) * 100 + k for r in range(world) for k in range(1, steps + 1))
        assert 0 < applied[0][0].item() <= published
        sts = [c.stats() for c in w.channels]
        assert all(s["status"] == 0 for s in sts)
        assert all(s["sync_rounds"] == steps // 6 for s in sts)
    finally:
        w.close()


def test_contributor_average_and_stale_flag():
    from eagersgd_b200.parallel.nvlink_channel import EmulatedWorld
    world, count = 4, 1024
    w = EmulatedWorld(world, count, _dev(), slot_dtype=torch.float32, mode="sync", limiter=-1,
                      average="contributors", timeout_s=2.0)
    try:
        for r in range(world):
            w.grads[r].fill_(float(r + 1))
        w.step()
        torch.cuda.synchronize()
        for r in range(world):
            assert torch.allclose(w.outs[r], torch.full_like(w.outs[r], 2.5))
    finally:
        w.close()


@pytest.mark.parametrize("param_dtype", [torch.float32, torch.bfloat16])
def test_fused_momentum_sgd_matches_torch(param_dtype):
    """world=1 channel with the fused update vs torch.optim.SGD on fp32 master weights."""
    from eagersgd_b200.parallel.nvlink_channel import NvlinkChannel, create_arenas, HYPER_LEN
    dev = _dev()
    count = 8192
    torch.manual_seed(0)
    w0 = torch.randn(count, device=dev)
    slot_dtype = param_dtype
    arena, bases = create_arenas(count, slot_dtype, 0, 1)
    grad = torch.zeros(count, dtype=param_dtype, device=dev)
    w32, mom = w0.clone(), torch.zeros(count, device=dev)
    w16 = w0.to(torch.bfloat16) if param_dtype == torch.bfloat16 else None
    hyper = torch.tensor([0.1, 0.9, 1e-2, 0.0, 1.0, 0, 0, 0], dtype=torch.float32, device=dev)
    ch = NvlinkChannel(count, 0, 1, bases, dev, grad, slot_dtype=slot_dtype, mode="solo", limiter=3, w32=w32,
                       mom=mom, w16=w16, hyper=hyper, timeout_s=2.0)
    ref = torch.nn.Parameter(w0.clone())
    opt = torch.optim.SGD([ref], lr=0.1, momentum=0.9, weight_decay=1e-2)
    for k in range(5):
        g = torch.randn(count, device=dev)
        grad.copy_(g)
        ref.grad = grad.float().clone()
        opt.step()
        ch.step()
        torch.cuda.synchronize()
        assert torch.allclose(w32, ref.detach(), rtol=1e-5, atol=1e-6), k
        if w16 is not None:
            assert torch.equal(w16, w32.to(torch.bfloat16))
    assert ch.stats()["status"] == 0
    arena.free()


def test_bounded_wait_reports_status_and_context_survives():
    """A synchronous round whose second rank never publishes: the kernel's wait runs
    out after ~0.3 s, the status word says so, and the CUDA context stays usable."""
    from eagersgd_b200.parallel.nvlink_channel import Arena, ArenaLayout, NvlinkChannel
    dev = _dev()
    count = 1024
    layout = ArenaLayout(count, torch.float32)
    arenas = [Arena(layout.total, export=False) for _ in range(2)]
    grad = torch.ones(count, device=dev)
    out = torch.zeros(count, device=dev)
    ch = NvlinkChannel(count, 0, 2, [a.base for a in arenas], dev, grad, slot_dtype=torch.float32, mode="sync",
                       limiter=-1, out=out, timeout_s=0.3)
    ch.step()
    torch.cuda.synchronize()
    st = ch.stats()
    assert st["status"] & 3, st     # the round never opened, or it opened and a rank never arrived
    assert torch.all(out == 0)
    from eagersgd_b200.parallel import ChannelError
    with pytest.raises(ChannelError):
        ch.check()
    assert (torch.ones(4, device=dev) * 2).sum().item() == 8.0
    for a in arenas:
        a.free()


def test_optimizer_wrapper_fused_matches_sgd():
    import eagersgd_b200 as es
    dev = _dev()
    torch.manual_seed(1)
    mk = lambda: torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.ReLU(), torch.nn.Linear(128, 10)).to(dev)
    m1, m2 = mk(), mk()
    m2.load_state_dict(m1.state_dict())
    o1 = torch.optim.SGD(m1.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4)
    o2 = es.SoloAllreduceOptimizer(torch.optim.SGD(m2.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-4),
                                   es.Group(), limiter=2, bucket_mb=0.02)
    assert o2.fused and len(o2.buckets) > 1
    for k in range(6):
        x = torch.randn(32, 64, device=dev)
        y = torch.randint(0, 10, (32,), device=dev)
        for m, o in ((m1, o1), (m2, o2)):
            o.zero_grad()
            torch.nn.functional.cross_entropy(m(x), y).backward()
            o.step()
    torch.cuda.synchronize()
    for p1, p2 in zip(m1.parameters(), m2.parameters()):
        assert torch.allclose(p1, p2, rtol=1e-4, atol=1e-5)
    assert o2.stats()["status"] == 0
    o2.close()


def test_optimizer_wrapper_generic_inner_optimizer():
    """Any torch optimizer can be wrapped: the averaged gradient lands in .grad (Adam here)."""
    import eagersgd_b200 as es
    dev = _dev()
    torch.manual_seed(2)
    m1 = torch.nn.Linear(32, 8).to(dev)
    m2 = torch.nn.Linear(32, 8).to(dev)
    m2.load_state_dict(m1.state_dict())
    o1 = torch.optim.Adam(m1.parameters(), lr=1e-2)
    o2 = es.MajorityAllreduceOptimizer(torch.optim.Adam(m2.parameters(), lr=1e-2), es.Group())
    assert not o2.fused
    for k in range(4):
        x = torch.randn(16, 32, device=dev)
        for m, o in ((m1, o1), (m2, o2)):
            o.zero_grad()
            m(x).square().mean().backward()
            o.step()
    for p1, p2 in zip(m1.parameters(), m2.parameters()):
        assert torch.allclose(p1, p2, rtol=1e-5, atol=1e-6)
    o2.close()


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("slot_dtype,fused", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
def test_two_shot_reduction_is_bit_identical_to_one_shot(world, slot_dtype, fused):
    """Reduce-scatter + pull-gather (both by peer loads) gives the very bits of the one-shot reduction:
    averaged gradients, and fp32 master weights / momentum / bf16 weights after fused updates.  The value
    a round hands out is rounded to the slot's element type in both forms."""
    from eagersgd_b200.parallel.nvlink_channel import EmulatedWorld
    count = 8 * 1237          # not a multiple of the number of participants
    gdt = torch.bfloat16 if slot_dtype == torch.bfloat16 else torch.float32
    worlds = [EmulatedWorld(world, count, _dev(), slot_dtype=slot_dtype, grad_dtype=gdt, fused=fused, mode="sync",
                            limiter=-1, average="contributors", timeout_s=2.0, two_shot_min=tsm)
              for tsm in (None, 0)]
    try:
        torch.manual_seed(world)
        for w in worlds:
            w.hyper[:5] = torch.tensor([0.1, 0.9, 1e-4, 0.0, 1.0])
            if fused:
                for r in range(world):
                    w.w32[r].copy_(torch.linspace(-1, 1, count))
        for k in range(4):
            gs = [torch.randn(count, device=_dev()).to(gdt) for _ in range(world)]
            for w in worlds:
                for r in range(world):
                    w.grads[r].copy_(gs[r])
                w.step()
            torch.cuda.synchronize()
            a, b = worlds
            for r in range(world):
                if fused:
                    assert torch.equal(a.w32[r], b.w32[r]) and torch.equal(a.mom[r], b.mom[r])
                    assert torch.equal(a.w16[r], b.w16[r]) and torch.equal(b.w32[r], b.w32[0])
                else:
                    assert torch.equal(a.outs[r], b.outs[r]), (k, r)
                    ref = torch.stack([g.float() for g in gs]).sum(0) / world
                    tol = dict(rtol=1e-5, atol=1e-6) if slot_dtype == torch.float32 else dict(rtol=8e-3, atol=1e-3)
                    assert torch.allclose(b.outs[r], ref, **tol)
        for w in worlds:
            assert all(c.stats()["status"] == 0 for c in w.channels)
    finally:
        for w in worlds:
            w.close()


@pytest.mark.parametrize("mode", ["solo", "majority"])
def test_two_shot_eager_rounds_replicas_agree(mode):
    """Two-shot data phase under random late arrivals: participants change from round to round, absent ranks
    collect their mailbox, and every rank ends with the same accumulated total."""
    from eagersgd_b200.parallel.nvlink_channel import EmulatedWorld
    world, count, steps = 6, 8 * 511, 40
    w = EmulatedWorld(world, count, _dev(), slot_dtype=torch.float32, mode=mode, limiter=7, average="sum",
                      timeout_s=2.0, grace_us=0.0, two_shot_min=0)
    rng = random.Random(17 + len(mode))
    ramp = torch.arange(count, device=_dev(), dtype=torch.float32) % 13
    applied = [torch.zeros(count, dtype=torch.float64, device=_dev()) for _ in range(world)]
    try:
        for k in range(1, steps + 1):
            for r in range(world):
                w.grads[r].copy_(ramp + float((r + 1) * 100 + k))
            w.step(delays_us=[rng.choice([0, 0, 0, 30, 300]) for _ in range(world)])
            torch.cuda.synchronize()
            for r in range(world):
                applied[r] += w.outs[r].double()
        w.step(flush=True)
        torch.cuda.synchronize()
        for r in range(world):
            applied[r] += w.outs[r].double()
        for r in range(1, world):
            assert torch.equal(applied[r], applied[0])
        # every element saw the same number of gradients: (total - ramp * n) is constant over the vector
        n_applied = (applied[0][1] - applied[0][0]).item()        # ramp[1] - ramp[0] = 1 per gradient
        assert n_applied > 0
        assert torch.allclose(applied[0] - ramp.double() * n_applied, (applied[0][0]).expand(count), rtol=0, atol=1e-6)
        sts = [c.stats() for c in w.channels]
        assert all(s["status"] == 0 for s in sts)
        assert sum(s["participated"] for s in sts) > steps      # rounds with several participants happened
    finally:
        w.close()


@pytest.mark.parametrize("mode", ["solo", "majority"])
@pytest.mark.parametrize("two_shot_min", [None, 0])
def test_accumulate_loses_no_gradient(mode, two_shot_min):
    """With ``accumulate`` a gradient that no round picked up rides along with the rank's next publish of the
    same slot; after two closing rounds in which everybody is on time, every published gradient has been
    applied exactly once on every rank and none was dropped."""
    from eagersgd_b200.parallel.nvlink_channel import EmulatedWorld
    world, count, steps = 4, 8 * 129, 36
    w = EmulatedWorld(world, count, _dev(), slot_dtype=torch.float32, mode=mode, limiter=-1, average="sum",
                      timeout_s=2.0, grace_us=1000.0, adaptive_grace=False, accumulate=True, two_shot_min=two_shot_min)
    rng = random.Random(3 + len(mode))
    applied = [torch.zeros(count, dtype=torch.float64, device=_dev()) for _ in range(world)]
    try:
        for k in range(1, steps + 1):
            for r in range(world):
                w.grads[r].fill_(float((r + 1) * 100 + k))
            late = k <= steps - 2       # the last two rounds: everybody inside the grace window
            w.step(delays_us=[rng.choice([0, 0, 50, 4000]) if late else 0 for _ in range(world)])
            torch.cuda.synchronize()
            for r in range(world):
                applied[r] += w.outs[r].double()
        w.step(flush=True)
        torch.cuda.synchronize()
        for r in range(world):
            applied[r] += w.outs[r].double()
        published = float(sum((r + 1) * 100 + k for r in range(world) for k in range(1, steps + 1)))
        sts = [c.stats() for c in w.channels]
        for r in range(world):
            assert torch.all(applied[r] == published), (r, applied[r][0].item(), published)
            assert sts[r]["status"] == 0 and sts[r]["dropped_grads"] == 0
        assert sum(s["folded_grads"] for s in sts) > 0
    finally:
        w.close()


def test_late_ranks_pull_what_they_missed_fused():
    """Fused update under imbalance with plain SGD (no momentum, no weight decay): whatever order the rounds
    reach a rank in, participants and late ranks end with the same fp32 master weights up to rounding."""
    from eagersgd_b200.parallel.nvlink_channel import EmulatedWorld
    world, count, steps = 8, 8 * 640, 24
    w = EmulatedWorld(world, count, _dev(), slot_dtype=torch.bfloat16, grad_dtype=torch.bfloat16, fused=True,
                      mode="solo", limiter=5, average="contributors", timeout_s=2.0, grace_us=0.0, two_shot_min=0)
    rng = random.Random(5)
    try:
        w.hyper[:5] = torch.tensor([0.05, 0.0, 0.0, 0.0, 1.0])
        for k in range(steps):
            for r in range(world):
                w.grads[r].copy_(torch.randn(count, device=_dev()).to(torch.bfloat16))
            w.step(delays_us=[rng.choice([0, 0, 0, 40, 400]) for _ in range(world)])
        w.step(flush=True)
        torch.cuda.synchronize()
        sts = [c.stats() for c in w.channels]
        assert all(s["status"] == 0 for s in sts)
        assert sum(s["absent"] for s in sts) > 0 and sum(s["participated"] for s in sts) > steps
        for r in range(1, world):
            assert torch.allclose(w.w32[r], w.w32[0], rtol=0, atol=2e-5), (r, (w.w32[r] - w.w32[0]).abs().max())
        assert w.w32[0].abs().max() > 0
    finally:
        w.close()


def test_half_precision_float16_is_rejected():
    """The kernels read and write float32 and bfloat16 only: float16 tensors are refused up front
    instead of being read with the wrong element size."""
    import eagersgd_b200 as es
    from eagersgd_b200.parallel.nvlink_channel import NvlinkChannel, create_arenas
    dev = _dev()
    m = torch.nn.Linear(16, 16).to(dev).half()
    with pytest.raises(ValueError):
        es.SoloAllreduceOptimizer(torch.optim.SGD(m.parameters(), lr=0.1), es.Group())
    arena, bases = create_arenas(64, torch.float32, 0, 1)
    try:
        with pytest.raises(ValueError):
            NvlinkChannel(64, 0, 1, bases, dev, torch.zeros(64, dtype=torch.float16, device=dev),
                          slot_dtype=torch.float32, out=torch.zeros(64, device=dev))
        with pytest.raises(ValueError):
            NvlinkChannel(64, 0, 1, bases, dev, torch.zeros(64, device=dev), slot_dtype=torch.float16,
                          out=torch.zeros(64, device=dev))
    finally:
        arena.free()


def test_wrapped_optimizer_keeps_fp32_masters_and_skips_idle_steps():
    """A generic optimizer around bf16 parameters steps fp32 master copies (small updates are not rounded
    away) and the bf16 weights follow them."""
    import eagersgd_b200 as es
    dev = _dev()
    torch.manual_seed(3)
    m = torch.nn.Linear(64, 64, bias=False).to(dev).to(torch.bfloat16)
    w0 = m.weight.detach().float().clone()
    opt = es.SoloAllreduceOptimizer(torch.optim.Adam(m.parameters(), lr=1e-5), es.Group())
    assert not opt.fused
    for _ in range(8):
        opt.zero_grad()
        m(torch.randn(8, 64, device=dev, dtype=torch.bfloat16)).float().square().mean().backward()
        opt.step()
    torch.cuda.synchronize()
    (p, master), = list(opt.master_params())
    assert master.dtype == torch.float32 and p.dtype == torch.bfloat16
    moved = (master - w0).abs()
    assert moved.max() > 0 and moved.max() < 2e-4          # eight Adam steps of 1e-5: far below bf16 resolution of O(1) weights
    assert torch.equal(p.detach(), master.to(torch.bfloat16))
    opt.close()


def test_zero_copy_publishing_matches_the_staged_path():
    """Writing the gradient straight into the publish slot gives the same result as handing it over in a
    separate buffer (which the kernel copies into the slot)."""
    from eagersgd_b200.parallel.nvlink_channel import NvlinkChannel, create_arenas
    dev = _dev()
    count = 8 * 300
    outs = []
    for zero_copy in (False, True):
        arena, bases = create_arenas(count, torch.bfloat16, 0, 1)
        grad = torch.zeros(count, dtype=torch.bfloat16, device=dev)
        out = torch.zeros(count, device=dev)
        ch = NvlinkChannel(count, 0, 1, bases, dev, None if zero_copy else grad, slot_dtype=torch.bfloat16, mode="solo",
                           limiter=-1, average="world", out=out, timeout_s=2.0)
        res = []
        torch.manual_seed(9)
        for k in range(5):
            g = torch.randn(count, device=dev).to(torch.bfloat16)
            (ch.publish_view() if zero_copy else grad).copy_(g)
            ch.step()
            torch.cuda.synchronize()
            res.append(out.clone())
            assert torch.equal(out, g.float())
        assert ch.stats()["status"] == 0
        outs.append(res)
        arena.free()
    assert all(torch.equal(a, b) for a, b in zip(*outs))


def test_arena_guards_stay_intact_and_catch_an_overrun():
    """The guard regions between the sections of an arena survive real traffic (one-shot, two-shot, drains) and
    report a write that strays into them."""
    from eagersgd_b200.parallel.nvlink_channel import EmulatedWorld, device_view
    world, count = 4, 8 * 77
    w = EmulatedWorld(world, count, _dev(), slot_dtype=torch.bfloat16, grad_dtype=torch.bfloat16, mode="solo", limiter=3,
                      average="world", timeout_s=2.0, grace_us=0.0, two_shot_min=0)
    rng = random.Random(1)
    try:
        for k in range(12):
            for r in range(world):
                w.grads[r].copy_(torch.randn(count, device=_dev()).to(torch.bfloat16))
            w.step(delays_us=[rng.choice([0, 0, 50, 300]) for _ in range(world)])
        w.step(flush=True)
        for c in w.channels:
            c.check_canaries()
        ch = w.channels[2]
        device_view(ch.bases[2] + ch.layout.slot1 - 3, 1, torch.uint8, _dev()).fill_(0)    # one byte before slot 1
        with pytest.raises(RuntimeError, match="guard 1"):
            ch.check_canaries()
    finally:
        w.close()


def test_wrapped_lars_runs_as_fused_kernels_and_matches_the_python_optimizer():
    """LARS around bf16 and fp32 parameters: the wrapper steps it with the two fused kernels on fp32 master
    weights; same trajectory as the per-tensor Python LARS on fp32 copies."""
    import eagersgd_b200 as es
    from eagersgd_b200.optim.lars import LARS
    dev = _dev()
    torch.manual_seed(4)
    mk = lambda: torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.ReLU(), torch.nn.Linear(64, 8)).to(dev)
    m_ref, m = mk(), mk()
    m.load_state_dict(m_ref.state_dict())
    o_ref = LARS(m_ref.parameters(), lr=0.2, momentum=0.9, weight_decay=1e-3, eeta=0.02)
    o = es.SoloAllreduceOptimizer(LARS(m.parameters(), lr=0.2, momentum=0.9, weight_decay=1e-3, eeta=0.02), es.Group(),
                                  bucket_mb=0.004)
    assert o.lars and not o.fused and len(o.buckets) > 1
    n0 = es.parallel._native.launch_count()
    for k in range(5):
        x = torch.randn(16, 32, device=dev)
        for mod, opt in ((m_ref, o_ref), (m, o)):
            opt.zero_grad()
            mod(x).square().mean().backward()
            opt.step()
    torch.cuda.synchronize()
    for p, q in zip(m_ref.parameters(), m.parameters()):
        assert torch.allclose(p, q, rtol=1e-4, atol=1e-6), (p - q).abs().max()
    assert es.parallel._native.launch_count() - n0 == 5 * len(o.buckets) * 4      # 2 collective + 2 LARS launches per bucket
    o.close()


@pytest.mark.parametrize("world", [2, 3, 5, 8])
def test_classic_collectives_emulated_on_one_gpu(world):
    """Broadcast, gather, all-gather, all-reduce, send / receive, ring sum and barrier of the peer-memory
    collectives, all ranks on one GPU in one cooperative launch per operation, against closed forms."""
    from eagersgd_b200.parallel.peer_collectives import EmulatedCollectives
    dev = _dev()
    ec = EmulatedCollectives(world, dev)
    n = 10_007
    base = torch.arange(n, device=dev) % 13
    ts = [(base + r).float() for r in range(world)]
    ec.bcast(ts, world - 1)
    assert all(torch.equal(t, (base + world - 1).float()) for t in ts)
    us = [((torch.arange(1001, device=dev) % 251) + r).to(torch.uint8) for r in range(world)]
    outs = ec.allgather(us)
    for r in range(world):
        for j in range(world):
            assert torch.equal(outs[r][j], us[j])
    g = ec.gather(us, 1)
    assert all(torch.equal(g[j], us[j]) for j in range(world))
    torch.manual_seed(world)
    for dt in (torch.float32, torch.bfloat16):
        xs = [torch.randn(4096, device=dev).to(dt) for _ in range(world)]
        expect = torch.zeros(4096, device=dev)
        for x in xs:
            expect += x.float()
        ec.allreduce(xs)
        assert all(torch.equal(x, expect.to(dt)) for x in xs)
    a, b = torch.full((333,), 7.0, device=dev), torch.zeros(333, device=dev)
    ec.send_recv(a, world - 1, b, 0)
    assert torch.equal(a, b)
    if world >= 3:
        zs = [torch.full((64,), float(r + 1), device=dev) for r in range(world)]
        ec.neighbours(zs)
        for r in range(world):
            assert torch.all(zs[r] == float((r + 1) + ((r - 1) % world + 1) + ((r + 1) % world + 1)))
    ec.barrier()
    assert ec.status() == [0] * world


def test_collective_wait_for_a_silent_rank_runs_out_with_a_status():
    """A receive from a rank that never sends: the bounded wait ends, the status says which wait it was, the
    destination is untouched and the context keeps working."""
    from eagersgd_b200.parallel.peer_collectives import EmulatedCollectives, RED_NONE
    dev = _dev()
    ec = EmulatedCollectives(2, dev, timeout_s=0.2)
    b = torch.full((16,), 3.0, device=dev)
    ops = [(0, 0, 0, 0, 0, 0, RED_NONE, -1), (0, 1, 64, 0, b.data_ptr(), 0, RED_NONE, -1)]   # rank 1 reads, nobody writes
    ec._run(ops)
    assert ec.status() == [0, 2] and torch.all(b == 3.0)
    assert float((torch.ones(4, device=dev) * 2).sum()) == 8.0


@pytest.mark.parametrize("dtype,n", [(torch.float32, 4096), (torch.bfloat16, 1003), (torch.float32, 77)])
def test_partial_allreduce_object_on_one_gpu(dtype, n):
    """The schedule-like object on a CUDA tensor (world of one): post returns at once, wait delivers the average in
    place or into ``out``, sizes that are no multiple of eight are padded inside, the counters count."""
    import eagersgd_b200 as es
    dev = _dev()
    g = es.Group()
    t = (torch.arange(n, device=dev, dtype=torch.float32) % 17 - 8).to(dtype)
    ref = t.clone()
    seen = []
    with es.PartialAllreduce(t, g, mode="solo", limiter=2, on_complete=seen.append) as ar:
        for k in range(4):
            ar.post()
            info = ar.wait()
            assert info["applied"] and info["role"] == "participant" and info["contributors"] == 1
            assert torch.equal(t, ref)                      # the average over one rank is the tensor itself
        out = torch.zeros(n, device=dev, dtype=dtype)
        ar.resize(t, out)
        ar.post()
        assert ar.wait()["applied"] and torch.equal(out, ref)
        st = ar.stats()
        assert st["steps"] == 1 and st["status"] == 0 and "NVLink" in ar.describe()
    assert len(seen) == 5
