"""The process group's collectives and the gradient-exchange operations of the graph executor on CPU ranks
(gloo): every method of the reference's CommunicationNetwork (deep500/lv3/communication.py:14-119)."""
import numpy as np
import torch

from mp_util import run_ranks


def _group_methods(rank, world):
    import eagersgd_b200 as es
    g = es.init()
    res = {}
    t = torch.full((5,), float(rank + 1))
    g.sync_all(t)
    res["sync_all"] = bool(torch.all(t == sum(range(1, world + 1))))
    t = torch.full((5,), float(rank + 1))
    g.sync_all_at_root(t, average=True)
    res["sync_all_at_root"] = bool(torch.all(t == (world + 1) / 2.0)) if rank == 0 else True
    parts = g.gather_at_root(torch.tensor([float(rank)]))
    res["gather_at_root"] = (parts is None) if rank else [float(p) for p in parts] == [float(r) for r in range(world)]
    b = torch.full((3,), float(rank))
    g.sync_all_with_root(b, root=world - 1)
    res["bcast"] = bool(torch.all(b == world - 1))
    if rank == 0:
        buf = torch.empty(2)
        srcs = sorted(g.wait_for_any_rank(buf) for _ in range(world - 1))
        res["any"] = srcs == list(range(1, world))
        for r in range(1, world):
            g.send_to_rank(torch.tensor([float(r), 7.0]), r)
    else:
        g.send_to_root(torch.tensor([float(rank), 0.0]))
        back = torch.empty(2)
        g.wait_for_root(back)
        res["any"] = back.tolist() == [float(rank), 7.0]
    n = torch.full((4,), float(rank + 1))
    g.reduce_from_neighbors(n)
    left, right = (rank - 1) % world, (rank + 1) % world
    res["neighbours"] = bool(torch.all(n == float(rank + 1 + left + 1 + right + 1)))
    from eagersgd_b200.utils.launch import end_barrier
    end_barrier()                                               # meets the others once more and leaves the group
    res["left_group"] = not torch.distributed.is_initialized()
    return res


def test_every_group_method_on_three_cpu_ranks():
    for r, res in enumerate(run_ranks(_group_methods, 3)):
        assert all(res.values()), (r, res)


def _ps_gradient_graph(rank, world):
    """A graph with a ConsistentParameterServerGradients node: every rank ends up with the mean gradient."""
    import eagersgd_b200 as es
    from eagersgd_b200.graph import Graph, GraphNetwork
    group = es.init()
    g = Graph("ps")
    g.add_input("x")
    g.add_initializer("w", np.ones((2, 4), np.float32))
    g.add("Gemm", ["x", "w"], ["h"], transB=1)
    g.add("ConsistentParameterServerGradients", ["h"], ["hs"])
    g.add("InconsistentParameterServerGradients", ["hs"], ["out"])
    g.add_output("out")
    net = GraphNetwork(g, group=group)
    x = torch.full((1, 4), float(rank + 1), requires_grad=True)
    net(x).sum().backward()
    # d out / d h = 1 on every rank, so the mean is 1 and dx = w^T 1 = 2 everywhere; scale the loss by the rank to see
    # the averaging: d/dh = rank + 1 -> mean (world + 1) / 2
    x2 = torch.ones(1, 4, requires_grad=True)
    (net(x2).sum() * float(rank + 1)).backward()
    es.finalize()
    return x.grad.flatten().tolist(), x2.grad.flatten().tolist()


def test_parameter_server_gradient_operations_in_a_graph():
    res = run_ranks(_ps_gradient_graph, 2)
    for gx, gx2 in res:
        assert gx == [2.0] * 4
        assert gx2 == [2.0 * 1.5] * 4


def _partial_allreduce_object(rank, world):
    """The schedule-like life cycle on CPU ranks: start, post / wait and post / test, in place and out of place,
    a completion callback, resize, describe, close."""
    import time
    import eagersgd_b200 as es
    g = es.init()
    seen = []
    t = torch.zeros(10)
    ar = es.PartialAllreduce(t, g, mode="sync", average="sum", on_complete=seen.append).start()
    ok = True
    for k in range(1, 4):
        t.fill_(float(rank + k))
        ar.post()
        info = ar.wait()
        ok = ok and bool(torch.all(t == sum(r + k for r in range(world)))) and info["role"] == "participant" \
            and info["contributors"] == world and info["sync"]
    out = torch.zeros(10)
    ar.resize(torch.full((10,), 2.0), out)                 # out of place after a resize
    ar.post()
    while not ar.test():
        time.sleep(0.001)
    ok = ok and bool(torch.all(out == 2.0 * world)) and len(seen) == 4 and "sync" in ar.describe()
    ar.close()
    # solo: every post returns without waiting for the others; whoever misses a round gets it at the next step or flush
    x = torch.ones(16) * (rank + 1)
    with es.PartialAllreduce(x, g, mode="solo", limiter=4, average="world") as solo:
        for k in range(6):
            if rank == 1:
                time.sleep(0.01)
            solo.post()
            solo.wait()
        st = solo.flush()
    ok = ok and st["status"] == 0 and st["steps"] == 6
    es.finalize()
    return ok, st["forced_sync"]


def test_partial_allreduce_object_on_cpu_ranks():
    res = run_ranks(_partial_allreduce_object, 3)
    assert all(r[0] for r in res), res
    assert all(r[1] >= 1 for r in res)                     # the limiter forced a synchronous round


def test_partial_allreduce_object_single_rank():
    import eagersgd_b200 as es
    g = es.Group()
    t = torch.arange(5, dtype=torch.float64)
    with es.PartialAllreduce(t, g, mode="majority") as ar:
        ar.post()
        info = ar.wait()
        assert info["applied"] and torch.equal(t, torch.arange(5, dtype=torch.float64))
        assert not ar.test() is False
    import pytest
    with pytest.raises(RuntimeError):
        es.PartialAllreduce(torch.zeros(3), g).post()
