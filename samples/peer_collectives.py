"""Broadcast, all-gather, all-reduce and a ring of sends on this package's peer-memory kernels.

    torchrun --nproc-per-node 4 samples/peer_collectives.py          # one process per GPU
    python samples/peer_collectives.py --emulate 4                   # four ranks on one GPU

Stands where the reference ships MPI operators for its Caffe2 backend
(deep500/frameworks/caffe2/custom_operators/mpi/*.cpp) and a test program per operator.
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def emulated(world: int) -> None:
    from eagersgd_b200.parallel.peer_collectives import EmulatedCollectives
    dev = torch.device("cuda", 0)
    ec = EmulatedCollectives(world, dev)
    ts = [torch.full((8,), float(r), device=dev) for r in range(world)]
    ec.allreduce(ts)
    print("all-reduce:", ts[0][:2].tolist(), "(expected %.1f)" % sum(range(world)))
    ts = [torch.full((8,), float(r), device=dev) for r in range(world)]
    ec.bcast(ts, world - 1)
    print("broadcast from the last rank:", [t[0].item() for t in ts])
    print("all-gather on rank 0:", ec.allgather([torch.full((2,), float(r), device=dev) for r in range(world)])[0].tolist())
    print("status words:", ec.status())


def distributed() -> None:
    import eagersgd_b200 as es
    group = es.init()
    pc = group.peer_collectives(stage_mb=8.0)
    dev, r, world = group.device, group.rank, group.world
    t = torch.full((1 << 20,), float(r), device=dev)
    pc.allreduce(t)
    got = pc.allgather(torch.tensor([float(r)], device=dev)).flatten().tolist()
    x, y = torch.full((16,), float(r), device=dev), torch.empty(16, device=dev)
    pc.send(x, (r + 1) % world)
    pc.recv(y, (r - 1) % world)
    pc.barrier()
    pc.check()
    if r == 0:
        print("all-reduce:", t[0].item(), "all-gather:", got, "received from the left neighbour:", y[0].item())
    es.finalize()


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--emulate", type=int, default=0, help="run N ranks on one GPU instead of one process per GPU")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("this sample needs a GPU")
    emulated(a.emulate) if a.emulate else distributed()
