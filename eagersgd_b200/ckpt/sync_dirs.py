"""Make every rank's checkpoint directory a copy of rank 0's, between two jobs of a long run.

    python -m eagersgd_b200.ckpt.sync_dirs <model_dir> [--world N]

The reference trains ImageNet as a chain of jobs and, between them, replaces the per-rank directories
``<model_dir>/1 .. <model_dir>/63`` by copies of ``<model_dir>/0`` with a shell loop
(test_scripts_imagenet/synchm.sh:4-12), so that the replicas — which eager-SGD lets drift apart — start the next
job from one model.  Inside a running job the same is done in place, without files, by
``ckpt.resync_from_rank0`` / ``--resync_epochs``.  ``--world`` defaults to the rank directories that exist.
"""
from __future__ import annotations

import argparse
import os
import shutil
import sys


def sync_dirs(model_dir: str, world: int = 0) -> int:
    """Returns the number of directories rewritten."""
    src = os.path.join(model_dir, "0")
    if not os.path.isdir(src):
        raise FileNotFoundError("no rank-0 checkpoint directory under %s" % model_dir)
    if world <= 0:
        ranks = sorted(int(d) for d in os.listdir(model_dir) if d.isdigit() and d != "0")
    else:
        ranks = list(range(1, world))
    for r in ranks:
        dst = os.path.join(model_dir, str(r))
        tmp = dst + ".incoming"
        if os.path.isdir(tmp):
            shutil.rmtree(tmp)
        shutil.copytree(src, tmp)          # the old directory goes only once the copy is complete
        if os.path.isdir(dst):
            shutil.rmtree(dst)
        os.replace(tmp, dst)
    return len(ranks)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("model_dir")
    ap.add_argument("--world", type=int, default=0)
    a = ap.parse_args(argv)
    n = sync_dirs(a.model_dir, a.world)
    print("model synchronized: %d rank directories now equal rank 0's" % n)
    return 0


if __name__ == "__main__":
    sys.exit(main())
