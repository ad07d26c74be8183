"""How long does it take to draw a minibatch from each data set?

    python samples/dataset_latency.py [--batch 128] [--batches 5]

Counterpart of deep500 samples/dataset_latency.py:10-32 (a wall-clock metric on the sampler): synthetic images,
synthetic variable-length feature sequences (bucketed), decoded video clips and JPEG files in the ImageNet layout.
"""
import argparse
import tempfile
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from eagersgd_b200.data import (BucketSampler, ImageNetFolder, ShuffleSampler, SyntheticImageDataset,  # noqa: E402
                                SyntheticSequenceDataset, VideoFolderDataset, VideoLoader, write_synthetic_imagenet,
                                write_synthetic_ucf101)
from eagersgd_b200.ops.validation import test_sampler  # noqa: E402


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--batches", type=int, default=3)
    args = ap.parse_args(argv)
    tmp = tempfile.mkdtemp()
    seqs = SyntheticSequenceDataset(256, 256, 101, max_len=300, seed=0)
    video = VideoFolderDataset(write_synthetic_ucf101(os.path.join(tmp, "ucf"), classes=3, clips_per_class=4),
                               "trainlist01.txt", VideoLoader(skip_frames=4))
    inet = ImageNetFolder(write_synthetic_imagenet(os.path.join(tmp, "inet"), classes=3, per_class=6), "train")
    cases = [("synthetic CIFAR images", ShuffleSampler(SyntheticImageDataset(1024, (3, 32, 32), 10), args.batch, seed=0)),
             ("synthetic ImageNet images", ShuffleSampler(SyntheticImageDataset(256, (3, 224, 224), 1000), args.batch, seed=0)),
             ("feature sequences (bucketed)", BucketSampler(seqs, 8, seqs.lengths, num_buckets=10, max_length=300, seed=0)),
             ("video clips from disk", BucketSampler(video, 2, video.lengths, num_buckets=4, max_length=100, seed=0)),
             ("JPEG files, ImageNet layout", ShuffleSampler(inet, 6, seed=0))]
    out = {}
    for name, sampler in cases:
        r = test_sampler(sampler, batches=args.batches)
        out[name] = r
        print("%-32s %s" % (name, ", ".join("%s %.4g" % kv for kv in sorted(r.items()))))
    return out


if __name__ == "__main__":
    main()
