import numpy as np
from eagersgd_b200 import data as D


def test_ordered_and_shuffle_cover_dataset():
    ds = D.NumpyDataset(np.arange(103, dtype=np.float32)[:, None], "x", np.arange(103), "y")
    s = D.OrderedSampler(ds, 10)
    got = [b["y"] for b in s]
    assert len(got) == 10 and np.array_equal(np.concatenate(got), np.arange(100))
    s2 = D.ShuffleSampler(ds, 10, seed=3, drop_last_batch=False)
    ys = np.concatenate([b["y"] for b in s2])
    assert sorted(ys.tolist()) == list(range(103))
    s2.reset()
    ys2 = np.concatenate([b["y"] for b in s2])
    assert not np.array_equal(ys, ys2) and sorted(ys2.tolist()) == list(range(103))


def test_bucket_sampler_pads_little():
    ds = D.SyntheticSequenceDataset(400, feature_dim=8, min_len=30, max_len=1800, seed=1)
    s = D.BucketSampler(ds, 4, ds.lengths, num_buckets=30, max_length=500, seed=0)
    waste, n = 0.0, 0
    for b in s:
        t = b["x"].shape[1]
        assert b["x"].shape[0] == 4 and t <= 500
        assert np.all(b["lengths"] <= t)
        for i, l in enumerate(b["lengths"]):            # left padding is zeros
            assert np.all(b["x"][i, : t - l] == 0)
        waste += 1 - b["lengths"].sum() / (4 * t)
        n += 1
    assert n > 50 and waste / n < 0.15


def test_partitioned_and_distributed_samplers():
    ds = D.NumpyDataset(np.arange(100, dtype=np.float32)[:, None], "x", np.arange(100), "y")
    seen = []
    for r in range(4):
        s = D.PartitionedDistributedSampler(D.OrderedSampler, ds, 5, r, 4)
        seen.append(np.concatenate([b["y"] for b in s]))
        assert seen[-1].min() == r * 25 and seen[-1].max() == r * 25 + 24
    d = D.DistributedSampler(D.ShuffleSampler(ds, 5, seed=1), rank=2, world=4)
    assert len(d) == 5 and len([b for b in d]) == 5


def test_augmentations():
    x = {"x": np.random.rand(6, 3, 32, 32).astype(np.float32), "y": np.arange(6)}
    assert D.Crop((28, 28), random_crop=True, padding=(4, 4), seed=0)(x)["x"].shape == (6, 3, 28, 28)
    assert D.Resize((16, 16))(x)["x"].shape == (6, 3, 16, 16)
    n = D.Normalize([0.5] * 3, [0.25] * 3)(x)["x"]
    assert np.allclose(n, (x["x"] - 0.5) / 0.25)
    f = D.RandomFlip(1.0)(x)["x"]
    assert np.array_equal(f, x["x"][:, :, :, ::-1])
    c = D.Cutout(8, seed=0)(x)["x"]
    assert (c == 0).sum() > 0
    r = D.ReplicateBatch(3)(x)
    assert r["x"].shape[0] == 18 and r["y"].tolist() == [0, 0, 0, 1, 1, 1, 2, 2, 2, 3, 3, 3, 4, 4, 4, 5, 5, 5]


def test_synthetic_image_dataset_is_deterministic():
    ds = D.SyntheticImageDataset(50, (3, 8, 8), classes=10, seed=4)
    a, b = ds[7], ds[7]
    assert np.array_equal(a["x"], b["x"]) and a["y"] == b["y"]
    batch = ds[np.array([1, 2, 3])]
    assert batch["x"].shape == (3, 3, 8, 8) and batch["y"].shape == (3,)
