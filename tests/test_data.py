import numpy as np
import pytest
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
    import types
    comm = types.SimpleNamespace(rank=1, world=4)                  # a process group, as the reference passes its communicator
    g = D.DistributedSampler(D.ShuffleSampler(ds, 5, seed=1), comm)
    assert (g.rank, g.world, len(g)) == (1, 4, 5)
    p = D.PartitionedDistributedSampler(D.OrderedSampler, ds, 5, comm)
    assert np.concatenate([b["y"] for b in p]).tolist() == list(range(25, 50))
    q = D.PartitionedDistributedSampler(D.ShuffleSampler(ds, 5, seed=3), comm)       # a ready sampler and a group
    assert sorted(np.concatenate([b["y"] for b in q]).tolist()) == list(range(25, 50))
    assert len(D.PartitionedDistributedSampler(D.OrderedSampler(ds, 10), None)) == 10  # no group: everything
    alone = D.DistributedSampler(D.OrderedSampler(ds, 10))         # no job: one rank
    assert (alone.rank, alone.world, len(alone)) == (0, 1, 10)


def test_augmentations():
    x = {"x": np.random.rand(6, 3, 32, 32).astype(np.float32), "y": np.arange(6)}
    assert D.Crop((28, 28), random_crop=True, padding=(4, 4), seed=0)(x)["x"].shape == (6, 3, 28, 28)
    assert D.Resize((16, 16))(x)["x"].shape == (6, 3, 16, 16)
    n = D.Normalize([0.5] * 3, [0.25] * 3)(x)["x"]
    assert np.allclose(n, (x["x"] - 0.5) / 0.25)
    assert np.allclose(D.Normalize(0.5, stddev=2.0)(x)["x"], (x["x"] - 0.5) / 2.0)          # one number for every channel
    f = D.RandomFlip(p=1.0)(x)["x"]
    assert np.array_equal(f, x["x"][:, :, :, ::-1])
    assert np.array_equal(D.RandomFlip(1, 1.0)(x)["x"], x["x"][:, :, ::-1, :])              # axis 1 of a sample: up-down
    assert np.array_equal(D.RandomFlip(p=0.0)(x)["x"], x["x"])
    c = D.Cutout(1, 8, seed=0)(x)["x"]                                                     # holes, length: the reference's order
    assert 0 < (c == 0).sum() <= 6 * 3 * 64
    two = D.Cutout(holes=2, length=4, random_fill=True, seed=0)(x)["x"]
    changed = (two != x["x"])
    assert 0 < changed.sum() <= 6 * 3 * 2 * 16 and two[changed].min() >= -0.5 and two[changed].max() < 0.5
    back = D.Crop((16, 16), resize=True)(x)["x"]                                            # centre crop scaled back up
    assert back.shape == (6, 3, 32, 32) and np.array_equal(back[:, :, ::2, ::2], x["x"][:, :, 8:24, 8:24])
    r = D.ReplicateBatch(3)(x)
    assert r["x"].shape[0] == 18 and r["y"].tolist() == [0, 0, 0, 1, 1, 1, 2, 2, 2, 3, 3, 3, 4, 4, 4, 5, 5, 5]


def test_synthetic_image_dataset_is_deterministic():
    ds = D.SyntheticImageDataset(50, (3, 8, 8), classes=10, seed=4)
    a, b = ds[7], ds[7]
    assert np.array_equal(a["x"], b["x"]) and a["y"] == b["y"]
    batch = ds[np.array([1, 2, 3])]
    assert batch["x"].shape == (3, 3, 8, 8) and batch["y"].shape == (3,)


def test_video_loader_follows_the_reference_pipeline(tmp_path):
    """Left zero-padding to the longest clip, [:max_length:skip] sub-sampling, 1/255 scaling, channels first
    (deep500/datasets/ucf101.py:92-109), and the UCF101 list files."""
    import numpy as np
    from eagersgd_b200.data import BucketSampler, VideoFolderDataset, VideoLoader, read_split, write_synthetic_ucf101
    root = write_synthetic_ucf101(str(tmp_path / "ucf"), classes=3, clips_per_class=4, frames=(12, 30), size=(16, 24))
    paths, labels, classes = read_split(root, "trainlist01.txt")
    assert len(classes) == 3 and len(paths) == len(labels) > 0 and all(p.endswith(".npy") for p in paths)
    loader = VideoLoader(normalize=False, max_length=25, skip_frames=3)
    a, b = np.load(paths[0]), np.load(paths[1])
    batch = loader([paths[0], paths[1]])
    longest = max(len(a), len(b))
    expect_t = len(range(0, min(longest, 25), 3))
    assert batch.shape == (2, expect_t, 3, 16, 24)
    short, n_short = (0, len(a)) if len(a) < len(b) else (1, len(b))
    padded = np.concatenate([np.zeros((longest - n_short, 16, 24, 3), np.float32), (a if short == 0 else b).astype(np.float32)])
    assert np.allclose(batch[short], np.moveaxis(padded[:25:3] / 255.0, -1, -3))
    ds = VideoFolderDataset(root, "trainlist01.txt", loader)
    s = BucketSampler(ds, 2, ds.lengths, num_buckets=4, max_length=50, seed=0)
    got = s()
    assert got["x"].ndim == 5 and got["x"].shape[0] == 2 and got["x"].shape[2] == 3


def test_resnet_lstm_video_model_runs_on_cpu():
    import torch
    from eagersgd_b200.models.resnet import cifar_resnet
    from eagersgd_b200.models.video import ResNetLSTM
    torch.manual_seed(0)
    net = cifar_resnet(8, 1, 10)
    m = ResNetLSTM(5, hidden=16, frame_net=net, feature_dim=net.fc.in_features, frame_chunk=7)
    x = torch.randn(2, 6, 3, 16, 16)
    out = m(x)
    assert out.shape == (2, 5)
    out.sum().backward()
    assert m.rnn.w_hh[0].grad is not None and next(net.parameters()).grad is not None


def test_imagenet_from_disk_folder_shards_and_preprocessing(tmp_path):
    """The folder layout and the packed shards give the same images and labels; evaluation pre-processing is the
    aspect-preserving resize + central crop with the channel means subtracted, training pre-processing a random
    crop / flip of the right size (official/resnet/imagenet_preprocessing.py)."""
    import numpy as np
    from eagersgd_b200.data import (CHANNEL_MEANS, ImageNetFolder, ShardedImageDataset, build_shards, decode_image,
                                    preprocess_image, random_crop_box, write_synthetic_imagenet)
    root = write_synthetic_imagenet(str(tmp_path / "inet"), classes=3, per_class=4)
    val = ImageNetFolder(root, "val")
    assert len(val) == 3 * 2 and len(val.classes) == 3 and not val.is_training
    one = val[0]
    assert one["x"].shape == (3, 224, 224) and one["x"].dtype == np.float32 and one["y"] == 0
    raw = decode_image(val.files[0])
    h, w = raw.shape[:2]
    assert np.allclose(preprocess_image(raw, False), one["x"])
    assert one["x"].min() >= -max(CHANNEL_MEANS) - 1e-3 and one["x"].max() <= 255.0
    train = ImageNetFolder(root, "train", seed=3, label_offset=1)
    b = train[[0, 5, 9]]
    assert b["x"].shape == (3, 3, 224, 224) and list(b["y"]) == [1, 2, 3]          # 1001-class convention
    train.batchaug = 3                                   # every sample three times, each copy with its own crop and flip
    a = train[[0, 5]]
    assert a["x"].shape == (6, 3, 224, 224) and list(a["y"]) == [1, 1, 1, 2, 2, 2]
    assert not (np.array_equal(a["x"][0], a["x"][1]) and np.array_equal(a["x"][0], a["x"][2]))
    train.num_parallel_calls = 2
    assert train[[0, 5]]["x"].shape == (6, 3, 224, 224)
    train.batchaug, train.num_parallel_calls = 1, 1
    val.batchaug = 3
    assert val[[0, 1]]["x"].shape == (2, 3, 224, 224)    # evaluation batches are never replicated
    rng = np.random.default_rng(0)
    for _ in range(50):
        t, l, ch, cw = random_crop_box(60, 80, rng)
        assert 0 <= t and 0 <= l and t + ch <= 60 and l + cw <= 80 and 0.74 <= cw / ch <= 1.35 or (ch, cw) == (60, 80)
    shards = build_shards(root, "val", str(tmp_path / "shards"), shard_size=4)
    assert len(shards) == 2
    sv = ShardedImageDataset(str(tmp_path / "shards"), "val")
    assert len(sv) == len(val) and sorted(sv.labels.tolist()) == sorted(val.labels.tolist())
    by_label = {int(l): i for i, l in enumerate(sv.labels)}
    i_sh = by_label[int(val.labels[-1])]
    assert sv[i_sh]["x"].shape == (3, 224, 224)


def test_download_helpers_against_a_mirror_on_disk(tmp_path):
    """``real_download`` and the MNIST helper against a ``file://`` mirror (no network here): files arrive once, are
    kept on a second call, load as a data set; a wrong checksum removes the file; a missing file leaves nothing
    behind; archives unpack inside their folder only."""
    import gzip
    import os
    import struct
    import tarfile
    import pytest
    from eagersgd_b200.data.dataset import load_mnist
    from eagersgd_b200.utils import download as D
    mirror = tmp_path / "mirror"
    mirror.mkdir()

    def idx(arr):
        arr = np.asarray(arr, dtype=np.uint8)
        return struct.pack(">I", 0x0800 | arr.ndim) + struct.pack(">" + "I" * arr.ndim, *arr.shape) + arr.tobytes()

    rng = np.random.RandomState(0)
    for stem, arr in (("train-images-idx3-ubyte", rng.randint(0, 255, (12, 28, 28))), ("train-labels-idx1-ubyte", np.arange(12) % 10),
                      ("t10k-images-idx3-ubyte", rng.randint(0, 255, (4, 28, 28))), ("t10k-labels-idx1-ubyte", np.arange(4))):
        with gzip.open(mirror / (stem + ".gz"), "wb") as f:
            f.write(idx(arr))
    cache = tmp_path / "cache"
    paths = D.download_mnist_and_get_file_paths(str(cache), base_url="file://" + str(mirror) + "/")
    assert set(paths) == {"train_images", "train_labels", "test_images", "test_labels"}
    stamp = os.path.getmtime(paths["train_images"])
    assert D.download_mnist_and_get_file_paths(str(cache), base_url="file:///nowhere/") == paths     # kept, not fetched again
    assert os.path.getmtime(paths["train_images"]) == stamp
    train, test = load_mnist(os.path.dirname(paths["train_images"]))
    assert len(train) == 12 and len(test) == 4
    name = "train-labels-idx1-ubyte.gz"
    with pytest.raises(IOError, match="checksum"):
        D.real_download("file://" + str(mirror), [name], "other", str(cache), sha256={name: "0" * 64})
    assert not (cache / "other" / name).exists()
    with pytest.raises(IOError):
        D.real_download("file://" + str(mirror), ["missing.bin"], "other", str(cache))
    assert list((cache / "other").iterdir()) == []
    good = D.real_download("file://" + str(mirror), [name], "other", str(cache), sha256={name: D.sha256_of(str(mirror / name))})
    assert D.unpack(good[name]).endswith("train-labels-idx1-ubyte")
    evil = tmp_path / "evil.tar.gz"
    with tarfile.open(evil, "w:gz") as t:
        info = tarfile.TarInfo("../escaped.txt")
        info.size = 0
        t.addfile(info)
    with pytest.raises(IOError, match="escapes"):
        D.unpack(str(evil), str(tmp_path / "x"))


def test_sampler_invariants_over_random_sizes():
    """Property test of the samplers: an epoch of the ordered and the shuffling sampler visits every sample at most
    once and all of them unless the ragged last batch is dropped; the bucket sampler's batches stay inside one length
    bucket, visit every sequence once, and pad on the left to the longest sequence of the batch."""
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st
    from eagersgd_b200.data.dataset import NumpyDataset
    from eagersgd_b200.data.sampler import BucketSampler, OrderedSampler, ShuffleSampler

    @settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
    @given(n=st.integers(1, 70), bs=st.integers(1, 12), drop=st.booleans(), seed=st.integers(0, 1000))
    def plain(n, bs, drop, seed):
        ds = NumpyDataset(np.arange(n, dtype=np.float32).reshape(n, 1), "x", np.arange(n), "y")
        for cls in (OrderedSampler, ShuffleSampler):
            s = cls(ds, bs, seed=seed, drop_last_batch=drop)
            for _ in range(2):                                   # two epochs
                seen = np.concatenate([b["y"] for b in s] or [np.zeros(0, np.int64)])
                assert len(seen) == len(set(seen.tolist()))
                assert len(seen) == ((n // bs) * bs if drop else n)
                assert len(s) == (n // bs if drop else -(-n // bs))
                s.reset()

    class Seqs:
        data_node, label_node = "x", "y"

        def __init__(self, lengths):
            self.seqs = [np.full((int(l), 2), i, dtype=np.float32) for i, l in enumerate(lengths)]

        def __len__(self):
            return len(self.seqs)

        def __getitem__(self, i):
            return {"x": self.seqs[i], "y": i}

    @settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
    @given(lengths=st.lists(st.integers(1, 50), min_size=1, max_size=40), bs=st.integers(1, 6), nb=st.integers(1, 8),
           seed=st.integers(0, 1000))
    def buckets(lengths, bs, nb, seed):
        ds = Seqs(lengths)
        s = BucketSampler(ds, bs, np.asarray(lengths), num_buckets=nb, seed=seed, drop_last_batch=False)
        width = max(lengths) / nb
        seen = []
        for b in s:
            ids = b["y"].tolist()
            seen += ids
            lens = [lengths[i] for i in ids]
            assert b["x"].shape[1] == max(lens) and b["lengths"].tolist() == lens
            for row, i in zip(b["x"], ids):                      # left padding: zeros, then the sequence
                pad = b["x"].shape[1] - lengths[i]
                assert np.all(row[:pad] == 0) and np.all(row[pad:] == i)
            which = {min(int(np.ceil(l / width)) - 1, nb - 1) if l > 0 else 0 for l in lens}
            assert len(which) == 1 or max(lens) - min(lens) <= width + 1e-9, (lens, width)
        assert sorted(seen) == list(range(len(lengths)))

    plain()
    buckets()


def test_imagenet_preprocessing_over_random_image_sizes():
    """Images of any size, tiny and extreme aspect ratios included, come out as float32 [3, 224, 224] in both the
    training and the evaluation path; the random crop always lies inside the image."""
    pytest = __import__("pytest")
    pytest.importorskip("PIL")
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st
    from eagersgd_b200.data.imagenet import preprocess_image, random_crop_box

    @settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow])
    @given(h=st.integers(1, 400), w=st.integers(1, 400), seed=st.integers(0, 10 ** 6), train=st.booleans())
    def check(h, w, seed, train):
        rng = np.random.default_rng(seed)
        t, l, ch, cw = random_crop_box(h, w, rng)
        assert 0 <= t and 0 <= l and ch >= 1 and cw >= 1 and t + ch <= h and l + cw <= w
        img = rng.integers(0, 256, size=(h, w, 3), dtype=np.uint8)
        out = preprocess_image(img, train, rng)
        assert out.shape == (3, 224, 224) and out.dtype == np.float32 and np.isfinite(out).all()
        assert out.min() >= -130.0 and out.max() <= 160.0          # 0..255 minus channel means of 104..124

    check()


def _write_cifar10_bin(root, per_file=16, seed=0):
    """A miniature cifar-10-batches-bin: records of one label byte and 3072 pixel bytes, channel-major."""
    import os
    d = os.path.join(root, "cifar-10-batches-bin")
    os.makedirs(d, exist_ok=True)
    rng = np.random.RandomState(seed)
    everything = []
    for name in ["data_batch_%d.bin" % i for i in range(1, 6)] + ["test_batch.bin"]:
        labels = rng.randint(0, 10, size=per_file).astype(np.uint8)
        pixels = rng.randint(0, 256, size=(per_file, 3, 32, 32)).astype(np.uint8)
        np.concatenate([labels[:, None], pixels.reshape(per_file, -1)], axis=1).tofile(os.path.join(d, name))
        everything.append((labels, pixels))
    return d, everything


def test_cifar10_binary_files_and_the_reference_pipeline(tmp_path):
    """The binary CIFAR-10 files the reference's main program reads, and its input pipeline: pad by four, random crop,
    random flip, per-image standardisation; copies for batch augmentation are made before the random steps
    (official/resnet/cifar10_main.py:33-125)."""
    import pickle
    from eagersgd_b200.data import (OrderedSampler, PerImageStandardization, ShuffleSampler, cifar10_transforms,
                                    load_cifar10)
    d, files = _write_cifar10_bin(str(tmp_path))
    for path in (str(tmp_path), d):                                 # the folder itself or its parent
        train, test = load_cifar10(path)
        assert len(train) == 80 and len(test) == 16
        assert np.array_equal(train[16:32]["y"], files[1][0]) and np.allclose(train[16:32]["x"] * 255, files[1][1])
        assert np.array_equal(test[:]["y"], files[5][0]) and test[0]["x"].shape == (3, 32, 32)
    py = tmp_path / "py" / "cifar-10-batches-py"                    # the pickled form gives the same data
    py.mkdir(parents=True)
    for k, name in enumerate(["data_batch_%d" % i for i in range(1, 6)] + ["test_batch"]):
        with open(py / name, "wb") as f:
            pickle.dump({b"data": files[k][1].reshape(16, -1), b"labels": files[k][0].tolist()}, f)
    train_py, _ = load_cifar10(str(tmp_path / "py"))
    assert np.array_equal(train_py[:]["x"], train[:]["x"]) and np.array_equal(train_py[:]["y"], train[:]["y"])
    with pytest.raises(FileNotFoundError):
        load_cifar10(str(tmp_path / "nothing"))
    (tmp_path / "bad").mkdir()
    for i in range(1, 6):
        (tmp_path / "bad" / ("data_batch_%d.bin" % i)).write_bytes(b"x" * 100)
    with pytest.raises(ValueError, match="3073"):
        load_cifar10(str(tmp_path / "bad"))
    # standardisation: zero mean, unit variance per image; a constant image does not divide by zero
    x = np.concatenate([train[:4]["x"], np.full((1, 3, 32, 32), 0.25, np.float32)])
    z = PerImageStandardization().apply(x)
    assert np.allclose(z[:4].reshape(4, -1).mean(1), 0, atol=1e-5) and np.allclose(z[:4].reshape(4, -1).std(1), 1, atol=1e-4)
    assert np.all(z[4] == 0) and z.dtype == np.float32
    # training pipeline: three copies of every sample, each with its own crop / flip of the padded image
    s = ShuffleSampler(train, 8, seed=1)
    for t in cifar10_transforms(True, seed=5, batchaug=3):
        s.add_input_transformation(t)
    b = s()
    assert b["x"].shape == (24, 3, 32, 32) and b["x"].dtype == np.float32
    assert b["y"].shape == (24,) and np.array_equal(b["y"][0::3], b["y"][1::3])
    assert np.allclose(b["x"].reshape(24, -1).mean(1), 0, atol=1e-4)
    copies = b["x"][:3]
    assert not np.allclose(copies[0], copies[1]) or not np.allclose(copies[0], copies[2])
    # without the last step the crop is a window of the zero-padded original, possibly mirrored
    crop, flip = cifar10_transforms(True, seed=9)[:2]
    one = train[:1]
    out = flip(crop(one))["x"][0]
    padded = np.pad(one["x"][0], ((0, 0), (4, 4), (4, 4)))
    windows = [padded[:, t:t + 32, l:l + 32] for t in range(9) for l in range(9)]
    assert any(np.array_equal(out, wnd) or np.array_equal(out, wnd[:, :, ::-1]) for wnd in windows)
    # evaluation: standardisation only, order kept
    v = OrderedSampler(test, 16)
    for t in cifar10_transforms(False):
        v.add_input_transformation(t)
    e = v()
    assert np.array_equal(e["y"], files[5][0]) and np.allclose(e["x"], PerImageStandardization().apply(test[:]["x"]))


def test_cifar10_main_trains_from_binary_files(tmp_path):
    from eagersgd_b200.train import resnet_main
    _write_cifar10_bin(str(tmp_path / "data"), per_file=16)
    rc = resnet_main.main(["--dataset", "cifar10", "--data_dir", str(tmp_path / "data"), "-rs", "8", "-bs", "8", "--train_epochs", "1",
                           "--max_train_steps", "3", "--mode", "sync", "--dtype", "fp32", "--batchaug", "2",
                           "--model_dir", str(tmp_path / "m"), "--train_acc_steps", "1"])
    assert rc == 0 and (tmp_path / "m" / "0" / "checkpoint").exists()


def test_imagenet_main_trains_from_a_folder_on_disk(tmp_path):
    """The main program on ImageNet read from class folders: decode, the reference's pre-processing, batch-augmentation
    copies made before it, a step, an evaluation pass, a checkpoint."""
    from eagersgd_b200.data import write_synthetic_imagenet
    from eagersgd_b200.train import resnet_main
    root = write_synthetic_imagenet(str(tmp_path / "inet"), classes=3, per_class=4)
    rc = resnet_main.main(["--dataset", "imagenet", "--data_dir", root, "-rs", "18", "-bs", "2", "--train_epochs", "1",
                           "--max_train_steps", "2", "--mode", "sync", "--dtype", "fp32", "--batchaug", "2",
                           "--num_parallel_calls", "2", "--model_dir", str(tmp_path / "m"), "--train_acc_steps", "1"])
    assert rc == 0 and (tmp_path / "m" / "0" / "checkpoint").exists()


def test_cifar100_files_the_registry_and_the_fast_schedule(tmp_path):
    """CIFAR-100's binary records carry a coarse and a fine label; the registry reads either CIFAR by name and
    normalises by the channel statistics as the reference's loaders do (deep500/datasets/cifar.py:58-128)."""
    import os
    d = tmp_path / "c100" / "cifar-100-binary"
    os.makedirs(d)
    rng = np.random.RandomState(0)
    data = {}
    for name, n in (("train.bin", 24), ("test.bin", 8)):
        coarse, fine = rng.randint(0, 20, n).astype(np.uint8), rng.randint(0, 100, n).astype(np.uint8)
        px = rng.randint(0, 256, size=(n, 3, 32, 32)).astype(np.uint8)
        np.concatenate([coarse[:, None], fine[:, None], px.reshape(n, -1)], axis=1).tofile(d / name)
        data[name] = (fine, px)
    train, test = D.load_cifar100(str(tmp_path / "c100"))
    assert len(train) == 24 and np.array_equal(train[:]["y"], data["train.bin"][0]) and np.allclose(test[:]["x"] * 255, data["test.bin"][1])
    tr, te = D.load_dataset("cifar100", "input", "label", path=str(tmp_path / "c100"))
    b = tr[:]
    assert set(b) == {"input", "label"} and np.array_equal(b["label"], data["train.bin"][0])
    mean = np.asarray(D.CIFAR_MEAN["cifar100"], np.float32).reshape(1, 3, 1, 1)
    std = np.asarray(D.CIFAR_STD["cifar100"], np.float32).reshape(1, 3, 1, 1)
    assert np.allclose(b["input"], (data["train.bin"][1] / 255.0 - mean) / std, atol=1e-5)
    raw, _ = D.load_dataset("cifar100", path=str(tmp_path / "c100"), normalize=False)
    assert raw[:]["x"].min() >= 0 and raw[:]["x"].max() <= 1
    _write_cifar10_bin(str(tmp_path / "c10"), per_file=4)
    t10, _ = D.load_dataset("cifar10", path=str(tmp_path / "c10"))
    assert len(t10) == 20 and t10[:]["x"].min() < 0                   # normalised
    assert D.dataset_shape("cifar100") == (100, 3, 32, 32) and D.dataset_shape("mnist") == (10, 1, 28, 28)
    with pytest.raises(KeyError):
        D.dataset_shape("svhn")
    syn_tr, syn_te = D.load_dataset("fashion_mnist", synthetic_samples=64)
    assert syn_tr[:]["x"].shape == (64, 1, 28, 28) and len(syn_te) == 32
    assert [round(D.cifar_learning_rate(e), 6) for e in (0, 60, 61, 121, 161)] == [0.1, 0.1, 0.02, 0.004, 0.0008]


def test_ucf101_through_the_registry(tmp_path):
    root = D.write_synthetic_ucf101(str(tmp_path / "ucf"), classes=2, clips_per_class=3)
    assert D.dataset_shape("ucf101") == (101, None, 3, 240, 320)
    train, test = D.load_dataset("ucf101", "frames", "label", path=root)
    assert len(train) + len(test) == 6 and (train.data_node, train.label_node) == ("frames", "label")
    with pytest.raises(FileNotFoundError, match="path="):
        D.load_dataset("ucf101")
