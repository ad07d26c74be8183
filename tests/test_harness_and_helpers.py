"""The validation harness for executors / optimizers / samplers, and small helpers that every run relies on:
file-backed datasets, sequence collation, sampling with replacement, contiguous shards, logger hooks,
NumPy oracles, schedules, status words."""
import json
import os

import numpy as np
import pytest
import torch


def _executor(seed=0):
    from eagersgd_b200.train.executor import GraphExecutor, mse_loss
    torch.manual_seed(seed)
    return GraphExecutor(torch.nn.Linear(6, 3), mse_loss)


def test_executor_harness_against_closed_form_gradients():
    """Linear layer with a mean-squared-error loss: output and gradients are known in closed form
    (deep500/lv1/validation/executor.py compares an executor with reference outputs the same way)."""
    from eagersgd_b200.ops.validation import test_executor_backprop, test_executor_inference
    ex = _executor()
    rng = np.random.RandomState(1)
    x, y = rng.randn(5, 6).astype(np.float32), rng.randn(5, 3).astype(np.float32)
    w, b = ex.network.fetch_tensor("weight"), ex.network.fetch_tensor("bias")
    out = x @ w.T + b
    assert test_executor_inference(ex, {"x": x, "y": y}, out)["max_error"] < 1e-5
    d = 2 * (out - y) / out.size
    res = test_executor_backprop(ex, {"x": x, "y": y}, {"weight": d.T @ x, "bias": d.sum(0)})
    assert set(res) == {"weight", "bias"} and max(res.values()) < 1e-5
    with pytest.raises(AssertionError):
        test_executor_inference(ex, {"x": x, "y": y}, out + 0.1)
    with pytest.raises(AssertionError):
        test_executor_backprop(ex, {"x": x, "y": y}, {"weight": d.T @ x * 1.5})


def test_numerical_jacobian_of_a_known_map():
    from eagersgd_b200.ops.validation import numerical_jacobian, test_op_gradient
    a = torch.tensor([[1.0, 2.0], [3.0, 4.0]], dtype=torch.float64)
    x = torch.tensor([0.5, -1.0], dtype=torch.float64)
    J = numerical_jacobian(lambda m, v: m @ v, [a, x], wrt=1)
    assert torch.allclose(J, a, atol=1e-8)                       # d(Ax)/dx = A
    Ja = numerical_jacobian(lambda m, v: m @ v, [a, x], wrt=0)  # d(Ax)_i / dA_jk = delta_ij x_k
    expect = torch.zeros(2, 4, dtype=torch.float64)
    expect[0, :2], expect[1, 2:] = x, x
    assert torch.allclose(Ja, expect, atol=1e-8)
    assert max(test_op_gradient(lambda m, v: torch.tanh(m @ v), [a, x], eps=1e-5).values()) < 1e-6

    class WrongGrad(torch.autograd.Function):                    # an operator whose backward is off by a factor
        @staticmethod
        def forward(ctx, v):
            return v * 3

        @staticmethod
        def backward(ctx, g):
            return g * 2

    with pytest.raises(AssertionError, match="finite differences"):
        test_op_gradient(WrongGrad.apply, [x])


def test_optimizer_and_sampler_harness():
    from eagersgd_b200.data import NumpyDataset, ShuffleSampler
    from eagersgd_b200.ops.validation import test_optimizer, test_sampler
    from eagersgd_b200.optim.base import GradientDescent
    rng = np.random.RandomState(0)
    x = rng.randn(64, 6).astype(np.float32)
    y = (x @ rng.randn(6, 3)).astype(np.float32)
    ds = NumpyDataset(x, "x", y, "y")
    ex = _executor()
    r = test_optimizer(GradientDescent(ex, learning_rate=0.1), ShuffleSampler(ds, 16, seed=0), steps=12)
    assert r["last_loss"] < r["first_loss"] and r["median_step_ms"] > 0          # 12 steps wrap the 4-batch epoch
    s = test_sampler(ShuffleSampler(ds, 16, seed=0), batches=9)
    assert s["median_batch_ms"] >= 0 and s["distinct_sample_shapes"] == 1


def test_gradient_modifier_runs_before_the_update():
    from eagersgd_b200.optim.base import GradientDescent
    ex = _executor()
    opt = GradientDescent(ex, learning_rate=0.5)
    names = []

    def freeze_bias(name, g):
        names.append(name)
        return torch.zeros_like(g) if name == "bias" else g

    opt.gradient_modifier = freeze_bias
    w0, b0 = ex.network.fetch_tensor("weight").copy(), ex.network.fetch_tensor("bias").copy()
    opt.step({"x": np.ones((4, 6), np.float32), "y": np.zeros((4, 3), np.float32)})
    assert sorted(names) == ["bias", "weight"]
    assert np.array_equal(ex.network.fetch_tensor("bias"), b0) and not np.array_equal(ex.network.fetch_tensor("weight"), w0)


def test_file_list_dataset_and_folder_listing(tmp_path):
    from eagersgd_b200.data import FileListDataset, OrderedSampler
    from eagersgd_b200.data.imagenet import list_folder
    for c, cls in enumerate(["n02", "n01"]):
        os.makedirs(tmp_path / "train" / cls)
        for k in range(3):
            (tmp_path / "train" / cls / ("img_%d.jpeg" % k)).write_bytes(bytes([c, k]))
        (tmp_path / "train" / cls / "notes.txt").write_text("not an image")
    (tmp_path / "train" / "stray.jpg").write_bytes(b"x")        # not inside a class folder
    files, labels, classes = list_folder(str(tmp_path), "train")
    assert classes == ["n01", "n02"] and labels.tolist() == [0, 0, 0, 1, 1, 1] and len(files) == 6
    assert all(f.endswith(".jpeg") for f in files) and os.path.basename(os.path.dirname(files[0])) == "n01"
    reads = []

    def decode(path):
        reads.append(path)
        return np.frombuffer(open(path, "rb").read(), dtype=np.uint8).astype(np.float32)

    ds = FileListDataset(files, "x", labels, "y", decode)
    assert len(ds) == 6 and reads == []                          # nothing is decoded before it is asked for
    one = ds[4]
    assert one["x"].tolist() == [0.0, 1.0] and one["y"] == 1 and len(reads) == 1
    assert ds[1:3]["x"].shape == (2, 2) and ds[[5, 0]]["y"].tolist() == [1, 0]
    s = OrderedSampler(ds, 4)
    b = s()
    assert b["x"].shape == (4, 2) and b["y"].tolist() == [0, 0, 0, 1]


def test_collate_pads_on_the_left_and_keeps_lengths():
    from eagersgd_b200.data import collate_sequences
    seqs = [np.full((2, 3), 1.0, np.float32), np.full((4, 3), 2.0, np.float32), np.full((1, 3), 3.0, np.float32)]
    b = collate_sequences(seqs, np.array([7, 8, 9]))
    assert b["x"].shape == (3, 4, 3) and b["lengths"].tolist() == [2, 4, 1] and b["y"].tolist() == [7, 8, 9]
    assert (b["x"][0, :2] == 0).all() and (b["x"][0, 2:] == 1).all() and (b["x"][2, :3] == 0).all() and (b["x"][2, 3] == 3).all()
    frames = collate_sequences([np.ones((2, 3, 4, 4), np.uint8), np.ones((3, 3, 4, 4), np.uint8)], np.array([0, 1]))
    assert frames["x"].shape == (2, 3, 3, 4, 4) and frames["x"].dtype == np.uint8 and frames["x"][0, 0].sum() == 0


def test_choice_sampler_draws_with_replacement_and_shards_tile_the_dataset():
    from eagersgd_b200.data import ChoiceSampler, NumpyDataset, PartitionedDataset, partition
    ds = NumpyDataset(np.arange(10, dtype=np.float32).reshape(10, 1), "x", np.arange(10), "y")
    s = ChoiceSampler(ds, 64, seed=3)
    assert len(s) == 0 and s() is None                           # an epoch is len // batch draws: none here
    s = ChoiceSampler(ds, 5, seed=3)
    batches = []
    while True:
        b = s()
        if b is None:
            break
        batches.append(b["y"])
    assert len(batches) == 2 and all(len(b) == 5 for b in batches)
    many = ChoiceSampler(NumpyDataset(np.zeros((4, 1), np.float32), "x", np.arange(4), "y"), 4, seed=0)
    drew_repeat = False
    for _ in range(20):
        many.reset()
        drew_repeat |= len(set(many()["y"].tolist())) < 4
    assert drew_repeat
    shards = [partition(ds, r, 3) for r in range(3)]
    assert [len(p) for p in shards] == [3, 3, 4]                  # the last shard takes the remainder
    assert np.concatenate([p[:]["y"] for p in shards]).tolist() == list(range(10))
    assert isinstance(shards[1], PartitionedDataset) and shards[1][0]["y"] == 3 and shards[1][[2, 0]]["y"].tolist() == [5, 3]
    assert shards[0].data_node == "x" and shards[0].label_node == "y"


def test_logger_hooks_and_run_info(tmp_path):
    from eagersgd_b200.train import logger as L
    log = L.BenchmarkFileLogger(str(tmp_path))
    hook = L.LoggingMetricHook(log, every_n_iter=3)
    for k in range(7):
        hook.after_step({"loss": 1.0 / (k + 1), "lr": 0.1})
    info = L.gather_run_info("resnet", "synthetic", {"batch_size": 32, "mode": "solo"}, test_id="t1")
    log.log_run_info("resnet", "synthetic", {"batch_size": 32, "mode": "solo"}, test_id="t1")
    with pytest.raises(ValueError):
        with L.benchmark_context(log):
            raise ValueError("boom")
    rows = [json.loads(l) for l in open(tmp_path / "metric.log")]
    assert [(r["name"], r["global_step"]) for r in rows] == [("loss", 3), ("lr", 3), ("loss", 6), ("lr", 6)]
    assert rows[2]["value"] == pytest.approx(1 / 6)
    assert info["model_name"] == "resnet" and info["dataset"] == {"name": "synthetic"} and info["test_id"] == "t1"
    assert {"name": "mode", "value": "solo"} in info["run_parameters"]
    assert info["machine_config"]["cpu_info"]["num_cores"] == os.cpu_count()
    on_disk = json.load(open(tmp_path / "benchmark_run.log"))
    assert on_disk["model_name"] == "resnet" and on_disk["run_parameters"] == info["run_parameters"]
    assert json.load(open(tmp_path / "run_status.log")) == {"run_status": "failure"} and log.status == L.RUN_STATUS_FAILURE
    assert info["machine_config"]["memory_total"] >= info["machine_config"]["memory_available"] > 0
    assert all(v["name"].startswith(("ESGD_", "NCCL_", "CUDA_", "OMP_")) for v in info["environment_variables"])
    assert L.parse_hooks("LoggingTensorHook, examplespersecondhook") == {"LoggingTensorHook", "ExamplesPerSecondHook"}
    with pytest.raises(ValueError, match="unknown hook"):
        L.parse_hooks("nosuchhook")


def test_numpy_oracles_against_torch():
    from eagersgd_b200.ref import numpy_ops as R
    rng = np.random.RandomState(0)
    a, b, c = (rng.randn(3, 4) for _ in range(3))
    np.testing.assert_allclose(R.sum_(a, b, c), a + b + c)
    loss, grad = R.mean_squared_error(a, b)
    ta = torch.tensor(a, requires_grad=True)
    tl = torch.nn.functional.mse_loss(ta, torch.tensor(b))
    tl.backward()
    assert loss == pytest.approx(tl.item()) and np.allclose(grad, ta.grad.numpy())
    H = 5
    cell = torch.nn.LSTMCell(7, H).double()
    x, h0, c0 = torch.randn(2, 7).double(), torch.randn(2, H).double(), torch.randn(2, H).double()
    h1, c1 = cell(x, (h0, c0))
    hn, cn = R.lstm_cell((x @ cell.weight_ih.T).detach().numpy(), (h0 @ cell.weight_hh.T).detach().numpy(),
                         (cell.bias_ih + cell.bias_hh).detach().numpy(), c0.numpy())
    assert np.allclose(hn, h1.detach().numpy()) and np.allclose(cn, c1.detach().numpy())


def test_learning_rate_with_decay_pieces():
    from eagersgd_b200.train.schedule import learning_rate_with_decay
    lr = learning_rate_with_decay(batch_size=64, batch_denom=128, num_images=640, boundary_epochs=[2, 4],
                                  decay_rates=[1, 0.1, 0.01], base_lr=0.2)
    assert lr(0) == pytest.approx(0.1) and lr(19) == pytest.approx(0.1)          # 10 batches an epoch
    assert lr(20) == pytest.approx(0.01) and lr(39) == pytest.approx(0.01) and lr(40) == pytest.approx(0.001)
    warm = learning_rate_with_decay(64, 128, 640, [2, 4], [1, 0.1, 0.01], base_lr=0.2, warmup=True, warmup_epochs=1)
    assert warm(0) == 0 and warm(5) == pytest.approx(0.05) and warm(10) == pytest.approx(0.1)
    resumed = learning_rate_with_decay(64, 128, 640, [2, 4], [1, 0.1, 0.01], base_lr=0.2, start_epoch=3)
    assert resumed(0) == pytest.approx(0.01) and resumed(10) == pytest.approx(0.001)


def test_status_words_segments_and_switches(monkeypatch):
    from eagersgd_b200.parallel import _native as N
    from eagersgd_b200.parallel.cpu_channel import segment_bytes
    from eagersgd_b200.parallel.nvlink_channel import multicast_wanted
    assert N.status_text(0) == "ok"
    bits = list(N.STATUS_BITS)
    assert N.status_text(bits[0]) == N.STATUS_BITS[bits[0]]
    both = N.status_text(bits[0] | bits[-1])
    assert N.STATUS_BITS[bits[0]] in both and N.STATUS_BITS[bits[-1]] in both
    assert str(N.ChannelError(bits[0], "bucket 3")).startswith("partial allreduce failed (bucket 3): ")
    small, large = segment_bytes(1024, np.float32), segment_bytes(4096, np.float32)
    assert large - small >= 3072 * 4 and segment_bytes(1024, np.float64) > small     # slots grow with count and width
    monkeypatch.delenv("ESGD_MULTICAST", raising=False)
    monkeypatch.delenv("NCCL_NVLS_ENABLE", raising=False)
    assert multicast_wanted()
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    assert not multicast_wanted()
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "1")
    monkeypatch.setenv("ESGD_MULTICAST", "0")
    assert not multicast_wanted()


def test_optimizer_harness_with_expected_parameters_and_lbfgs():
    """One step of gradient descent on a linear layer has a closed form; ``test_optimizer`` takes plain dictionaries
    of inputs and compares the parameters after the step with it (deep500/lv2/validation/optimizer.py:29-93).  L-BFGS,
    the one optimizer that needs the loss re-evaluated inside a step, solves the least-squares problem outright."""
    from eagersgd_b200.ops.validation import OneInputDataset, test_optimizer
    from eagersgd_b200.optim.base import GradientDescent, LBFGSOptimizer
    rng = np.random.RandomState(0)
    x, y = rng.randn(8, 6).astype(np.float32), rng.randn(8, 3).astype(np.float32)
    ex = _executor()
    w, b = ex.network.fetch_tensor("weight").copy(), ex.network.fetch_tensor("bias").copy()
    d = 2 * (x @ w.T + b - y) / y.size
    expect = {"weight": w - 0.25 * d.T @ x, "bias": b - 0.25 * d.sum(0)}
    res = test_optimizer(GradientDescent(ex, learning_rate=0.25), ({"x": x}, {"y": y}), expected_params=expect)
    assert res["weight"] < 1e-5 and res["bias"] < 1e-5 and res["loss"] == pytest.approx(float(((x @ w.T + b - y) ** 2).mean()), rel=1e-5)
    with pytest.raises(AssertionError, match="weight"):
        test_optimizer(GradientDescent(_executor(), learning_rate=0.25), {"x": x, "y": y}, expected_params=[w, b])
    with pytest.raises(ValueError):
        test_optimizer(GradientDescent(_executor(), learning_rate=0.25), 3)
    ds = OneInputDataset({"x": x}, {"y": y})
    assert len(ds) == 1 and set(ds[0]) == {"x", "y"} and ds.data_node == "x" and ds.label_node == "y"
    ex2 = _executor()
    opt = LBFGSOptimizer(ex2, learning_rate=1.0, max_iter=50, history_size=20, line_search_fn="strong_wolfe")
    first = opt.step({"x": x, "y": y})
    assert opt.evaluations > 1                                      # the line search re-evaluated the loss
    A = np.concatenate([x, np.ones((8, 1), np.float32)], 1)
    best = float(((A @ np.linalg.lstsq(A, y, rcond=None)[0] - y) ** 2).mean())
    after = float(ex2.inference({"x": x, "y": y})["loss"])
    assert after < float(first["loss"]) and after == pytest.approx(best, abs=1e-4)
    opt.set_parameter("learning_rate", 0.5)
    assert opt.opt.param_groups[0]["lr"] == 0.5


def test_process_wide_logger_and_per_device_batch(tmp_path):
    import types
    from eagersgd_b200.train import logger as L
    from eagersgd_b200.train.model_helpers import per_device_batch_size
    assert isinstance(L.get_benchmark_logger(), L.BaseBenchmarkLogger)
    flags = types.SimpleNamespace(benchmark_logger_type="BenchmarkFileLogger", benchmark_log_dir=str(tmp_path / "logs"))
    log = L.config_benchmark_logger(flags)
    assert isinstance(log, L.BenchmarkFileLogger) and L.get_benchmark_logger() is log
    L.get_benchmark_logger().log_metric("accuracy", 0.5, global_step=3)
    assert json.loads(open(tmp_path / "logs" / "metric.log").readline())["name"] == "accuracy"
    with pytest.raises(ValueError, match="Unrecognized benchmark_logger_type"):
        L.config_benchmark_logger(types.SimpleNamespace(benchmark_logger_type="BenchmarkBigQueryLogger"))
    assert type(L.config_benchmark_logger()) is L.BaseBenchmarkLogger          # back to standard output
    assert per_device_batch_size(256, 1) == 256 and per_device_batch_size(256, 8) == 32
    with pytest.raises(ValueError, match="try --batch_size=96"):
        per_device_batch_size(100, 8)


def test_sampler_harness_with_metrics():
    """d5.test_sampler(sampler, metrics=[...]) as the reference's dataset_latency and mnist_bias samples call it."""
    from eagersgd_b200.data import NumpyDataset, ShuffleSampler
    from eagersgd_b200.ops.validation import test_sampler
    from eagersgd_b200.train import metrics as M
    y = np.repeat(np.arange(4), [10, 20, 30, 4])
    ds = NumpyDataset(np.zeros((64, 2), np.float32), "x", y, "y")
    s = ShuffleSampler(ds, 16, seed=0)
    latency, bias = M.SamplerEventMetric(), M.DatasetBias(4)
    t, hist = test_sampler(s, batches=4, metrics=[latency, bias])
    assert len(latency.times) == 4 and t == latency.measure() and t >= 0
    assert hist.tolist() == [10, 20, 30, 4]                       # one epoch: the data set's own class counts
    assert s.events == []                                          # the metrics were detached again
    assert set(test_sampler(s, batches=3)) == {"median_batch_ms", "distinct_sample_shapes"}
