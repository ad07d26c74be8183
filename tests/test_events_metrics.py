"""Events and metrics of the training loop: every class does what its name says, on CPU.

The reference's counterparts are deep500/lv2/events/*.py (terminal bar, time aborts, hyper-parameter
schedules, plot generators) and deep500/lv0..lv3 metrics (norm errors, heatmaps, accuracies, sampler time,
communication volume)."""
import io
import json
import time

import numpy as np
import pytest
import torch


def _toy(events=None):
    from eagersgd_b200.data import NumpyDataset, OrderedSampler, ShuffleSampler
    rng = np.random.RandomState(0)
    x = rng.randn(256, 16).astype(np.float32)
    w = rng.randn(16, 4).astype(np.float32)
    y = (x @ w).argmax(1).astype(np.int64)
    ds = NumpyDataset(x, "x", y, "y")
    return ds, ShuffleSampler(ds, 32, seed=0, events=events), OrderedSampler(ds, 64)


def _trainer(lr=0.1, events=None):
    from eagersgd_b200.optim.base import GradientDescent
    from eagersgd_b200.train.executor import GraphExecutor, classification_loss
    from eagersgd_b200.train.trainer import Trainer
    torch.manual_seed(0)
    ds, tr, te = _toy(events)
    ex = GraphExecutor(torch.nn.Linear(16, 4), classification_loss)
    opt = GradientDescent(ex, learning_rate=lr)
    return Trainer(tr, te, ex, opt), opt


def test_terminal_bar_prints_one_line_per_epoch():
    from eagersgd_b200.train import events as E
    out = io.StringIO()
    tr, _ = _trainer()
    stats = tr.run_loop(2, [E.SummaryGeneratorEvent(), E.TerminalBarEvent(out)])
    lines = [l for l in out.getvalue().replace("\r", "\n").split("\n") if l.startswith("epoch ") and "loss" in l and "train-acc" in l]
    assert len(lines) == 2
    assert lines[1].startswith("epoch 1: loss %.4f" % stats.train_summaries[1].mean_loss)


def test_time_abort_immediate_stops_inside_the_epoch():
    from eagersgd_b200.train import events as E
    tr, _ = _trainer()
    ev = E.TimeAbortImmediateEvent(-1.0)                       # the budget is already used up
    stats = tr.run_loop(3, [ev])
    assert len(stats.train_summaries) == 1 and len(stats.train_summaries[0].losses) == 1
    assert len(stats.test_summaries) == 1                       # only the pass before training ran
    tr2, _ = _trainer()
    after = E.TimeAbortAfterTestEvent(-1.0)                     # the same budget, checked after a test pass only
    s2 = tr2.run_loop(3, [after])
    assert len(s2.train_summaries) == 0 and len(s2.test_summaries) == 1


def test_step_schedule_sets_the_rate_before_every_step():
    from eagersgd_b200.train import events as E
    seen = []

    class Spy(E.TrainingEvent):
        def after_optimizer_step(self, executor, optimizer, loss):
            seen.append(optimizer.hyper["learning_rate"])

    tr, opt = _trainer()
    tr.run_loop(2, [E.StepHPSchedule(learning_rate=lambda k: 0.1 / (1 + k)), Spy()])
    assert seen == pytest.approx([0.1 / (1 + k) for k in range(16)])   # 8 steps an epoch, the count runs on


def test_box_plot_quartiles(tmp_path):
    from eagersgd_b200.train import events as E
    tr, _ = _trainer()
    stats = tr.run_loop(2, [E.BoxPlotGeneratorEvent(str(tmp_path / "box"))])
    q = json.load(open(tmp_path / "box.json"))["loss_quartiles_per_epoch"]
    assert len(q) == 2
    for quart, s in zip(q, stats.train_summaries):
        assert quart[0] == pytest.approx(min(s.losses)) and quart[4] == pytest.approx(max(s.losses))
        assert quart[2] == pytest.approx(float(np.median(s.losses)))
        assert quart == sorted(quart)


def test_norm_errors_and_heatmaps():
    from eagersgd_b200.train import metrics as M
    a = torch.tensor([[1.0, -2.0], [3.0, 4.0]])
    b = np.array([[0.0, 0.0], [0.0, 1.0]])
    assert M.L1Error().measure(None, a, b) == pytest.approx(9.0)
    assert M.L2Error().measure(None, a, b) == pytest.approx(np.sqrt(1 + 4 + 9 + 9))
    assert M.MaxError().measure(None, a, b) == pytest.approx(3.0)
    assert M.MaxError().measure(None, a.bfloat16(), b) == pytest.approx(3.0)     # low-precision outputs are widened
    np.testing.assert_allclose(M.DiffHeatmap().measure(None, a, b), [[1, 2], [3, 3]])
    v = M.VarHeatmap()
    for k in range(4):
        var = v.measure(None, torch.full((2, 3), float(k)))
    np.testing.assert_allclose(var, np.full((2, 3), np.var([0, 1, 2, 3])))


def test_accuracy_metrics_accumulate_over_batches():
    from eagersgd_b200.train import metrics as M
    for cls in (M.TrainingAccuracy, M.TestAccuracy):
        m = cls()
        assert m.measure() == 0.0
        m.update(torch.tensor([[0.1, 0.9], [0.8, 0.2]]), torch.tensor([1, 1]))
        m.update(np.array([[0.3, 0.7], [0.3, 0.7], [0.9, 0.1]]), [1, 1, 0])
        assert m.measure() == pytest.approx(4 / 5)
    l = torch.tensor([[0.1, 0.5, 0.4], [0.7, 0.2, 0.1]])
    assert M.topk_accuracy(l, torch.tensor([2, 1]), ks=(1, 2)) == pytest.approx([0.0, 1.0])


def test_sampler_event_metric_times_every_draw():
    from eagersgd_b200.train import metrics as M
    m = M.SamplerEventMetric()
    bias = M.DatasetBias(4)
    assert m.measure() is None
    ds, tr, _ = _toy([m])
    n = 0
    while True:
        b = tr()
        if b is None:
            break
        bias.update(b["y"])
        n += 1
    assert n == 8 and len(m.times) in (8, 9)                    # the draw that finds the epoch over may be timed too
    assert 0 <= m.measure() < 1.0
    labels = np.concatenate([ds[i]["y"].reshape(-1) for i in range(len(ds))])
    assert (bias.measure() == np.bincount(labels, minlength=4)).all()      # one epoch saw every sample once


def test_wallclock_time_takes_the_median_of_reruns():
    from eagersgd_b200.train import metrics as M
    w = M.WallclockTime(reruns=5, avg_over=1, device=torch.device("cpu"))
    t = w.time_callable(lambda: time.sleep(0.002), warmup=1)
    assert 1.5 < t < 50 and w.measure() == pytest.approx(t) and len(w.times) == 5       # milliseconds


def test_communication_metrics_follow_the_optimizer_counters():
    import eagersgd_b200 as es
    from eagersgd_b200.train import metrics as M
    torch.manual_seed(0)
    m = torch.nn.Linear(8, 4)
    o = es.SoloAllreduceOptimizer(torch.optim.SGD(m.parameters(), lr=0.1), es.Group())
    try:
        for _ in range(2):                                      # steps before begin() are not counted
            o.zero_grad(); m(torch.randn(2, 8)).sum().backward(); o.step()
        vol, prof = M.CommunicationVolume(o), M.CommProfiling(o)
        vol.begin(); prof.begin()
        for _ in range(3):
            o.zero_grad(); m(torch.randn(2, 8)).sum().backward(); o.step()
        prof.end()
        r = vol.measure()
        per_round = sum(b.count for b in o.buckets) * 4
        assert r["steps"] == 3 and r["bytes_published"] == 3 * per_round and per_round >= 36 * 4
        assert r["bytes_read_from_peers"] == 0                  # one rank: nothing crosses
        assert 0 <= prof.measure() < 1000
    finally:
        o.close()


def test_inference_summary_event_times_forward_passes_and_steps():
    from eagersgd_b200.optim.base import GradientDescent
    from eagersgd_b200.train import events as E
    from eagersgd_b200.train.executor import GraphExecutor, classification_loss
    from eagersgd_b200.train.trainer import Trainer
    torch.manual_seed(0)
    ds, tr, te = _toy()
    ev = E.SummaryGeneratorInferenceEvent()
    ex = GraphExecutor(torch.nn.Linear(16, 4), classification_loss, events=[ev])      # the executor's hooks time the forward
    stats = Trainer(tr, te, ex, GradientDescent(ex, learning_rate=0.1)).run_loop(2, [ev])
    for s in stats.train_summaries:
        assert len(s.losses) == len(s.time_used_inference) == len(s.time_used_optimizing) == 8
        assert all(0 < a <= b for a, b in zip(s.time_used_inference, s.time_used_optimizing))   # a step contains its forward
    assert all(s.time_used_optimizing == [] for s in stats.test_summaries)


def test_norm_difference_over_lists_and_orders():
    from eagersgd_b200.train import metrics as M
    a, b = np.array([3.0, -4.0]), np.zeros(2)
    assert M.NormDifference(2).measure(None, a, b) == pytest.approx(5.0)
    assert M.NormDifference(1).measure(None, a, b) == pytest.approx(7.0)
    assert M.NormDifference(np.inf).measure(None, a, b) == pytest.approx(4.0)
    assert M.L2Error().measure(None, [a, 2 * a], [b, b]) == pytest.approx([5.0, 10.0])
    with pytest.raises(ValueError):
        M.L1Error().measure(None, [a], [b, b])
    assert isinstance(M.MaxError(), M.NormDifference) and M.MaxError().ord == np.inf


def test_default_event_and_metric_sets():
    from eagersgd_b200.ops.validation import DefaultOpMetrics, DefaultOptimizerMetrics, DefaultTrainingMetrics
    from eagersgd_b200.train import events as E, metrics as M
    from eagersgd_b200.train.trainer import DefaultTrainerEvents
    assert [type(m) for m in DefaultOpMetrics()] == [M.L2Error, M.MaxError, M.DiffHeatmap, M.WallclockTime]
    assert [type(m) for m in DefaultOptimizerMetrics()] == [M.L2Error, M.WallclockTime]
    assert [type(m) for m in DefaultTrainingMetrics()] == [M.TrainingAccuracy, M.TestAccuracy]
    out = io.StringIO()
    ev = DefaultTrainerEvents(1, out)
    assert len(ev) == 1 and isinstance(ev[0], E.TerminalBarEvent)
    tr, _ = _trainer()
    tr.run_loop(1, ev)
    assert "epoch 0: loss" in out.getvalue()


def test_schedules_given_as_lists_of_positions_and_values():
    """EpochHPSchedule(lr=[(0, 1e-1), (81, 1e-2), ...]) as the reference's recipes write it."""
    from eagersgd_b200.train import events as E
    seen = []

    class Spy(E.TrainingEvent):
        def after_optimizer_step(self, executor, optimizer, loss):
            seen.append((optimizer.hyper["learning_rate"], optimizer.hyper.get("momentum")))

    from eagersgd_b200.optim.base import MomentumOptimizer
    from eagersgd_b200.train.executor import GraphExecutor, classification_loss
    from eagersgd_b200.train.trainer import Trainer
    ds, tr, te = _toy()
    ex = GraphExecutor(torch.nn.Linear(16, 4), classification_loss)
    opt = MomentumOptimizer(ex, learning_rate=1.0, momentum=0.5)
    sched = E.EpochHPSchedule(learning_rate=[(2, 0.01), (0, 0.1), (1, 0.05)])            # any order
    per_step = E.StepHPSchedule(momentum=[(4, 0.9)])                                        # silent before step 4
    assert isinstance(sched, E.HyperparameterSchedule) and sched.per_epoch and not per_step.per_epoch
    Trainer(tr, te, ex, opt).run_loop(3, [sched, per_step, Spy()])
    assert [lr for lr, _ in seen] == [0.1] * 8 + [0.05] * 8 + [0.01] * 8
    assert [m for _, m in seen] == [0.5] * 4 + [0.9] * 20


def test_accuracy_metrics_as_events_read_the_summaries():
    """TestAccuracy(max_acc=True) in a trainer's event list, as the reference's recipes use it."""
    from eagersgd_b200.train import metrics as M
    tr, _ = _trainer(lr=0.5)
    last, best, train = M.TestAccuracy(), M.TestAccuracy(max_acc=True), M.TrainingAccuracy()
    stats = tr.run_loop(3, [last, best, train])
    accs = [s.accuracy for s in stats.test_summaries]
    assert last.measure() == accs[-1] and best.measure() == max(accs) and best.measure() >= last.measure()
    assert train.measure() == stats.train_summaries[-1].accuracy
    assert M.TestAccuracy().measure() == 0.0


def test_test_training_takes_data_sets_and_metrics(tmp_path):
    """d5.test_training(executor, training_set, validation_set, optimizer, epochs, batch_size, ..., metrics, events)."""
    from eagersgd_b200.optim.base import GradientDescent
    from eagersgd_b200.train import events as E, metrics as M
    from eagersgd_b200.train.executor import GraphExecutor, classification_loss
    from eagersgd_b200.train.trainer import test_training
    torch.manual_seed(0)
    ds, _, _ = _toy()
    ex = GraphExecutor(torch.nn.Linear(16, 4), classification_loss)
    acc = M.TestAccuracy(max_acc=True)
    stats = test_training(ex, ds, ds, GradientDescent(ex, learning_rate=0.5), epochs=2, batch_size=32, metrics=[acc],
                          events=[E.CsvWriterEvent("run.csv", str(tmp_path)), E.LossPlotGeneratorEvent("loss", str(tmp_path))])
    assert len(stats.train_summaries) == 2 and len(stats.train_summaries[0].losses) == 8
    assert acc.measure() == max(s.accuracy for s in stats.test_summaries) > 0.5
    assert (tmp_path / "run.csv").exists() and (tmp_path / "loss.json").exists()


def test_communication_volume_as_an_event_finds_the_eager_optimizer():
    """metrics = d5.DefaultTrainingMetrics() + [d5.CommunicationVolume()] handed to test_training, as the reference's
    distributed sample does."""
    import eagersgd_b200 as es
    from eagersgd_b200.ops.validation import DefaultTrainingMetrics
    from eagersgd_b200.optim.base import TorchOptimizer
    from eagersgd_b200.train import metrics as M
    from eagersgd_b200.train.executor import from_model
    from eagersgd_b200.train.trainer import test_training
    torch.manual_seed(0)
    ds, _, _ = _toy()
    model = torch.nn.Linear(16, 4)
    ex = from_model(model, torch.device("cpu"))
    eager = es.SoloAllreduceOptimizer(torch.optim.SGD(model.parameters(), lr=0.1), es.Group())
    try:
        vol = M.CommunicationVolume()
        assert vol.measure()["steps"] == 0
        metrics = DefaultTrainingMetrics() + [vol]
        test_training(ex, ds, ds, TorchOptimizer(ex, eager), 1, 32, metrics=metrics)
        assert vol.opt is eager and vol.measure()["steps"] == 8 and vol.measure()["bytes_published"] > 0
        assert 0 < metrics[1].measure() <= 1.0
    finally:
        eager.close()


def test_statistics_tables():
    tr, _ = _trainer()
    stats = tr.run_loop(2, [])
    train_rows, test_rows = stats.to_dict()
    assert [r["epoch"] for r in train_rows] == [0, 1] and [r["epoch"] for r in test_rows] == [-1, 0, 1]
    assert train_rows[0]["n_batches"] == 8 and train_rows[0]["train"] and not test_rows[0]["train"]
    assert train_rows[1]["total_used_time"] == pytest.approx(train_rows[0]["time_used"] + train_rows[1]["time_used"])
    assert train_rows[1]["avg_loss"] == pytest.approx(stats.train_summaries[1].mean_loss)
    stats.clear()
    assert stats.to_dict() == ([], [])


def test_every_hook_of_the_reference_event_interface_fires():
    """before / after_training_set, before / after_test_batch and on_sampler_reset (deep500/lv2/event.py) beside the
    epoch, step and test-set hooks."""
    from eagersgd_b200.train import events as E
    calls = []

    class Recorder(E.TrainingEvent):
        def before_training_set(self, runner, stats, sampler): calls.append("train_set+")
        def after_training_set(self, runner, stats): calls.append("train_set-")
        def before_test_batch(self, runner, stats, batch): calls.append("test_batch+")
        def after_test_batch(self, runner, stats, outputs): calls.append("test_batch-")
        def on_sampler_reset(self, sampler): calls.append("reset")
        def before_epoch(self, epoch, runner, stats): calls.append("epoch+")
        def after_epoch(self, epoch, runner, stats): calls.append("epoch-")

    rec = Recorder()
    tr, _ = _trainer(events=[rec])                 # the training sampler knows the event too
    tr.run_loop(1, [rec])
    assert calls.count("test_batch+") == calls.count("test_batch-") == 8                 # two test passes of four batches
    i = calls.index("epoch+")
    assert calls[i:i + 3] == ["epoch+", "train_set+", "reset"] and calls.index("train_set-") < calls.index("epoch-")
