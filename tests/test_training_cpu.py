"""Trainer, optimizer bases, parity distributed optimizers, schedules, injectors, mains on CPU."""
import math

import numpy as np
import pytest
import torch

from mp_util import run_ranks


def _toy():
    from eagersgd_b200.data import NumpyDataset, ShuffleSampler, OrderedSampler
    rng = np.random.RandomState(0)
    x = rng.randn(512, 16).astype(np.float32)
    w = rng.randn(16, 4).astype(np.float32)
    y = (x @ w).argmax(1).astype(np.int64)
    ds = NumpyDataset(x, "x", y, "y")
    return ds, ShuffleSampler(ds, 32, seed=0), OrderedSampler(ds, 64)


@pytest.mark.parametrize("opt_name", ["GradientDescent", "MomentumOptimizer", "AdamOptimizer", "AdaGradOptimizer", "RMSPropOptimizer"])
def test_trainer_with_reference_update_rules(opt_name):
    from eagersgd_b200.optim import base
    from eagersgd_b200.train.executor import GraphExecutor, classification_loss
    from eagersgd_b200.train.trainer import Trainer
    from eagersgd_b200.train import events as E
    torch.manual_seed(0)
    ds, tr, te = _toy()
    ex = GraphExecutor(torch.nn.Linear(16, 4), classification_loss)
    lr = {"GradientDescent": 0.5, "MomentumOptimizer": 0.1, "AdamOptimizer": 0.05, "AdaGradOptimizer": 0.5, "RMSPropOptimizer": 0.02}[opt_name]
    opt = getattr(base, opt_name)(ex, learning_rate=lr)
    stats = Trainer(tr, te, ex, opt).run_loop(4, [E.SummaryGeneratorEvent(), E.AccuracyAbortEvent(0.999)])
    assert stats.test_summaries[-1].accuracy > 0.85
    assert stats.train_summaries[-1].mean_loss < stats.train_summaries[0].mean_loss


def test_momentum_rule_matches_torch_sgd():
    from eagersgd_b200.optim.base import MomentumOptimizer
    from eagersgd_b200.train.executor import GraphExecutor, mse_loss
    torch.manual_seed(1)
    m1, m2 = torch.nn.Linear(8, 1), torch.nn.Linear(8, 1)
    m2.load_state_dict(m1.state_dict())
    ex = GraphExecutor(m1, lambda o, b: mse_loss(o.squeeze(-1), b))
    opt = MomentumOptimizer(ex, learning_rate=0.05, momentum=0.9)
    ref = torch.optim.SGD(m2.parameters(), lr=0.05, momentum=0.9)
    for k in range(5):
        x, y = torch.randn(16, 8), torch.randn(16)
        opt.step({"x": x, "y": y})
        ref.zero_grad()
        torch.nn.functional.mse_loss(m2(x).squeeze(-1), y).backward()
        ref.step()
    assert torch.allclose(m1.weight, m2.weight, atol=1e-6)


def test_events_and_csv(tmp_path):
    from eagersgd_b200.optim.base import GradientDescent
    from eagersgd_b200.train.executor import GraphExecutor, classification_loss
    from eagersgd_b200.train.trainer import test_training
    from eagersgd_b200.train import events as E
    ds, tr, te = _toy()
    ex = GraphExecutor(torch.nn.Linear(16, 4), classification_loss)
    opt = GradientDescent(ex, learning_rate=0.1)
    sched = E.EpochHPSchedule(learning_rate=lambda e: 0.1 * 0.5 ** e)
    wrongs = E.SaveWrongsEvent()
    stats = test_training(ex, tr, te, opt, 2, [sched, wrongs, E.CsvWriterEvent(str(tmp_path / "s.csv")),
                                              E.LossPlotGeneratorEvent(str(tmp_path / "loss")),
                                              E.TimeAbortAfterTestEvent(1e9)])
    assert opt.hyper["learning_rate"] == pytest.approx(0.05)
    assert (tmp_path / "s.csv").exists() and (tmp_path / "loss.json").exists()
    assert len(wrongs.wrong) == round((1 - stats.test_summaries[-1].accuracy) * 512)


def test_lr_schedules():
    from eagersgd_b200.train.schedule import imagenet_schedule, cifar10_schedule
    from eagersgd_b200.optim.lars import poly_rate_schedule
    f = imagenet_schedule(8192, 1281167)
    bpe = 1281167 / 8192
    assert f(0) == 0.0 and f(int(bpe * 2.5)) == pytest.approx(3.2 * 0.5, rel=1e-2)   # linear warm-up to 0.1*8192/256
    assert f(int(bpe * 10)) == pytest.approx(3.2) and f(int(bpe * 31)) == pytest.approx(0.32)
    assert f(int(bpe * 95)) == pytest.approx(3.2e-4)
    g = cifar10_schedule(128)
    assert g(0) == pytest.approx(0.1) and g(int(50000 / 128 * 100)) == pytest.approx(0.01)
    assert poly_rate_schedule(0, batch_size=8192) == 0 and poly_rate_schedule(90, batch_size=8192, train_epochs=90) == 0


def test_injectors_agree_across_ranks():
    from eagersgd_b200.train.imbalance import FixedRanksSleep, ExponentialDelays, RandomRankFactor
    a, b = FixedRanksSleep(8, 0.32, 2, seed=5), FixedRanksSleep(8, 0.32, 2, seed=5)
    for _ in range(20):
        assert a.delays() == b.delays()
    d = ExponentialDelays(8, 0.1, 0.5, 2, seed=1).delays()
    assert sum(1 for v in d if v > 0) in (1, 2) and max(d) <= 0.5
    d = RandomRankFactor(4, 0.2, 1.5, seed=0).delays()
    assert sorted(d) == [0, 0, 0, pytest.approx(0.3)]


def test_lars_trust_ratio():
    from eagersgd_b200.optim.lars import LARS
    w = torch.nn.Parameter(torch.ones(4, 4) * 2.0)
    b = torch.nn.Parameter(torch.ones(4))
    opt = LARS([w, b], lr=1.0, momentum=0.0, weight_decay=0.0, eeta=0.1)
    w.grad, b.grad = torch.ones(4, 4), torch.ones(4)
    opt.step()
    trust = 0.1 * (2.0 * 4) / 4.0                      # eeta * ||w|| / ||g||
    assert torch.allclose(w, torch.full((4, 4), 2.0 - trust))
    assert torch.allclose(b, torch.zeros(4))           # 1-D tensors are not adapted: plain lr


def _parity(rank, world, name):
    import eagersgd_b200 as es
    from eagersgd_b200.optim import base, distributed as D
    from eagersgd_b200.train.executor import GraphExecutor, mse_loss
    g = es.init(backend="gloo")
    torch.manual_seed(0)
    m = torch.nn.Linear(8, 1)
    ex = GraphExecutor(m, lambda o, b: mse_loss(o.squeeze(-1), b))
    opt = getattr(D, name)(base.GradientDescent(ex, learning_rate=0.1), g)
    gen = torch.Generator().manual_seed(3)
    xs, ys = torch.randn(world, 16, 8, generator=gen), torch.randn(world, 16, generator=gen)
    if name == "InconsistentParameterServer":
        if rank == 0:
            opt.serve(3 * (world - 1))
        else:
            for _ in range(3):
                opt.step({"x": xs[rank], "y": ys[rank]})
        out = m.weight.detach().clone()
    else:
        for _ in range(3):
            opt.step({"x": xs[rank], "y": ys[rank]})
        out = m.weight.detach().clone()
    g.barrier()
    es.finalize()
    return out.tolist()   # plain lists travel safely through the result queue


@pytest.mark.parametrize("name", ["ConsistentDecentralized", "HorovodStyleOptimizer", "ConsistentParameterServer",
                                  "ModelAverageDecentralized", "ConsistentNeighbors", "InconsistentParameterServer"])
def test_parity_distributed_optimizers(name):
    world = 3
    outs = [torch.tensor(o) for o in run_ranks(_parity, world, (name,))]
    if name in ("ConsistentDecentralized", "HorovodStyleOptimizer", "ConsistentParameterServer",
                "ModelAverageDecentralized", "ConsistentNeighbors"):
        for o in outs[1:]:
            assert torch.allclose(o, outs[0], atol=1e-6)   # world 3: ring neighbours cover everyone
    if name in ("ConsistentDecentralized", "HorovodStyleOptimizer", "ConsistentParameterServer"):
        torch.manual_seed(0)
        m = torch.nn.Linear(8, 1)
        gen = torch.Generator().manual_seed(3)
        xs, ys = torch.randn(world, 16, 8, generator=gen), torch.randn(world, 16, generator=gen)
        ref = torch.optim.SGD(m.parameters(), lr=0.1)
        for _ in range(3):
            ref.zero_grad()
            torch.nn.functional.mse_loss(m(xs.view(-1, 8)).squeeze(-1), ys.view(-1)).backward()
            ref.step()
        assert torch.allclose(outs[0], m.weight.detach(), atol=1e-5)
    if name == "InconsistentParameterServer":
        assert torch.isfinite(outs[0]).all() and not torch.allclose(outs[0], outs[0] * 0)


def test_resnet_main_smoke(tmp_path):
    from eagersgd_b200.train import resnet_main
    rc = resnet_main.main(["--dataset", "cifar10", "--synthetic", "--synthetic_train_size", "64", "-rs", "8", "-bs", "16",
                           "--train_epochs", "1", "--max_train_steps", "3", "--mode", "solo", "--dtype", "fp32",
                           "--model_dir", str(tmp_path / "m"), "--export_dir", str(tmp_path / "e"),
                           "--train_acc_steps", "2", "--benchmark_logger_type", "BenchmarkFileLogger",
                           "--benchmark_log_dir", str(tmp_path / "log")])
    assert rc == 0
    assert (tmp_path / "m" / "0" / "checkpoint").exists()
    z = np.load(tmp_path / "e" / "model.npz")
    assert "resnet_model/conv2d/kernel" in z and "resnet_model/dense/bias" in z
    assert (tmp_path / "log" / "metric.log").exists()
    from eagersgd_b200.graph import GraphNetwork, load_onnx          # the exported inference graph loads and runs
    net = GraphNetwork(load_onnx(str(tmp_path / "e" / "model.onnx"))).eval()
    with torch.no_grad():
        out = net(torch.randn(2, 3, 32, 32))
    out = out[0] if isinstance(out, (list, tuple)) else out
    assert out.shape == (2, 10) and torch.isfinite(out).all()


def test_flags_that_change_behaviour(tmp_path):
    """--hooks (profiler trace), --fine_tune (only the dense layer moves), --virtual_batch_size (ghost batch
    norm) and --batchaug (replicated batch) are read by the run loop, not just parsed."""
    import numpy as np
    import torch
    from eagersgd_b200.models.resnet import BatchNormAct, cifar_resnet
    from eagersgd_b200.train.logger import ProfilerHook, parse_hooks
    assert parse_hooks("profilerhook, ExamplesPerSecondHook") == {"ProfilerHook", "ExamplesPerSecondHook"}
    with pytest.raises(ValueError):
        parse_hooks("NoSuchHook")
    hook = ProfilerHook(str(tmp_path), save_steps=2, first_step=1)
    for step in range(3):
        with hook.step(step):
            torch.randn(8, 8) @ torch.randn(8, 8)
    assert len(hook.written) == 2 and all(p.endswith(".json") for p in hook.written)
    # ghost batch norm: statistics per group of 2 samples differ from statistics over the batch of 4
    torch.manual_seed(0)
    bn = BatchNormAct(4)
    x = torch.randn(4, 4, 3, 3) * torch.tensor([1.0, 2.0, 3.0, 4.0]).view(4, 1, 1, 1)
    full = bn(x, relu=False)
    bn.virtual_batch_size = 2
    ghost = bn(x, relu=False)
    assert not torch.allclose(full, ghost)
    ref = torch.cat([torch.nn.functional.batch_norm(x[i:i + 2], None, None, bn.weight, bn.bias, True, 0.0, bn.eps)
                     for i in (0, 2)])
    assert torch.allclose(ghost, ref, atol=1e-5)
    # the main program with --fine_tune leaves everything but the dense layer untouched
    from eagersgd_b200.train import resnet_main
    before = cifar_resnet(8, 1, 10)
    torch.manual_seed(0)
    rc = resnet_main.main(["--dataset", "cifar10", "--synthetic", "--synthetic_train_size", "8", "--resnet_size", "8",
                           "--batch_size", "4", "--max_train_steps", "2", "--train_epochs", "1", "--dtype", "fp32",
                           "--model_dir", str(tmp_path / "md"), "--fine_tune", "--batchaug", "2", "--hooks",
                           "ExamplesPerSecondHook", "--baseseed", "0"])
    assert rc == 0
    state = torch.load(str(tmp_path / "md" / "0" / "ckpt-2.pt"), weights_only=False)["model"]
    torch.manual_seed(0)
    fresh = cifar_resnet(8, 1, 10).state_dict()
    moved = [k for k in fresh if fresh[k].dtype.is_floating_point and "running" not in k and not torch.equal(fresh[k], state[k])]
    assert moved and all(k.startswith("fc.") for k in moved), moved


def test_dataset_accuracy_metric():
    """Accuracy of a model over a sampler, measured on demand."""
    import numpy as np
    from eagersgd_b200.train.metrics import DatasetAccuracy
    xs = np.eye(4, dtype=np.float32)
    batches = [(torch.from_numpy(xs[:2]), torch.tensor([0, 1])), (torch.from_numpy(xs[2:]), torch.tensor([2, 0]))]
    model = torch.nn.Linear(4, 4, bias=False)
    with torch.no_grad():
        model.weight.copy_(torch.eye(4))
    assert DatasetAccuracy(batches).measure(model) == 0.75
    assert DatasetAccuracy(batches, max_batches=1).measure(model) == 1.0


def test_update_rule_optimizer_of_the_tutorial():
    """The optimizer written in docs/custom_optimizer.md: one overridden method, driven by an executor."""
    from eagersgd_b200.optim.base import UpdateRuleOptimizer
    from eagersgd_b200.train.executor import GraphExecutor, classification_loss

    class SignSGD(UpdateRuleOptimizer):
        def __init__(self, executor, loss="loss", learning_rate=0.01):
            super().__init__(executor, loss)
            self.hyper["learning_rate"] = learning_rate

        def update_rule(self, grad, old_param, name):
            return old_param - self.hyper["learning_rate"] * grad.sign()

    torch.manual_seed(0)
    opt = SignSGD(GraphExecutor(torch.nn.Linear(4, 2), loss_fn=classification_loss))
    batch = {"x": torch.randn(8, 4), "y": torch.randint(0, 2, (8,))}
    first = float(opt.step(batch)["loss"])
    for _ in range(30):
        last = float(opt.step(batch)["loss"])
    assert last < first


def test_model_helpers_and_the_synthetic_integration_run(tmp_path):
    from eagersgd_b200.train import resnet_main
    from eagersgd_b200.train.model_helpers import (MockBenchmarkLogger, apply_clean, generate_synthetic_data,
                                                   past_stop_threshold, run_synthetic)
    assert not past_stop_threshold(None, 0.9) and past_stop_threshold(0.5, 0.5) and not past_stop_threshold(0.5, 0.4)
    with pytest.raises(ValueError):
        past_stop_threshold("high", 0.1)
    it = generate_synthetic_data((2, 3), 1.5, label_shape=(2,), label_value=7, batches=3)
    batches = list(it)
    assert len(batches) == 3 and torch.all(batches[0][0] == 1.5) and torch.all(batches[2][1] == 7)
    d = tmp_path / "m"
    d.mkdir()
    (d / "x").write_text("1")
    apply_clean(False, str(d))
    assert d.exists()
    apply_clean(True, str(d))
    assert not d.exists()
    log = MockBenchmarkLogger()
    log.log_evaluation_result({"accuracy": 0.5, "global_step": 3})
    assert log.logged_metric == [{"name": "accuracy", "value": 0.5, "unit": None, "global_step": 3, "extras": None}]
    rc = run_synthetic(resnet_main.main, str(tmp_path), ["--dataset", "cifar10", "-rs", "8", "-bs", "8", "--dtype", "fp32",
                                                          "--synthetic_train_size", "16"], max_train=1)
    assert rc == 0 and [p for p in tmp_path.iterdir() if p.is_dir()] == []      # the scratch directory is gone


def test_shuffleaug_groups_share_data_and_regime_moves_the_boundaries():
    """--shuffleaug 2 on four ranks: ranks 0,1 and ranks 2,3 read the same samples in the same order, the two groups
    different halves of the data; --regime selects the ImageNet learning-rate boundaries."""
    from types import SimpleNamespace
    from eagersgd_b200.train import resnet_main
    from eagersgd_b200.train import flags as F
    from eagersgd_b200.train.schedule import imagenet_schedule
    p = F.build_parser("t")
    p.add_argument("--synthetic_train_size", type=int, default=None)
    args = F.resolve(p.parse_args(["--synthetic", "--synthetic_train_size", "64", "-bs", "4", "--shuffleaug", "2"]))
    args.dataset = "cifar10"
    info = dict(resnet_main.DATASETS["cifar10"])
    firsts = []
    for rank in range(4):
        train, _ = resnet_main.build_data(args, info, SimpleNamespace(rank=rank, world=4))
        b = next(iter(train))
        x, y = (b["x"], b["y"]) if isinstance(b, dict) else b
        firsts.append((len(train.dataset), np.asarray(y).tolist(), float(np.asarray(x, dtype=np.float64).sum())))
    assert firsts[0] == firsts[1] and firsts[2] == firsts[3] and firsts[0] != firsts[2]
    assert firsts[0][0] == 32                                   # two groups: half of the 64 samples each
    lr0, lr2 = imagenet_schedule(256, 2560, warmup=False), imagenet_schedule(256, 2560, warmup=False, regime=2)
    steps = 2560 // 256                                         # batches per epoch
    assert lr0(steps * 16) == pytest.approx(0.1) and lr2(steps * 16) == pytest.approx(0.01)


def test_update_rule_optimizers_follow_torch_optim_over_random_hyperparameters():
    """Property test: the update-rule optimizers (gradient descent, momentum with weight decay, Adam, AdaGrad,
    RMSProp) take the same six steps as their torch.optim counterparts from the same start, for random
    hyper-parameters."""
    from hypothesis import HealthCheck, given, settings
    from hypothesis import strategies as st
    from eagersgd_b200.optim import base as B
    from eagersgd_b200.train.executor import GraphExecutor, classification_loss

    lr = st.floats(1e-3, 0.5)

    @settings(max_examples=30, deadline=None, suppress_health_check=[HealthCheck.too_slow])
    @given(kind=st.sampled_from(["gd", "momentum", "adam", "adagrad", "rmsprop"]), lr=lr, a=st.floats(0.5, 0.99),
           b=st.floats(0.9, 0.9999), wd=st.sampled_from([0.0, 1e-3, 1e-1]), seed=st.integers(0, 10 ** 6))
    def check(kind, lr, a, b, wd, seed):
        torch.manual_seed(seed)
        m1 = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.Tanh(), torch.nn.Linear(7, 3))
        m2 = torch.nn.Sequential(torch.nn.Linear(5, 7), torch.nn.Tanh(), torch.nn.Linear(7, 3))
        m2.load_state_dict(m1.state_dict())
        ex = GraphExecutor(m1, loss_fn=classification_loss)
        ours, theirs = {
            "gd": lambda: (B.GradientDescent(ex, learning_rate=lr), torch.optim.SGD(m2.parameters(), lr=lr)),
            "momentum": lambda: (B.MomentumOptimizer(ex, learning_rate=lr, momentum=a, weight_decay=wd),
                                 torch.optim.SGD(m2.parameters(), lr=lr, momentum=a, weight_decay=wd)),
            "adam": lambda: (B.AdamOptimizer(ex, learning_rate=lr * 0.1, beta1=a, beta2=b, epsilon=1e-8),
                             torch.optim.Adam(m2.parameters(), lr=lr * 0.1, betas=(a, b), eps=1e-8)),
            "adagrad": lambda: (B.AdaGradOptimizer(ex, learning_rate=lr, epsilon=1e-10),
                                torch.optim.Adagrad(m2.parameters(), lr=lr, eps=1e-10)),
            "rmsprop": lambda: (B.RMSPropOptimizer(ex, learning_rate=lr * 0.1, decay=a, epsilon=1e-8),
                                torch.optim.RMSprop(m2.parameters(), lr=lr * 0.1, alpha=a, eps=1e-8)),
        }[kind]()
        g = torch.Generator().manual_seed(seed)
        for _ in range(6):
            x, y = torch.randn(8, 5, generator=g), torch.randint(0, 3, (8,), generator=g)
            ours.step({"x": x, "y": y})
            theirs.zero_grad()
            torch.nn.functional.cross_entropy(m2(x), y).backward()
            theirs.step()
        for p, q in zip(m1.parameters(), m2.parameters()):
            assert torch.allclose(p, q, rtol=1e-4, atol=1e-5), (kind, (p - q).abs().max())

    check()


def test_weight_decay_skips_normalisation_layers_when_asked():
    """The reference's ImageNet objective keeps the batch-norm variables out of its L2 term
    (resnet_run_loop_solo_imagenet_300.py:328-339), its CIFAR-10 objective includes them (cifar10_main.py:244-250).
    With a loss that has no gradient only weight decay moves the weights, which shows who is decayed."""
    import eagersgd_b200 as es
    from eagersgd_b200.models import cifar_resnet
    from eagersgd_b200.train.resnet_main import DATASETS
    from eagersgd_b200.train.step import TrainStep
    assert DATASETS["imagenet"]["wd"] == DATASETS["cifar10"]["wd"] == 1e-4
    assert DATASETS["imagenet"]["decay_norm"] is False and DATASETS["cifar10"]["decay_norm"] is True
    x, y = torch.randn(4, 3, 32, 32), torch.zeros(4, dtype=torch.long)
    ddp = TrainStep(cifar_resnet(8), es.Group(), impl="ddp", weight_decay=0.1, compute_dtype=torch.float32, decay_norm_params=False)
    assert [(g["weight_decay"], len(g["params"])) for g in ddp.opt.param_groups] == [(0.1, 12), (0.0, 20)]   # the plain arm too
    for decay_norm, impl in ((False, "ours"), (True, "ours")):
        torch.manual_seed(0)
        step = TrainStep(cifar_resnet(8), es.Group(), impl=impl, mode="sync", lr=0.5, momentum=0.0, weight_decay=0.1,
                         compute_dtype=torch.float32, loss_fn=lambda out, t: out.sum() * 0.0, decay_norm_params=decay_norm)
        bn = next(m for m in step.model.modules() if isinstance(m, torch.nn.BatchNorm2d))
        g0, w0 = bn.weight.detach().clone(), step.model.stem.weight.detach().clone()
        step.run_device(x, y)
        assert torch.allclose(step.model.stem.weight, w0 * (1 - 0.5 * 0.1), atol=1e-6)       # convolutions are always decayed
        if decay_norm:
            assert torch.allclose(bn.weight, g0 * (1 - 0.5 * 0.1), atol=1e-6)
        else:
            assert torch.equal(bn.weight, g0)
        if hasattr(step.opt, "close"):
            step.opt.close()


def test_main_program_defaults_follow_the_data_set(monkeypatch):
    """Without -rs / -te / -ebe the CIFAR-10 program is ResNet-32 for 190 epochs evaluated every 10
    (cifar10_main.py:274-279), the ImageNet one ResNet-50 for 90 epochs evaluated after each."""
    from eagersgd_b200.train import resnet_main
    seen = {}

    class Stop(Exception):
        pass

    def fake_build_model(args, info):
        seen[args.dataset] = (args.resnet_size, args.train_epochs, args.epochs_between_evals)
        raise Stop()
    monkeypatch.setattr(resnet_main, "build_model", fake_build_model)
    for ds in ("cifar10", "imagenet"):
        with pytest.raises(Stop):
            resnet_main.main(["--dataset", ds, "--synthetic"])
    assert seen == {"cifar10": (32, 190, 10), "imagenet": (50, 90, 1)}
    with pytest.raises(Stop):
        resnet_main.main(["--dataset", "cifar10", "--synthetic", "-rs", "56", "-te", "3", "-ebe", "2"])
    assert seen["cifar10"] == (56, 3, 2)
