"""Checkpoint layout against the names in the reference's golden ResNet checkpoints."""
import os

import numpy as np
import pytest
import torch

from eagersgd_b200 import ckpt
from eagersgd_b200.models.resnet import _Block, cifar_resnet, imagenet_resnet



def test_resnet50_variable_inventory():
    m = imagenet_resnet(50, 1, 1001)
    names = [n for n, _, _ in ckpt.tf_variables(m)]
    assert names[0] == "resnet_model/conv2d/kernel" and names[1] == "resnet_model/batch_normalization/gamma"
    assert "resnet_model/conv2d_52/kernel" in names and "resnet_model/batch_normalization_52/moving_variance" in names
    assert names[-2:] == ["resnet_model/dense/kernel", "resnet_model/dense/bias"]
    trainable = [n for n, _, k in ckpt.tf_variables(m) if k not in ("mean", "var")]
    assert len(trainable) == 161
    assert sum(t.numel() for _, t, k in ckpt.tf_variables(m) if k not in ("mean", "var")) == 25559081


def test_export_import_roundtrip(tmp_path):
    torch.manual_seed(0)
    m = cifar_resnet(8)
    opt = torch.optim.SGD(m.parameters(), lr=0.1, momentum=0.9)
    m(torch.randn(4, 3, 32, 32)).sum().backward()
    opt.step()
    arrays = ckpt.export_tf_layout(m, str(tmp_path / "model.npz"), opt, global_step=7)
    k = arrays["resnet_model/conv2d/kernel"]
    assert k.shape == (3, 3, 3, 16)  # HWIO
    assert np.allclose(k, m.stem.weight.detach().permute(2, 3, 1, 0).numpy())
    assert arrays["resnet_model/dense/kernel"].shape == (64, 10)
    assert "resnet_model/conv2d/kernel/Momentum" in arrays and arrays["global_step"] == 7
    m2 = cifar_resnet(8)
    step = ckpt.import_tf_layout(m2, str(tmp_path / "model.npz"), exclude=("dense",))
    assert step == 7
    assert torch.equal(m2.stem.weight, m.stem.weight)
    assert not torch.equal(m2.fc.weight, m.fc.weight)      # warm start without the dense layer


def test_per_rank_directories_and_resume(tmp_path):
    m = cifar_resnet(8)
    opt = torch.optim.SGD(m.parameters(), lr=0.1, momentum=0.9)
    d = ckpt.save(m, opt, str(tmp_path), rank=3, global_step=42)
    assert d.endswith(os.path.join(str(tmp_path), "3")) or d.endswith("/3")
    m2 = cifar_resnet(8)
    assert ckpt.load(m2, torch.optim.SGD(m2.parameters(), lr=0.1, momentum=0.9), str(tmp_path), 3) == 42
    assert torch.equal(m2.stem.weight, m.stem.weight)
    assert ckpt.load(m2, None, str(tmp_path), 0) == 0       # another rank has nothing to resume from


# Name fragments readable in the reference's golden block checkpoints
# (official/utils/testing/reference_data/resnet/<config>/model.ckpt.index; the index file
# prefix-compresses keys, so only these full names survive as plain text).
GOLDEN_FRAGMENTS = {
    ("bottleneck", 1, True): ["batch_normalization/beta", "batch_normalization_3/moving_variance", "conv2d/kernel"],
    ("bottleneck", 2, True): ["batch_normalization/beta", "conv2d/kernel", "conv2d_3/kernel"],
    ("bottleneck", 1, False): ["batch_normalization/beta", "conv2d/kernel"],
    ("bottleneck", 2, False): ["batch_normalization/beta", "conv2d/kernel"],
    ("building", 1, True): ["batch_normalization/beta", "conv2d/kernel"],
    ("building", 2, True): ["batch_normalization/beta", "conv2d/kernel"],
    ("building", 1, False): ["batch_normalization/beta", "conv2d/kernel"],
    ("building", 2, False): ["batch_normalization/beta", "conv2d/kernel"],
}
# Highest auto-numbering suffix each block type creates (projection conv/bn are created first).
EXPECTED_LAST = {
    ("bottleneck", 1, True): ("conv2d_3", "batch_normalization_3"),
    ("bottleneck", 2, True): ("conv2d_3", "batch_normalization_2"),
    ("bottleneck", 1, False): ("conv2d_2", "batch_normalization_2"),
    ("bottleneck", 2, False): ("conv2d_2", "batch_normalization_2"),
    ("building", 1, True): ("conv2d_2", "batch_normalization_2"),
    ("building", 2, True): ("conv2d_2", "batch_normalization_1"),
    ("building", 1, False): ("conv2d_1", "batch_normalization_1"),
    ("building", 2, False): ("conv2d_1", "batch_normalization_1"),
}


@pytest.mark.parametrize("cfg", sorted(GOLDEN_FRAGMENTS))
def test_block_names_match_golden_checkpoints(cfg):
    kind, version, projection = cfg

    class Holder(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.registry = []
            self.block = _Block(4, 4, 1, kind, version, projection, self.registry)
    names = [n for n, _, _ in ckpt.tf_variables(Holder(), scope="")]
    for frag in GOLDEN_FRAGMENTS[cfg]:
        assert frag in names, (frag, names)
    last_conv, last_bn = EXPECTED_LAST[cfg]
    assert last_conv + "/kernel" in names and last_bn + "/gamma" in names
    nxt = lambda s: s.rsplit("_", 1)[0] + "_%d" % (int(s.rsplit("_", 1)[1]) + 1)
    assert nxt(last_conv) + "/kernel" not in names and nxt(last_bn) + "/gamma" not in names


def test_rank_directories_become_copies_of_rank_zero(tmp_path):
    """Between two jobs of a chained run (the reference's synchm.sh): ranks 1.. get rank 0's files, stale files go."""
    from eagersgd_b200.ckpt.sync_dirs import main, sync_dirs
    for r in range(3):
        d = tmp_path / str(r)
        d.mkdir()
        (d / "checkpoint").write_text("rank %d" % r)
    (tmp_path / "2" / "stale.bin").write_text("old")
    (tmp_path / "0" / "sub").mkdir()
    (tmp_path / "0" / "sub" / "weights.npz").write_text("w")
    assert sync_dirs(str(tmp_path)) == 2
    for r in (1, 2):
        assert (tmp_path / str(r) / "checkpoint").read_text() == "rank 0"
        assert (tmp_path / str(r) / "sub" / "weights.npz").read_text() == "w"
    assert not (tmp_path / "2" / "stale.bin").exists()
    assert main([str(tmp_path), "--world", "4"]) == 0 and (tmp_path / "3" / "checkpoint").read_text() == "rank 0"
