"""Golden-data tests of the ResNet blocks, one per block type.

The reference keeps, per block type, a serialized graph, a checkpoint and hashes of the results
(official/resnet/layer_test.py:41-204, official/utils/testing/reference_data.py:62-307,
reference_data/resnet/*/results.json) so that a change of the layers' numerics or variable layout is noticed.
Here each case builds the block with weights drawn from a fixed generator, runs it in fp32 on the CPU in training
mode and compares the output's shape, a few statistics and sampled values, the gradient of the input, and the
ordered list of the block's variables (kind and shape) with ``tests/golden/resnet_blocks.json``.
``python tests/test_layer_golden.py --regenerate`` rewrites the file after a deliberate change.
"""
import json
import os
import sys

import pytest
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "resnet_blocks.json")

# name: (kind, version, channels in, filters, stride, projection shortcut)
CASES = {
    "building_v1_identity": ("building", 1, 16, 16, 1, False),
    "building_v1_projection": ("building", 1, 16, 32, 2, True),
    "building_v2_identity": ("building", 2, 16, 16, 1, False),
    "building_v2_projection": ("building", 2, 16, 32, 2, True),
    "bottleneck_v1_identity": ("bottleneck", 1, 64, 16, 1, False),
    "bottleneck_v1_projection": ("bottleneck", 1, 32, 16, 2, True),
    "bottleneck_v2_identity": ("bottleneck", 2, 64, 16, 1, False),
    "bottleneck_v2_projection": ("bottleneck", 2, 32, 16, 2, True),
}


def _run(name):
    from eagersgd_b200.models.resnet import _Block
    kind, version, cin, filters, stride, project = CASES[name]
    gen = torch.Generator().manual_seed(sum(map(ord, name)))
    registry = []
    block = _Block(cin, filters, stride, kind, version, project, registry).train()
    with torch.no_grad():
        for p in block.parameters():                  # every parameter from the fixed generator, zero-gammas too
            p.copy_(torch.randn(p.shape, generator=gen) * (0.2 if p.dim() > 1 else 0.5) + (1.0 if p.dim() == 1 else 0.0))
    x = torch.randn(2, cin, 8, 8, generator=gen, requires_grad=True)
    y = block(x)
    y.square().mean().backward()
    flat, gflat = y.detach().flatten(), x.grad.flatten()
    pick = torch.linspace(0, flat.numel() - 1, 7).long()
    gpick = torch.linspace(0, gflat.numel() - 1, 5).long()
    return {
        "variables": [[k, list(m.weight.shape)] for k, m in registry],
        "output_shape": list(y.shape),
        "output_mean": float(flat.mean()), "output_std": float(flat.std()), "output_absmax": float(flat.abs().max()),
        "output_samples": [float(v) for v in flat[pick]],
        "input_grad_norm": float(gflat.norm()), "input_grad_samples": [float(v) for v in gflat[gpick]],
    }


@pytest.mark.parametrize("name", sorted(CASES))
def test_block_matches_golden_data(name):
    with open(GOLDEN) as f:
        want = json.load(f)[name]
    got = _run(name)
    assert got["variables"] == want["variables"], "the block's variables changed (kind / order / shape)"
    assert got["output_shape"] == want["output_shape"]
    for key in ("output_mean", "output_std", "output_absmax", "input_grad_norm"):
        assert got[key] == pytest.approx(want[key], rel=1e-4, abs=1e-6), key
    for key in ("output_samples", "input_grad_samples"):
        assert got[key] == pytest.approx(want[key], rel=1e-4, abs=1e-5), key


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    if "--regenerate" in sys.argv:
        os.makedirs(os.path.dirname(GOLDEN), exist_ok=True)
        with open(GOLDEN, "w") as f:
            json.dump({n: _run(n) for n in sorted(CASES)}, f, indent=1)
        print("wrote", GOLDEN)
