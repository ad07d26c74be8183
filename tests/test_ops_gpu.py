"""Hand-written NHWC kernels against plain PyTorch fp32 references of the same ops."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _cl(x):
    return x.contiguous(memory_format=torch.channels_last)


@pytest.mark.parametrize("n,c,h,w,cout", [(4, 64, 14, 14, 256), (2, 256, 7, 9, 64), (8, 128, 28, 28, 512)])
def test_conv1x1_forward_backward(n, c, h, w, cout):
    from eagersgd_b200.ops import functional as ops
    torch.manual_seed(0)
    x = _cl(torch.randn(n, c, h, w, device=DEV)).to(torch.bfloat16).requires_grad_()
    wt = (torch.randn(cout, c, 1, 1, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
    y, stats = ops.conv1x1(x, wt, want_stats=True)
    g = _cl(torch.randn(n, cout, h, w, device=DEV)).to(torch.bfloat16)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), wt.detach().float().requires_grad_()
    yr = F.conv2d(xr, wr)
    yr.backward(g.float())
    assert torch.allclose(y.float(), yr, rtol=2e-2, atol=2e-2)
    assert torch.allclose(stats[0], yr.sum((0, 2, 3)), rtol=1e-2, atol=0.5)
    assert torch.allclose(stats[1], (yr * yr).sum((0, 2, 3)), rtol=1e-2, atol=0.5)
    assert torch.allclose(x.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)
    assert torch.allclose(wt.grad.float(), wr.grad, rtol=2e-2, atol=2e-2 * wr.grad.abs().max().item())


@pytest.mark.parametrize("relu,residual", [(True, False), (False, False), (True, True)])
@pytest.mark.parametrize("c", [64, 264, 2048])
def test_bn_act(relu, residual, c):
    from eagersgd_b200.ops import functional as ops
    torch.manual_seed(1)
    n, h, w = 4, 6, 5
    y = _cl(torch.randn(n, c, h, w, device=DEV) * 2 + 0.5).to(torch.bfloat16).requires_grad_()
    res = _cl(torch.randn(n, c, h, w, device=DEV)).to(torch.bfloat16).requires_grad_() if residual else None
    gamma = (torch.rand(c, device=DEV) + 0.5).requires_grad_()
    beta = torch.randn(c, device=DEV).requires_grad_()
    rm, rv = torch.zeros(c, device=DEV), torch.ones(c, device=DEV)
    z = ops.bn_act(y, gamma, beta, rm, rv, 0.1, relu, res)
    g = _cl(torch.randn(n, c, h, w, device=DEV)).to(torch.bfloat16)
    z.backward(g)
    yr = y.detach().float().requires_grad_()
    rr = res.detach().float().requires_grad_() if residual else None
    gr, br = gamma.detach().clone().requires_grad_(), beta.detach().clone().requires_grad_()
    rm2, rv2 = torch.zeros(c, device=DEV), torch.ones(c, device=DEV)
    zr = F.batch_norm(yr, rm2, rv2, gr, br, True, 0.1, 1e-5)
    if residual:
        zr = zr + rr
    if relu:
        zr = zr.relu()
    zr.backward(g.float())
    assert torch.allclose(z.float(), zr, rtol=2e-2, atol=3e-2)
    assert torch.allclose(rm, rm2, rtol=1e-3, atol=1e-3) and torch.allclose(rv, rv2, rtol=1e-3, atol=1e-3)
    assert torch.allclose(y.grad.float(), yr.grad, rtol=5e-2, atol=5e-2)
    assert torch.allclose(gamma.grad, gr.grad, rtol=5e-2, atol=0.3)
    assert torch.allclose(beta.grad, br.grad, rtol=5e-2, atol=0.3)
    if residual:
        assert torch.allclose(res.grad.float(), rr.grad, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("b,c", [(32, 1000), (7, 10), (256, 1001)])
def test_softmax_cross_entropy(dtype, b, c):
    from eagersgd_b200.ops import functional as ops
    torch.manual_seed(2)
    logits = (torch.randn(b, c, device=DEV) * 3).to(dtype).requires_grad_()
    labels = torch.randint(0, c, (b,), device=DEV)
    loss = ops.softmax_cross_entropy(logits, labels)
    (loss * 2.0).backward()
    lr = logits.detach().float().requires_grad_()
    ref = F.cross_entropy(lr, labels)
    (ref * 2.0).backward()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    assert abs(loss.item() - ref.item()) < 1e-4 * max(1.0, abs(ref.item())) + tol
    assert torch.allclose(logits.grad.float(), lr.grad, rtol=tol * 10, atol=tol)


@pytest.mark.parametrize("h,w", [(8, 8), (7, 9), (112, 112)])
def test_max_pool(h, w):
    from eagersgd_b200.ops import functional as ops
    torch.manual_seed(3)
    x = _cl(torch.randn(2, 64, h, w, device=DEV)).relu().to(torch.bfloat16).requires_grad_()  # many ties at zero
    y = ops.max_pool_3x3_s2(x)
    g = _cl(torch.randn_like(y.float())).to(torch.bfloat16)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = F.max_pool2d(xr, 3, 2, 1)
    yr.backward(g.float())
    assert torch.equal(y.float(), yr)
    assert torch.allclose(x.grad.float(), xr.grad, rtol=1e-2, atol=2e-2)


def test_global_avg_pool():
    from eagersgd_b200.ops import functional as ops
    x = _cl(torch.randn(4, 2048, 7, 7, device=DEV)).to(torch.bfloat16).requires_grad_()
    y = ops.global_avg_pool(x)
    g = torch.randn(4, 2048, device=DEV).to(torch.bfloat16)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = xr.mean((2, 3))
    yr.backward(g.float())
    assert torch.allclose(y.float(), yr, rtol=1e-2, atol=1e-2)
    assert torch.allclose(x.grad.float(), xr.grad, rtol=1e-2, atol=1e-3)


def test_linear_layer():
    from eagersgd_b200.ops import functional as ops
    torch.manual_seed(4)
    x = torch.randn(64, 2048, device=DEV).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(1000, 2048, device=DEV) * 0.02).to(torch.bfloat16).requires_grad_()
    b = torch.randn(1000, device=DEV).to(torch.bfloat16).requires_grad_()
    y = ops.linear(x, w, b)
    g = torch.randn(64, 1000, device=DEV)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = F.linear(xr, wr, br)
    yr.backward(g)
    assert y.dtype == torch.float32 and torch.allclose(y, yr, rtol=1e-2, atol=2e-2)
    assert torch.allclose(x.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)
    assert torch.allclose(w.grad.float(), wr.grad, rtol=2e-2, atol=0.2)
    assert torch.allclose(b.grad.float(), br.grad, rtol=2e-2, atol=0.1)


def test_resnet_native_matches_references():
    """Whole model: native bf16 NHWC kernels vs (a) the same bf16 model through PyTorch ops and
    (b) fp32 PyTorch.  The bf16-vs-fp32 gap of PyTorch's own ops calibrates the tolerance."""
    import copy
    from eagersgd_b200.models.resnet import imagenet_resnet
    from eagersgd_b200.ops import functional as ops
    from eagersgd_b200.train.step import prepare_model
    torch.manual_seed(5)
    ref = imagenet_resnet(18, 1, 1000).to(DEV)
    for m in ref.modules():  # give the zero-initialised gammas a value so every branch carries signal
        if isinstance(m, torch.nn.BatchNorm2d):
            torch.nn.init.uniform_(m.weight, 0.5, 1.0)
    nat = prepare_model(copy.deepcopy(ref), torch.device(DEV))
    tor = copy.deepcopy(nat)
    x = torch.randn(32, 3, 96, 96, device=DEV)
    y = torch.randint(0, 1000, (32,), device=DEV)
    F.cross_entropy(ref(x), y).backward()
    xb = _cl(x).to(torch.bfloat16)
    ln = ops.softmax_cross_entropy(nat(xb), y)
    ln.backward()
    with ops.reference_ops():
        lt = ops.softmax_cross_entropy(tor(xb), y)
        lt.backward()
    flat = lambda m: torch.cat([p.grad.float().flatten() for p in m.parameters()])
    g32, gn, gt = flat(ref), flat(nat), flat(tor)
    cos_nt = F.cosine_similarity(gn, gt, dim=0).item()
    cos_t32 = F.cosine_similarity(gt, g32, dim=0).item()
    cos_n32 = F.cosine_similarity(gn, g32, dim=0).item()
    print("cos native/torch-bf16 %.4f torch-bf16/fp32 %.4f native/fp32 %.4f" % (cos_nt, cos_t32, cos_n32))
    assert abs(ln.item() - lt.item()) < 0.05 * abs(lt.item())
    assert cos_n32 > min(0.97, cos_t32 - 0.03), (cos_nt, cos_t32, cos_n32)


def test_bottleneck_block_matches_reference_ops():
    """One bottleneck block with projection and stride (all conv paths of ResNet-50)."""
    import copy
    from eagersgd_b200.models.resnet import _Block
    from eagersgd_b200.ops import functional as ops
    torch.manual_seed(6)
    blk = _Block(64, 32, 2, "bottleneck", 1, True, []).to(DEV)
    for m in blk.modules():
        if isinstance(m, torch.nn.BatchNorm2d):
            torch.nn.init.uniform_(m.weight, 0.5, 1.0)
        if isinstance(m, torch.nn.Conv2d):
            m.to(torch.bfloat16)
    blk2 = copy.deepcopy(blk)
    x = _cl(torch.randn(8, 64, 16, 16, device=DEV)).to(torch.bfloat16)
    x1, x2 = x.clone().requires_grad_(), x.clone().requires_grad_()
    g = _cl(torch.randn(8, 128, 8, 8, device=DEV)).to(torch.bfloat16)
    z1 = blk(x1)
    z1.backward(g)
    with ops.reference_ops():
        z2 = blk2(x2)
        z2.backward(g)
    assert torch.allclose(z1.float(), z2.float(), rtol=5e-2, atol=5e-2)
    assert F.cosine_similarity(x1.grad.float().flatten(), x2.grad.float().flatten(), dim=0).item() > 0.99
    for (n1, p1), (_, p2) in zip(blk.named_parameters(), blk2.named_parameters()):
        c = F.cosine_similarity(p1.grad.float().flatten(), p2.grad.float().flatten(), dim=0).item()
        assert c > 0.98, (n1, c)


@pytest.mark.parametrize("T,B,I,H", [(5, 16, 64, 128), (12, 8, 256, 256), (6, 16, 512, 1024), (3, 40, 64, 128)])
def test_lstm_layer_forward_backward(T, B, I, H):
    from eagersgd_b200.ops.lstm import lstm_layer, lstm_layer_reference
    torch.manual_seed(7)
    x = (torch.randn(T, B, I, device=DEV) * 0.5).to(torch.bfloat16).requires_grad_()
    k = 1.0 / H ** 0.5
    w_ih = torch.empty(4 * H, I, device=DEV).uniform_(-k, k).to(torch.bfloat16).requires_grad_()
    w_hh = torch.empty(4 * H, H, device=DEV).uniform_(-k, k).to(torch.bfloat16).requires_grad_()
    bias = (torch.randn(4 * H, device=DEV) * 0.1).requires_grad_()
    y = lstm_layer(x, w_ih, w_hh, bias)
    g = torch.randn(T, B, H, device=DEV).to(torch.bfloat16)
    y.backward(g)
    xr, wi, wh, br = (t.detach().float().requires_grad_() for t in (x, w_ih, w_hh, bias))
    yr = lstm_layer_reference(xr, wi, wh, br)
    yr.backward(g.float())
    assert torch.allclose(y.float(), yr, rtol=3e-2, atol=3e-2)
    for a, b_, name in ((x.grad, xr.grad, "dx"), (w_ih.grad, wi.grad, "dw_ih"), (w_hh.grad, wh.grad, "dw_hh"),
                        (bias.grad, br.grad, "db")):
        cos = F.cosine_similarity(a.float().flatten(), b_.flatten(), dim=0).item()
        assert cos > 0.99, (name, cos)
        assert (a.float() - b_).abs().max().item() < 0.05 * b_.abs().max().item() + 5e-2, name


def test_conv1x1_tapped_input_adds_shortcut_gradient_in_the_gemm():
    """The shortcut's gradient reaches x through the tapped output and is added in the data-gradient GEMM."""
    from eagersgd_b200.ops import functional as ops
    torch.manual_seed(3)
    n, c, h, w, cout = 4, 256, 14, 14, 64
    x = _cl(torch.randn(n, c, h, w, device=DEV)).to(torch.bfloat16).requires_grad_()
    wt = (torch.randn(cout, c, 1, 1, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_()
    y, stats, tap = ops.conv2d(x, wt, 1, 0, want_stats=True, tap_input=True)
    assert tap.data_ptr() == x.data_ptr() and stats is not None
    g = _cl(torch.randn(n, cout, h, w, device=DEV)).to(torch.bfloat16)
    g2 = _cl(torch.randn(n, c, h, w, device=DEV)).to(torch.bfloat16)
    torch.autograd.backward([y, tap], [g, g2])
    xr, wr = x.detach().float().requires_grad_(), wt.detach().float().requires_grad_()
    F.conv2d(xr, wr).backward(g.float())
    ref = xr.grad + g2.float()
    assert torch.allclose(x.grad.float(), ref, rtol=2e-2, atol=3e-2)
    assert torch.allclose(wt.grad.float(), wr.grad, rtol=2e-2, atol=2e-2 * wr.grad.abs().max().item())
    # an unused tap costs nothing and changes nothing
    x2 = x.detach().clone().requires_grad_()
    y2, _, _ = ops.conv2d(x2, wt.detach(), 1, 0, want_stats=False, tap_input=True)
    y2.backward(g)
    assert torch.allclose(x2.grad.float(), xr.grad, rtol=2e-2, atol=3e-2)


def test_identity_bottleneck_block_matches_reference_ops():
    import copy
    from eagersgd_b200.models.resnet import _Block
    from eagersgd_b200.ops import functional as ops
    torch.manual_seed(8)
    blk = _Block(256, 64, 1, "bottleneck", 1, False, []).to(DEV)
    for m in blk.modules():
        if isinstance(m, torch.nn.BatchNorm2d):
            torch.nn.init.uniform_(m.weight, 0.5, 1.0)
        if isinstance(m, torch.nn.Conv2d):
            m.to(torch.bfloat16)
    blk2 = copy.deepcopy(blk)
    x = _cl(torch.randn(8, 256, 14, 14, device=DEV)).to(torch.bfloat16)
    x1, x2 = x.clone().requires_grad_(), x.clone().requires_grad_()
    g = _cl(torch.randn(8, 256, 14, 14, device=DEV)).to(torch.bfloat16)
    blk(x1).backward(g)
    with ops.reference_ops():
        blk2(x2).backward(g)
    assert F.cosine_similarity(x1.grad.float().flatten(), x2.grad.float().flatten(), dim=0).item() > 0.995
    rel = (x1.grad.float() - x2.grad.float()).norm() / x2.grad.float().norm()
    assert rel.item() < 0.05, rel.item()


def test_cifar_resnet_step_launches_no_library_convolution_or_gemm():
    """The ResNet-32 training step, narrow 16- and 32-channel layers included, runs its convolutions and
    dense layer on this package's kernels: no cuDNN, cuBLAS or CUTLASS kernel shows up in the profile."""
    import eagersgd_b200 as es
    from eagersgd_b200.models.resnet import cifar_resnet
    from eagersgd_b200.train.step import TrainStep
    torch.manual_seed(0)
    step = TrainStep(cifar_resnet(32, 1, 10), es.Group(), mode="solo", lr=0.05)
    x = _cl(torch.randn(32, 3, 32, 32, device=DEV)).to(torch.bfloat16)
    y = torch.randint(0, 10, (32,), device=DEV)
    l0 = float(step.run_device(x, y))
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            loss = step.run_device(x, y)
        torch.cuda.synchronize()
    names = {e.key for e in prof.key_averages() if getattr(e, "device_time_total", 0) > 0 or "kernel" in e.key.lower()}
    library = [n for n in names if any(t in n.lower() for t in ("cudnn", "cublas", "cutlass", "xmma", "implicit_convolve",
                                                               "sgemm", "gemv", "wgrad", "dgrad"))
               and "conv_wgrad" not in n and "esgd" not in n and "anonymous namespace" not in n]
    assert not library, library
    assert any("conv_kernel" in n or "gemm_kernel" in n for n in names), sorted(names)[:20]
    assert float(loss) < l0          # and it learns the batch
    step.close()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fused_lars_matches_the_per_tensor_reference(dtype):
    """Two launches for all tensors: per-tensor trust ratios, momentum on the scaled gradient, fp32 master
    weights — against the per-tensor PyTorch implementation of the same rule on fp32 copies."""
    from eagersgd_b200.optim.lars import LARS, FusedLARS
    torch.manual_seed(0)
    shapes = [(64, 32, 3, 3), (64,), (10, 64), (10,), (300, 77)]
    ref_params = [torch.nn.Parameter(torch.randn(s, device=DEV) * 0.1) for s in shapes]
    fused_params = [torch.nn.Parameter(p.detach().clone().to(dtype)) for p in ref_params]
    if dtype == torch.bfloat16:
        for p, q in zip(ref_params, fused_params):
            p.data.copy_(q.detach().float())
    ref = LARS(ref_params, lr=0.5, momentum=0.9, weight_decay=1e-3, eeta=0.01)
    fused = FusedLARS(fused_params, lr=0.5, momentum=0.9, weight_decay=1e-3, eeta=0.01)
    for k in range(5):
        fused.zero_grad()
        for p, q in zip(ref_params, fused_params):
            g = torch.randn_like(p).to(dtype)
            p.grad = g.float()
            q.grad.copy_(g)
        ref.step()
        fused.step()
    torch.cuda.synchronize()
    for p, q, off in zip(ref_params, fused_params, fused.offsets):
        master = fused.w32[off:off + p.numel()].view(p.shape)
        assert torch.allclose(master, p.detach(), rtol=2e-4, atol=2e-6), (p.shape, (master - p).abs().max())
        assert torch.equal(q.detach().float(), master.to(dtype).float())


@pytest.mark.parametrize("graph", [False, True])
def test_pipelined_host_loop_gives_the_losses_of_the_plain_one(graph):
    """``run_host_stream`` (next batch copied while the step runs, loss read one step late) returns, in order,
    the losses that ``run_host`` returns for the same batches from the same start."""
    import eagersgd_b200 as es
    from eagersgd_b200.models.resnet import cifar_resnet
    from eagersgd_b200.train.step import TrainStep
    batches = []
    g = torch.Generator().manual_seed(5)
    for _ in range(6):
        x = torch.randn(16, 32, 32, 3, generator=g).permute(0, 3, 1, 2).to(torch.bfloat16).pin_memory()
        batches.append((x, torch.randint(0, 10, (16,), generator=g).pin_memory()))
    out = []
    for stream in (False, True):
        torch.manual_seed(1)
        step = TrainStep(cifar_resnet(8, 1, 10), es.Group(), mode="solo", lr=0.05)
        if graph:
            step.capture(batches[0][0].to(DEV), batches[0][1].to(DEV), warmup=0)
        if stream:
            out.append(list(step.run_host_stream(iter(batches))))
        else:
            out.append([step.run_host(x, y) for x, y in batches])
        step.close()
    assert len(out[1]) == len(batches)
    for a, b in zip(*out):
        assert abs(a - b) <= 2e-2 * max(1.0, abs(a)), out      # fp32 atomics in the weight gradients: not bit-equal
    assert out[0][-1] != out[0][0]


def test_pipelined_host_loop_with_batches_of_changing_shape():
    """Variable-length sequence batches make the loop re-allocate its staging buffers: the early copy of the next
    batch must never land in memory that queued kernels of the running step still use."""
    import eagersgd_b200 as es
    from eagersgd_b200.models import create_model
    from eagersgd_b200.train.step import TrainStep
    g = torch.Generator().manual_seed(3)
    batches = []
    for _ in range(8):
        T = int(torch.randint(5, 60, (1,), generator=g))
        batches.append((torch.randn(16, T, 64, generator=g).to(torch.bfloat16).pin_memory(),
                        torch.randint(0, 7, (16,), generator=g).pin_memory()))
    out = []
    for stream in (True, False):
        torch.manual_seed(0)
        step = TrainStep(create_model("lstm", input_dim=64, hidden=128, layers=2, num_classes=7), es.Group(), mode="solo",
                         lr=0.05)
        out.append(list(step.run_host_stream(iter(batches))) if stream else [step.run_host(x, y) for x, y in batches])
        step.close()
    for a, b in zip(*out):
        assert a == a and abs(a - b) <= 1e-2 * max(1.0, abs(a)), out
