"""Fused bias + ReLU (+ pooling) kernels of the convolution blocks (`csrc/kernels/model_ops.cu`,
`bagua_core_b200/ops/fused_conv.py`): the CUDA kernels against their host restatement and against
plain fp32 PyTorch math, the modules under autocast, and the fused VGG-16 against the unfused one."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("rows,C", [(1, 8), (37, 64), (1000, 128), (4099, 256), (32 * 14 * 14, 512), (3, 2048)])
def test_bias_relu_forward_and_backward_match_fp32_math(rows, C):
    import bagua_core_b200 as bb

    g = torch.Generator().manual_seed(rows + C)
    z = torch.randn(rows, C, generator=g).to(torch.bfloat16).cuda()
    bias = torch.randn(C, generator=g).to(torch.bfloat16).cuda()
    ref = torch.relu(z.float() + bias.float())
    y = z.clone()
    bb._C.k_bias_relu_(y, bias, _stream())
    assert torch.allclose(y.float(), ref, rtol=8e-3, atol=8e-3)
    assert torch.equal(y > 0, ref.to(torch.bfloat16) > 0)

    dy = torch.randn(rows, C, generator=g).to(torch.bfloat16).cuda()
    dz = torch.empty_like(dy)
    db = torch.empty(C, device="cuda")
    bb._C.k_bias_relu_backward(dy, y, dz, db, _stream())
    dz_ref = torch.where(y > 0, dy, torch.zeros_like(dy))
    assert torch.equal(dz, dz_ref)
    db_ref = dz_ref.double().sum(0)
    assert torch.allclose(db.double(), db_ref, rtol=1e-4, atol=1e-3 * max(1.0, rows ** 0.5))
    # bit-reproducible
    db2 = torch.empty_like(db)
    bb._C.k_bias_relu_backward(dy, y, torch.empty_like(dy), db2, _stream())
    assert torch.equal(db, db2)


def test_channels_last_activation_is_accepted_and_nchw_rejected():
    import bagua_core_b200 as bb

    z = torch.randn(4, 64, 6, 5).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    bias = torch.randn(64).to(torch.bfloat16).cuda()
    ref = torch.relu(z.float() + bias.float().view(1, -1, 1, 1))
    bb._C.k_bias_relu_(z, bias, _stream())
    assert torch.allclose(z.float(), ref, rtol=8e-3, atol=8e-3)
    with pytest.raises(RuntimeError, match="channels-last"):
        bb._C.k_bias_relu_(torch.zeros(4, 64, 6, 5, dtype=torch.bfloat16, device="cuda"), bias, _stream())


@pytest.mark.parametrize("shape", [(1, 8, 2, 2), (2, 64, 6, 10), (3, 128, 56, 56), (32, 512, 14, 14)])
def test_maxpool2x2_matches_torch_bit_for_bit(shape):
    from bagua_core_b200.ops.fused_conv import MaxPool2x2

    g = torch.Generator().manual_seed(sum(shape))
    # values on a coarse grid so that windows contain ties; half of them clamped to zero like a ReLU output
    x = torch.relu((torch.randn(*shape, generator=g) * 4).round() / 4).to(torch.bfloat16).cuda()
    x = x.contiguous(memory_format=torch.channels_last)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ya = MaxPool2x2()(xa)
    yb = torch.nn.functional.max_pool2d(xb, 2, 2)
    assert ya.is_contiguous(memory_format=torch.channels_last)
    assert torch.equal(ya, yb)
    go = torch.randn(ya.shape, generator=g).to(torch.bfloat16).cuda().contiguous(memory_format=torch.channels_last)
    ya.backward(go)
    yb.backward(go)
    assert torch.equal(xa.grad, xb.grad)


def test_maxpool2x2_falls_back_for_odd_sizes_and_fp32():
    from bagua_core_b200.ops.fused_conv import MaxPool2x2

    for x in (torch.randn(2, 8, 5, 7, device="cuda").to(torch.bfloat16).contiguous(memory_format=torch.channels_last),
              torch.randn(2, 8, 4, 4, device="cuda")):
        assert torch.equal(MaxPool2x2()(x), torch.nn.functional.max_pool2d(x, 2, 2))


def test_conv_bias_relu_module_matches_conv_plus_relu_under_autocast():
    from bagua_core_b200.ops.fused_conv import ConvBiasReLU

    torch.manual_seed(0)
    fused = ConvBiasReLU(16, 64, 3, padding=1).cuda().to(memory_format=torch.channels_last)
    plain = torch.nn.Conv2d(16, 64, 3, padding=1).cuda().to(memory_format=torch.channels_last)
    plain.load_state_dict(fused.state_dict())
    x = torch.randn(8, 16, 20, 20, device="cuda").contiguous(memory_format=torch.channels_last)
    xa = x.clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        ya = fused(xa)
        yb = torch.relu(plain(x))
    assert ya.dtype == torch.bfloat16 and torch.allclose(ya.float(), yb.float(), rtol=2e-2, atol=2e-2)
    # Backward against fp32 math on the forward's own ReLU mask and on the bf16-rounded operands
    # (a few masks differ between two bf16 forwards, so another bf16 backward is not a sharp reference).
    go = torch.randn_like(ya)
    ya.backward(go)
    dz = torch.where(ya > 0, go, torch.zeros_like(go)).float()
    w16, x16 = fused.weight.detach().to(torch.bfloat16).float(), x.to(torch.bfloat16).float()
    refs = [torch.nn.grad.conv2d_input(x.shape, w16, dz, padding=1), torch.nn.grad.conv2d_weight(x16, w16.shape, dz, padding=1),
            dz.sum((0, 2, 3))]
    for got, ref in zip([xa.grad, fused.weight.grad, fused.bias.grad], refs):
        assert got.dtype == torch.float32 and got.shape == ref.shape
        scale = ref.abs().max().item() + 1e-6
        assert (got - ref).abs().max().item() <= 1.5e-2 * scale


def test_fused_vgg16_step_matches_unfused():
    from bagua_core_b200.models import VGG16

    torch.manual_seed(1)
    a = VGG16(num_classes=10, dropout=0.0, fused_ops=True).cuda().to(memory_format=torch.channels_last)
    b = VGG16(num_classes=10, dropout=0.0).cuda().to(memory_format=torch.channels_last)
    for pa, pb in zip(a.parameters(), b.parameters()):
        pb.data.copy_(pa.data)
    x = torch.randn(4, 3, 64, 64, device="cuda").contiguous(memory_format=torch.channels_last)
    t = torch.randint(0, 10, (4,), device="cuda")
    losses = []
    for m in (a, b):
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(m(x).float(), t)
        loss.backward()
        losses.append(loss.item())
    assert abs(losses[0] - losses[1]) <= 2e-2 * max(1.0, abs(losses[1]))
    for pa, pb in zip(a.parameters(), b.parameters()):
        scale = pb.grad.abs().max().item() + 1e-6
        assert (pa.grad - pb.grad).abs().max().item() <= 0.2 * scale  # ReLU masks flip here and there between two bf16 runs


@pytest.mark.parametrize("shape", [(1, 8, 2, 2), (2, 64, 6, 10), (4, 128, 28, 28), (32, 512, 14, 14), (8, 64, 56, 56)])
def test_cuda_kernels_match_the_host_restatement_exactly(shape):
    """Every model kernel on the GPU against the same binding on CPU tensors (plain loops)."""
    import bagua_core_b200 as bb

    C = bb._C
    n, c, h, w = shape
    g = torch.Generator().manual_seed(sum(shape))

    def rnd(*s, relu=False):
        t = (torch.randn(*s, generator=g) * 4).round() / 4
        t = torch.relu(t) if relu else t
        t = t.to(torch.bfloat16)
        return t.contiguous(memory_format=torch.channels_last) if t.dim() == 4 else t

    s = _stream()
    # bias + ReLU
    z, bias = rnd(n, c, h, w), rnd(c)
    z_h, z_d = z.clone(), z.cuda()
    C.k_bias_relu_(z_h, bias, 0)
    C.k_bias_relu_(z_d, bias.cuda(), s)
    assert torch.equal(z_d.cpu(), z_h)
    dy = rnd(n, c, h, w)
    dz_h, db_h = torch.empty_like(dy), torch.empty(c)
    dz_d, db_d = torch.empty_like(dy).cuda(), torch.empty(c, device="cuda")
    C.k_bias_relu_backward(dy, z_h, dz_h, db_h, 0)
    C.k_bias_relu_backward(dy.cuda(), z_d, dz_d, db_d, s)
    assert torch.equal(dz_d.cpu(), dz_h)
    assert torch.allclose(db_d.cpu(), db_h, rtol=1e-4, atol=1e-2)
    # max pooling
    x = rnd(n, c, h, w, relu=True)
    y_h = torch.empty((n, c, h // 2, w // 2), dtype=torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y_d = y_h.cuda()
    C.k_maxpool2x2_forward(x, y_h, 0)
    C.k_maxpool2x2_forward(x.cuda(), y_d, s)
    assert torch.equal(y_d.cpu(), y_h)
    gy = rnd(n, c, h // 2, w // 2)
    dx_h, dx_d = torch.empty_like(x), torch.empty_like(x).cuda()
    C.k_maxpool2x2_backward(x, gy, dx_h, 0)
    C.k_maxpool2x2_backward(x.cuda(), gy.cuda(), dx_d, s)
    assert torch.equal(dx_d.cpu(), dx_h)
    # bias + ReLU + pooling in one pass
    a_h, a_d = z.clone(), z.cuda()
    p_h, p_d = torch.empty_like(y_h), torch.empty_like(y_h).cuda()
    C.k_bias_relu_pool_(a_h, p_h, bias, 0)
    C.k_bias_relu_pool_(a_d, p_d, bias.cuda(), s)
    assert torch.equal(a_d.cpu(), a_h) and torch.equal(p_d.cpu(), p_h)
    dzp_h, dbp_h = torch.empty_like(z), torch.empty(c)
    dzp_d, dbp_d = torch.empty_like(z).cuda(), torch.empty(c, device="cuda")
    C.k_bias_relu_pool_backward(gy, a_h, dzp_h, dbp_h, 0)
    C.k_bias_relu_pool_backward(gy.cuda(), a_d, dzp_d, dbp_d, s)
    assert torch.equal(dzp_d.cpu(), dzp_h)
    assert torch.allclose(dbp_d.cpu(), dbp_h, rtol=1e-4, atol=1e-2)


def test_conv_bias_relu_pool_module_matches_the_composition_under_autocast():
    from bagua_core_b200.ops.fused_conv import ConvBiasReLU, ConvBiasReLUPool

    torch.manual_seed(0)
    pooled = ConvBiasReLUPool(16, 64, 3, padding=1).cuda().to(memory_format=torch.channels_last)
    single = ConvBiasReLU(16, 64, 3, padding=1).cuda().to(memory_format=torch.channels_last)
    single.load_state_dict(pooled.state_dict())
    x = torch.randn(8, 16, 20, 24, device="cuda").contiguous(memory_format=torch.channels_last)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        pa = pooled(xa)
        pb = torch.nn.functional.max_pool2d(single(xb), 2, 2)
    assert torch.allclose(pa.float(), pb.float(), rtol=2e-2, atol=2e-2)  # same math; the library may pick another conv algorithm
    go = torch.randn_like(pa)
    pa.backward(go)
    pb.backward(go)
    for a, b in [(xa.grad, xb.grad), (pooled.weight.grad, single.weight.grad), (pooled.bias.grad, single.bias.grad)]:
        scale = b.abs().max().item() + 1e-6
        assert (a - b).abs().max().item() <= 6e-2 * scale  # masks agree except where two conv algorithms round apart




@pytest.mark.parametrize("n", [1, 7, 4096, (1 << 20) + 3])
def test_sgd_step_with_bf16_copy_equals_the_plain_step(n):
    import bagua_core_b200 as bb

    C = bb._C
    g = torch.Generator().manual_seed(n)
    p, grad = torch.randn(n, generator=g).cuda(), torch.randn(n, generator=g).cuda()
    m = torch.zeros(n, device="cuda")
    p2, m2, h = p.clone(), m.clone(), torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    for step in range(3):
        C.k_sgd_momentum_flat(p, grad, m, 0.1, 0.9, 0.0, 1e-4, True, step == 0, s)
        C.k_sgd_momentum_flat_shadow(p2, grad, m2, h, 0.1, 0.9, 0.0, 1e-4, True, step == 0, s)
        torch.cuda.synchronize()
        assert torch.equal(p, p2) and torch.equal(m, m2) and torch.equal(h, p2.to(torch.bfloat16))
    # an unaligned view takes the scalar path
    if n > 8:
        q = torch.randn(n + 1, generator=g).cuda()[1:]  # 4 bytes past a 16-byte boundary
        q2 = torch.empty(n + 1, device="cuda")[1:].copy_(q)
        hq = torch.zeros(n + 1, dtype=torch.bfloat16, device="cuda")[1:]
        C.k_sgd_momentum_flat(q, grad, m, 0.1, 0.9, 0.0, 0.0, False, False, s)
        C.k_sgd_momentum_flat_shadow(q2, grad, m2, hq, 0.1, 0.9, 0.0, 0.0, False, False, s)
        torch.cuda.synchronize()
        assert torch.equal(q, q2) and torch.equal(hq, q2.to(torch.bfloat16))


def test_vgg_training_with_bf16_weight_copies_is_bit_identical_to_casting():
    """Same model, same data: lookups switched off (the blocks cast the fp32 weights in every forward pass) against
    lookups on (they read the optimizer's copies)."""
    import os

    import bagua_core_b200.parallel as P
    from bagua_core_b200.models import VGG16
    from bagua_core_b200.ops import shadow as S

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29541")
    dev = torch.device("cuda", 0)
    results = []
    for use_copies in (False, True):
        S.enabled = use_copies
        torch.manual_seed(0)
        model = VGG16(num_classes=10, dropout=0.0, fused_ops=True).to(dev).to(memory_format=torch.channels_last)
        P.init_process_group(dev)
        opt = P.FlatSGD(model.parameters(), lr=0.01, momentum=0.9, bf16_shadow=True)
        bm = P.with_bagua(model, [opt], P.GradientAllReduceAlgorithm(), bucket_bytes=10 << 20)
        g = torch.Generator().manual_seed(5)
        hits0, losses = S.hits, []
        for _ in range(4):
            x = torch.randn(4, 3, 64, 64, generator=g).to(dev).contiguous(memory_format=torch.channels_last)
            y = torch.randint(0, 10, (4,), generator=g).to(dev)
            opt.zero_grad()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = torch.nn.functional.cross_entropy(bm(x).float(), y)
            loss.backward()
            opt.step()
            losses.append(loss.item())
        torch.cuda.synchronize()
        results.append((losses, torch.cat([p.detach().reshape(-1) for p in model.parameters()]).clone(), S.hits - hits0))
        P.destroy_process_group()
    S.enabled = True
    assert results[0][2] == 0 and results[1][2] == 3 * 16  # 13 convolutions + 3 linear layers, from the second step on
    assert results[0][0] == results[1][0]
    assert torch.equal(results[0][1], results[1][1])




@pytest.mark.parametrize("rows,n_in,n_out", [(32, 25088, 4096), (32, 4096, 1000), (5, 72, 24)])
def test_linear_weight_gradient_accumulated_in_place_is_the_fp32_product(rows, n_in, n_out):
    """The library GEMM adds dyᵀ x (bf16 operands) into the fp32 gradient; compared with the same
    operands multiplied in fp32 by plain PyTorch, twice in a row (the second call adds)."""
    from bagua_core_b200.ops import wgrad as W
    from bagua_core_b200.ops.fused_linear import ShadowLinear

    saved, W.enabled = W.enabled, True
    try:
        torch.manual_seed(rows + n_in)
        m = ShadowLinear(n_in, n_out).cuda()
        for p in m.parameters():
            p.grad = torch.zeros_like(p)
        fired = []
        m.weight.register_post_accumulate_grad_hook(lambda p: fired.append(1))
        x = torch.randn(rows, n_in, device="cuda")
        a0 = W.accumulated
        for k in (1, 2):
            with torch.autocast("cuda", dtype=torch.bfloat16):
                y = m(x)
            dy = torch.randn_like(y)
            y.backward(dy)
            torch.cuda.synchronize()
            assert W.accumulated == a0 + k and len(fired) == k, (W.accumulated, W.declined, W.cuda_mode)
            want = k * (dy.to(torch.bfloat16).float().t() @ x.to(torch.bfloat16).float()) if k == 1 else want + \
                dy.to(torch.bfloat16).float().t() @ x.to(torch.bfloat16).float()
            scale = want.abs().max().item()
            assert (m.weight.grad - want).abs().max().item() <= 2e-3 * scale + 1e-5
        assert W.cuda_mode in ("addmm", "mm_add")
    finally:
        W.enabled = saved


def test_vgg_training_with_in_place_weight_gradients_agrees_with_the_ordinary_path():
    import os

    import bagua_core_b200.parallel as P
    from bagua_core_b200.models import VGG16
    from bagua_core_b200.ops import wgrad as W

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29543")
    dev = torch.device("cuda", 0)
    saved, results = W.enabled, []
    try:
        for inplace in (False, True):
            W.enabled = inplace
            torch.manual_seed(0)
            model = VGG16(num_classes=10, dropout=0.0, fused_ops=True).to(dev).to(memory_format=torch.channels_last)
            P.init_process_group(dev)
            opt = P.FlatSGD(model.parameters(), lr=0.01, momentum=0.9)
            bm = P.with_bagua(model, [opt], P.GradientAllReduceAlgorithm(), bucket_bytes=10 << 20)
            g = torch.Generator().manual_seed(5)
            a0, losses = W.accumulated, []
            for _ in range(4):
                x = torch.randn(4, 3, 64, 64, generator=g).to(dev).contiguous(memory_format=torch.channels_last)
                y = torch.randint(0, 10, (4,), generator=g).to(dev)
                opt.zero_grad()
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    loss = torch.nn.functional.cross_entropy(bm(x).float(), y)
                loss.backward()
                opt.step()
                losses.append(loss.item())
            torch.cuda.synchronize()
            results.append((losses, torch.cat([p.detach().reshape(-1) for p in model.parameters()]).clone(),
                            W.accumulated - a0))
            P.destroy_process_group()
    finally:
        W.enabled = saved
    assert results[0][2] == 0 and results[1][2] == 4 * 3  # three linear layers, four steps
    assert all(abs(a - b) < 5e-2 for a, b in zip(results[0][0], results[1][0])), (results[0][0], results[1][0])
    assert (results[0][1] - results[1][1]).abs().max().item() < 2e-2
