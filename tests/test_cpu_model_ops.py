"""The fused convolution blocks on CPU tensors: the autograd glue of
`bagua_core_b200/ops/fused_conv.py` (argument order of the aten convolution calls, saved tensors,
gradient routing, channels-last handling) runs against the host restatement of the kernels
(`csrc/kernels/model_ops_cpu.cc`) and is compared with the plain PyTorch composition."""
import pytest
import torch
import torch.nn.functional as F


def _cl(t):
    return t.contiguous(memory_format=torch.channels_last)


def test_host_bias_relu_kernels_match_fp32_math():
    import bagua_core_b200 as bb

    g = torch.Generator().manual_seed(0)
    for rows, C in [(1, 8), (37, 64), (300, 128)]:
        z = torch.randn(rows, C, generator=g).to(torch.bfloat16)
        bias = torch.randn(C, generator=g).to(torch.bfloat16)
        ref = torch.relu(z.float() + bias.float()).to(torch.bfloat16)
        y = z.clone()
        bb._C.k_bias_relu_(y, bias, 0)
        assert torch.equal(y, ref)
        dy = torch.randn(rows, C, generator=g).to(torch.bfloat16)
        dz, db = torch.empty_like(dy), torch.empty(C)
        bb._C.k_bias_relu_backward(dy, y, dz, db, 0)
        dz_ref = torch.where(y > 0, dy, torch.zeros_like(dy))
        assert torch.equal(dz, dz_ref)
        assert torch.allclose(db, dz_ref.float().sum(0), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("shape", [(1, 8, 2, 2), (2, 16, 6, 4), (3, 64, 8, 8)])
def test_maxpool2x2_module_matches_torch_on_cpu(shape):
    from bagua_core_b200.ops.fused_conv import MaxPool2x2, _MaxPool2x2Fn

    g = torch.Generator().manual_seed(sum(shape))
    x = _cl(torch.relu((torch.randn(*shape, generator=g) * 4).round() / 4).to(torch.bfloat16))  # ties and zeros
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ya = _MaxPool2x2Fn.apply(xa)
    assert torch.equal(MaxPool2x2()(x), ya.detach())
    yb = F.max_pool2d(xb, 2, 2)
    assert torch.equal(ya, yb)
    go = _cl(torch.randn(ya.shape, generator=g).to(torch.bfloat16))
    ya.backward(go)
    yb.backward(go)
    assert torch.equal(xa.grad, xb.grad)


def test_conv_bias_relu_function_matches_conv_plus_relu_on_cpu():
    from bagua_core_b200.ops.fused_conv import ConvBiasReLU, _ConvBiasReLUFn

    torch.manual_seed(0)
    fused = ConvBiasReLU(16, 64, 3, padding=1).to(torch.bfloat16).to(memory_format=torch.channels_last)
    plain = torch.nn.Conv2d(16, 64, 3, padding=1).to(torch.bfloat16).to(memory_format=torch.channels_last)
    plain.load_state_dict(fused.state_dict())
    x = _cl(torch.randn(4, 16, 10, 10).to(torch.bfloat16))
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    calls = []
    orig = _ConvBiasReLUFn.apply
    try:
        _ConvBiasReLUFn.apply = staticmethod(lambda *a: calls.append(1) or orig(*a))
        ya = fused(xa)
    finally:
        _ConvBiasReLUFn.apply = orig
    assert calls, "the fused path was not taken"
    yb = torch.relu(plain(xb))
    assert ya.dtype == torch.bfloat16 and ya.shape == yb.shape
    assert torch.allclose(ya.float(), yb.float(), rtol=2e-2, atol=2e-2)
    # The yardstick for the backward is fp32 math on the forward's own ReLU mask (a handful of masks
    # differ between a bf16 and an fp32 forward, and the framework's bf16 CPU backward accumulates in
    # low precision, so neither of those is a sharp reference).
    go = torch.randn_like(ya)
    ya.backward(go)
    dz = torch.where(ya > 0, go, torch.zeros_like(go)).float()
    refs = [torch.nn.grad.conv2d_input(x.shape, fused.weight.detach().float(), dz, padding=1),
            torch.nn.grad.conv2d_weight(x.float(), fused.weight.shape, dz, padding=1),
            dz.sum((0, 2, 3))]
    for got, ref in zip([xa.grad, fused.weight.grad, fused.bias.grad], refs):
        assert got.dtype == torch.bfloat16 and got.shape == ref.shape
        scale = ref.abs().max().item() + 1e-6
        assert (got.float() - ref).abs().max().item() <= 1e-2 * scale


def test_conv_bias_relu_pool_function_on_cpu():
    from bagua_core_b200.ops.fused_conv import ConvBiasReLU, ConvBiasReLUPool

    torch.manual_seed(3)
    pooled = ConvBiasReLUPool(16, 64, 3, padding=1).to(torch.bfloat16).to(memory_format=torch.channels_last)
    single = ConvBiasReLU(16, 64, 3, padding=1).to(torch.bfloat16).to(memory_format=torch.channels_last)
    single.load_state_dict(pooled.state_dict())
    x = _cl(torch.randn(4, 16, 10, 12).to(torch.bfloat16))
    xa = x.clone().requires_grad_(True)
    pa = pooled(xa)
    with torch.no_grad():
        y = single(x)  # the same full-resolution activation the pooled block keeps for its backward
    assert pa.shape == (4, 64, 5, 6) and torch.equal(pa, F.max_pool2d(y, 2, 2))
    # backward against fp32 math on the block's own arg-max and ReLU masks
    go = _cl(torch.randn_like(pa))
    pa.backward(go)
    yy = y.float().requires_grad_(True)
    F.max_pool2d(yy, 2, 2).backward(go.float())
    dz = torch.where(y > 0, yy.grad, torch.zeros_like(yy.grad))
    refs = [torch.nn.grad.conv2d_input(x.shape, pooled.weight.detach().float(), dz, padding=1),
            torch.nn.grad.conv2d_weight(x.float(), pooled.weight.shape, dz, padding=1),
            dz.sum((0, 2, 3))]
    for got, ref in zip([xa.grad, pooled.weight.grad, pooled.bias.grad], refs):
        assert got.dtype == torch.bfloat16 and got.shape == ref.shape
        scale = ref.abs().max().item() + 1e-6
        assert (got.float() - ref).abs().max().item() <= 1e-2 * scale
    # odd output sizes take the plain composition
    x_odd = _cl(torch.randn(2, 16, 9, 9).to(torch.bfloat16))
    assert torch.allclose(pooled(x_odd).float(), F.max_pool2d(single(x_odd), 2, 2).float(), rtol=2e-2, atol=2e-2)


def test_fused_vgg16_matches_unfused_on_cpu_in_bf16():
    from bagua_core_b200.models import VGG16

    torch.manual_seed(1)
    a = VGG16(num_classes=10, dropout=0.0, fused_ops=True).to(torch.bfloat16).to(memory_format=torch.channels_last)
    b = VGG16(num_classes=10, dropout=0.0).to(torch.bfloat16).to(memory_format=torch.channels_last)
    for pa, pb in zip(a.parameters(), b.parameters()):
        pb.data.copy_(pa.data)
    x = _cl(torch.randn(2, 3, 32, 32).to(torch.bfloat16))
    t = torch.randint(0, 10, (2,))
    losses = []
    for m in (a, b):
        loss = F.cross_entropy(m(x).float(), t)
        loss.backward()
        losses.append(loss.item())
    assert abs(losses[0] - losses[1]) <= 3e-2 * max(1.0, abs(losses[1]))
    checked = 0
    for pa, pb in zip(a.parameters(), b.parameters()):
        assert pa.grad is not None and pa.grad.shape == pb.grad.shape
        scale = pb.grad.float().abs().max().item()
        if scale > 0:
            assert (pa.grad.float() - pb.grad.float()).abs().max().item() <= 0.15 * scale + 1e-6
            checked += 1
    assert checked >= 20


def test_fused_blocks_under_cpu_autocast_keep_fp32_parameters_and_gradients():
    """The benchmark's configuration, on the CPU: fp32 parameters and inputs inside a bf16 autocast
    region.  The blocks compute in bf16; weight, bias and input gradients come back in fp32."""
    from bagua_core_b200.ops.fused_conv import ConvBiasReLU, ConvBiasReLUPool

    torch.manual_seed(5)
    for cls, pool in ((ConvBiasReLU, False), (ConvBiasReLUPool, True)):
        fused = cls(8, 32, 3, padding=1).to(memory_format=torch.channels_last)
        plain = torch.nn.Conv2d(8, 32, 3, padding=1).to(memory_format=torch.channels_last)
        plain.load_state_dict(fused.state_dict())
        x = _cl(torch.randn(2, 8, 8, 8))
        xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        with torch.autocast("cpu", dtype=torch.bfloat16):
            ya = fused(xa)
            yb = torch.relu(plain(xb))
            if pool:
                yb = F.max_pool2d(yb, 2, 2)
        assert ya.dtype == torch.bfloat16 and ya.shape == yb.shape
        assert torch.allclose(ya.float(), yb.float(), rtol=3e-2, atol=3e-2)
        go = torch.randn_like(ya)
        ya.backward(go)
        yb.backward(go)
        for a, b in [(xa.grad, xb.grad), (fused.weight.grad, plain.weight.grad), (fused.bias.grad, plain.bias.grad)]:
            assert a.dtype == torch.float32 and a.shape == b.shape
            scale = b.abs().max().item() + 1e-6
            assert (a - b).abs().max().item() <= 0.15 * scale  # bf16 math and a few flipped ReLU masks
