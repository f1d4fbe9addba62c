"""Weight gradients accumulated in place by the GEMM that computes them (`bagua_core_b200.ops.wgrad`,
used by `ShadowLinear`): the result is the fp32 product (closer to exact than the bf16 matrix the
ordinary path hands to autograd), the trainer's gradient-ready hooks still run exactly once per
parameter, every case the shortcut must not take falls back to the ordinary path, and training
through `with_bagua` on two ranks agrees with training without it."""
import pytest
import torch

from mp_util import run_ranks


@pytest.fixture
def wgrad():
    from bagua_core_b200.ops import wgrad as W

    saved = W.enabled
    W.enabled = True
    yield W
    W.enabled = saved


def _pair(seed=0, n_in=48, n_out=24):
    from bagua_core_b200.ops.fused_linear import ShadowLinear

    torch.manual_seed(seed)
    m = ShadowLinear(n_in, n_out)
    ref = torch.nn.Linear(n_in, n_out)
    ref.load_state_dict(m.state_dict())
    for mod in (m, ref):
        for p in mod.parameters():
            p.grad = torch.zeros_like(p)
    return m, ref


def _backward(mod, x, scale=1.0):
    with torch.autocast("cpu", dtype=torch.bfloat16):
        (mod(x).float() * scale).square().sum().backward()


def test_gradient_is_the_fp32_product_and_hooks_run_once(wgrad):
    m, ref = _pair()
    fired = []
    m.weight.register_post_accumulate_grad_hook(lambda p: fired.append(p.grad.clone()))
    x = torch.randn(7, 3, 48)  # leading dimensions are flattened
    before = wgrad.accumulated
    _backward(m, x)
    _backward(ref, x)
    assert wgrad.accumulated == before + 1
    assert len(fired) == 1 and torch.equal(fired[0], m.weight.grad)  # the hook saw the finished gradient
    # exact: the same bf16 operands multiplied in fp64
    with torch.no_grad():
        xb = x.to(torch.bfloat16).reshape(-1, 48)
        y = torch.nn.functional.linear(xb, m.weight.to(torch.bfloat16), m.bias.to(torch.bfloat16))
        dy = (2 * y.float()).to(torch.bfloat16)
        exact = dy.double().t() @ xb.double()
    err_inplace = (m.weight.grad.double() - exact).abs().max().item()
    err_ordinary = (ref.weight.grad.double() - exact).abs().max().item()
    assert err_inplace <= err_ordinary and err_inplace < 1e-3 * exact.abs().max().item()
    assert torch.allclose(m.bias.grad, ref.bias.grad, rtol=1e-2, atol=1e-2)
    # a second backward adds to the first
    first = m.weight.grad.clone()
    _backward(m, x)
    assert torch.allclose(m.weight.grad, 2 * first, rtol=1e-6, atol=1e-6) and len(fired) == 2


@pytest.mark.filterwarnings("ignore:grad and param do not obey the gradient layout contract")  # the strided-gradient case
def test_cases_that_take_the_ordinary_path(wgrad):
    x = torch.randn(5, 48)
    # no gradient tensor yet: autograd creates it
    m, _ = _pair(1)
    m.weight.grad = None
    d0 = wgrad.declined
    _backward(m, x)
    assert wgrad.declined == d0 + 1 and m.weight.grad is not None
    # a tensor hook on the weight: autograd must see the gradient to apply it
    m, ref = _pair(2)
    m.weight.register_hook(lambda g: g * 0)
    _backward(m, x)
    assert wgrad.declined == d0 + 2 and torch.count_nonzero(m.weight.grad) == 0
    # the weight used twice in one graph: both uses decline, the sum is accumulated once
    m, ref = _pair(3)
    fired = []
    m.weight.register_post_accumulate_grad_hook(lambda p: fired.append(1))
    with torch.autocast("cpu", dtype=torch.bfloat16):
        (m(x).float().sum() + m(2 * x).float().sum()).backward()
        (ref(x).float().sum() + ref(2 * x).float().sum()).backward()
    assert wgrad.declined == d0 + 4 and len(fired) == 1
    assert torch.allclose(m.weight.grad, ref.weight.grad, rtol=2e-2, atol=2e-2)
    # a forward whose graph was dropped without a backward does not count as a use
    m, _ = _pair(4)
    with torch.autocast("cpu", dtype=torch.bfloat16):
        m(x)
    a0 = wgrad.accumulated
    _backward(m, x)
    assert wgrad.accumulated == a0 + 1
    # a gradient that is not contiguous (a strided view of a wider buffer)
    m, ref = _pair(5)
    m.weight.grad = torch.zeros(24, 96)[:, ::2]
    d1 = wgrad.declined
    _backward(m, x)
    _backward(ref, x)
    assert wgrad.declined == d1 + 1 and torch.allclose(m.weight.grad, ref.weight.grad, rtol=2e-2, atol=2e-2)
    # switched off: the module is nn.Linear again
    wgrad.enabled = False
    m, ref = _pair(6)
    a0, d1 = wgrad.accumulated, wgrad.declined
    _backward(m, x)
    _backward(ref, x)
    assert (wgrad.accumulated, wgrad.declined) == (a0, d1) and torch.equal(m.weight.grad, ref.weight.grad)


def test_autograd_runs_the_hooks_of_a_parameter_that_got_no_gradient(wgrad):
    """The property `accumulate` relies on instead of running the hooks itself (and checks once per
    process); if a torch version loses it, the module runs the hooks by hand."""
    assert wgrad._autograd_runs_hooks_without_a_gradient() is True


class _Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        from bagua_core_b200.ops.fused_conv import ConvBiasReLUPool
        from bagua_core_b200.ops.fused_linear import ShadowLinear

        self.c = ConvBiasReLUPool(3, 8, 3, padding=1)
        self.fc1 = ShadowLinear(8 * 4 * 4, 64)
        self.fc2 = ShadowLinear(64, 5)

    def forward(self, x):
        return self.fc2(torch.relu(self.fc1(torch.flatten(self.c(x), 1))))


def _train(rank, world, inplace, algorithm, steps):
    import bagua_core_b200.parallel as P
    from bagua_core_b200.ops import wgrad as W

    W.enabled = inplace
    torch.manual_seed(5)
    model = _Net().to(memory_format=torch.channels_last)
    P.init_process_group(torch.device("cpu"))
    opt = P.FlatSGD(model.parameters(), lr=0.05, momentum=0.9)
    algo = {"allreduce": P.GradientAllReduceAlgorithm, "bytegrad": P.ByteGradAlgorithm}[algorithm]()
    bm = P.with_bagua(model, [opt], algo, bucket_bytes=4096)
    g = torch.Generator().manual_seed(100 + rank)
    losses = []
    for s in range(steps):
        x = torch.randn(4, 3, 8, 8, generator=g).contiguous(memory_format=torch.channels_last)
        y = torch.randint(0, 5, (4,), generator=g)
        opt.zero_grad()
        ctx = bm.no_sync() if s == 2 else None  # one step of local accumulation
        if ctx is not None:
            ctx.__enter__()
        with torch.autocast("cpu", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(bm(x).float(), y)
        loss.backward()
        if ctx is not None:
            ctx.__exit__(None, None, None)
        else:
            opt.step()
        losses.append(loss.item())
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    counts = (W.accumulated, W.declined)
    P.destroy_process_group()
    return flat, losses, counts


@pytest.mark.parametrize("algorithm", ["allreduce", "bytegrad"])
def test_training_through_with_bagua_agrees_with_the_ordinary_path(algorithm):
    steps = 6
    plain = run_ranks(_train, 2, args=(False, algorithm, steps))
    fused = run_ranks(_train, 2, args=(True, algorithm, steps))
    for r in range(2):
        assert plain[r][2] == (0, 0)
        assert fused[r][2] == (2 * steps, 0)  # both linear layers, every step
        # same training up to the rounding the ordinary path applies to the weight gradients
        assert torch.allclose(plain[r][0], fused[r][0], rtol=0, atol=2e-2), (plain[r][0] - fused[r][0]).abs().max()
        assert all(abs(a - b) < 5e-2 for a, b in zip(plain[r][1], fused[r][1]))
    assert torch.equal(fused[0][0], fused[1][0])  # the ranks stay bit-identical to each other


def _train_bert(rank, world, inplace, shadow, steps):
    import bagua_core_b200.parallel as P
    from bagua_core_b200.models import BertConfig, BertForQuestionAnswering
    from bagua_core_b200.ops import wgrad as W

    W.enabled = inplace
    torch.manual_seed(11)
    cfg = BertConfig.tiny()
    cfg.dropout = 0.0
    model = BertForQuestionAnswering(cfg)
    P.init_process_group(torch.device("cpu"))
    opt = P.FlatSGD(model.parameters(), lr=0.05, momentum=0.9, bf16_shadow=shadow)
    bm = P.with_bagua(model, [opt], P.ByteGradAlgorithm(), bucket_bytes=64 << 10)
    g = torch.Generator().manual_seed(7 + rank)
    losses = []
    for _ in range(steps):
        ids = torch.randint(0, cfg.vocab_size, (2, 16), generator=g)
        span = torch.randint(0, 16, (2, 2), generator=g)
        opt.zero_grad()
        with torch.autocast("cpu", dtype=torch.bfloat16):
            loss = bm(ids, span[:, 0], span[:, 1])
        loss.backward()
        opt.step()
        losses.append(loss.item())
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    counts = (W.accumulated, W.declined)
    P.destroy_process_group()
    return flat, losses, counts


def test_bert_encoder_projections_take_both_options():
    """The encoder's four projections per layer are `ShadowLinear`: with in-place weight gradients (and
    bf16 weight copies on top) ByteGrad training of a two-layer BERT stays with the ordinary path."""
    steps = 4
    plain = run_ranks(_train_bert, 2, args=(False, False, steps))
    fused = run_ranks(_train_bert, 2, args=(True, False, steps))
    both = run_ranks(_train_bert, 2, args=(True, True, steps))
    for r in range(2):
        assert plain[r][2] == (0, 0)
        assert fused[r][2] == (2 * 4 * steps, 0) and both[r][2] == (2 * 4 * steps, 0)
        for other in (fused, both):
            assert (plain[r][0] - other[r][0]).abs().max().item() < 2e-2
            assert all(abs(a - b) < 5e-2 for a, b in zip(plain[r][1], other[r][1]))
        # the bf16 copies hold the values the casts would produce: same training, bit for bit
        assert torch.equal(fused[r][0], both[r][0]) and fused[r][1] == both[r][1]
    assert torch.equal(both[0][0], both[1][0])
