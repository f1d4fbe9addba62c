"""bf16 copies of the master weights, written by the optimizer kernel (`FlatSGD(bf16_shadow=True)`,
`bagua_core_b200.ops.shadow`): training with them is bit-identical to training with the per-forward
casts they replace, they are only used while provably current, and the fused step that writes them
equals the plain step."""
import torch

from mp_util import run_ranks


class _Net(torch.nn.Module):
    def __init__(self):
        super().__init__()
        from bagua_core_b200.ops.fused_conv import ConvBiasReLU, ConvBiasReLUPool
        from bagua_core_b200.ops.fused_linear import ShadowLinear

        self.c1 = ConvBiasReLU(3, 8, 3, padding=1)
        self.c2 = ConvBiasReLUPool(8, 16, 3, padding=1)
        self.fc1 = ShadowLinear(16 * 4 * 4, 32)
        self.fc2 = ShadowLinear(32, 5)

    def forward(self, x):
        x = self.c2(self.c1(x))
        return self.fc2(torch.relu(self.fc1(torch.flatten(x, 1))))


def _train(rank, world, use_copies, steps, disturb):
    """Both arms keep bf16 copies; with use_copies=False every lookup is made to miss, so the modules
    cast the fp32 weights in every forward pass, which is what the copies replace."""
    import bagua_core_b200.parallel as P
    from bagua_core_b200.ops import shadow as S

    S.enabled = use_copies
    torch.manual_seed(3)
    model = _Net().to(memory_format=torch.channels_last)
    P.init_process_group(torch.device("cpu"))
    opt = P.FlatSGD(model.parameters(), lr=0.05, momentum=0.9, weight_decay=1e-3, bf16_shadow=True)
    bm = P.with_bagua(model, [opt], P.GradientAllReduceAlgorithm(), bucket_bytes=4096)
    g = torch.Generator().manual_seed(100 + rank)
    losses, used = [], []
    for s in range(steps):
        x = torch.randn(4, 3, 8, 8, generator=g).contiguous(memory_format=torch.channels_last)
        y = torch.randint(0, 5, (4,), generator=g)
        if disturb and s == 3:
            with torch.no_grad():
                model.fc1.weight.mul_(0.5)  # an in-place change the optimizer did not make: bumps the version
        if disturb and s == 5:
            opt.refresh_bf16()
        before = S.hits
        opt.zero_grad()
        with torch.autocast("cpu", dtype=torch.bfloat16):
            loss = torch.nn.functional.cross_entropy(bm(x).float(), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
        used.append(S.hits - before)
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    copies_match = all(torch.equal(p._bagua_bf16.view, p.detach().to(torch.bfloat16)) for p in model.parameters())
    P.destroy_process_group()
    return flat, losses, used, copies_match


def test_training_with_bf16_shadows_is_bit_identical_to_casting():
    plain = run_ranks(_train, 2, args=(False, 6, False))
    shadowed = run_ranks(_train, 2, args=(True, 6, False))
    for r in range(2):
        assert torch.equal(plain[r][0], shadowed[r][0])
        assert plain[r][1] == shadowed[r][1]
        assert plain[r][2] == [0] * 6
        # no copy is trusted before the optimizer's first step; afterwards all four weights come from it
        assert shadowed[r][2] == [0, 4, 4, 4, 4, 4]
        assert shadowed[r][3]
    assert torch.equal(shadowed[0][0], shadowed[1][0])


def test_a_weight_changed_behind_the_optimizers_back_is_cast_again_until_refreshed():
    plain = run_ranks(_train, 2, args=(False, 8, True))
    shadowed = run_ranks(_train, 2, args=(True, 8, True))
    for r in range(2):
        assert torch.equal(plain[r][0], shadowed[r][0]) and plain[r][1] == shadowed[r][1]
        # step 3 changes fc1.weight in place: its copy is no longer trusted (3 of 4), refresh_bf16() at step 5 restores it
        assert shadowed[r][2] == [0, 4, 4, 3, 3, 4, 4, 4]
        assert shadowed[r][3]


def test_step_kernel_with_shadow_equals_the_plain_step():
    import bagua_core_b200 as bb

    C = bb._C
    for n in (1, 7, 1024, 4099):
        g = torch.Generator().manual_seed(n)
        p, grad = torch.randn(n, generator=g), torch.randn(n, generator=g)
        m = torch.zeros(n)
        p2, m2, h = p.clone(), m.clone(), torch.zeros(n, dtype=torch.bfloat16)
        for step in range(3):
            C.k_sgd_momentum_flat(p, grad, m, 0.1, 0.9, 0.0, 1e-4, True, step == 0, 0)
            C.k_sgd_momentum_flat_shadow(p2, grad, m2, h, 0.1, 0.9, 0.0, 1e-4, True, step == 0, 0)
            assert torch.equal(p, p2) and torch.equal(m, m2) and torch.equal(h, p2.to(torch.bfloat16))
