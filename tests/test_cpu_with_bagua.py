"""End-to-end training-loop tests of `with_bagua` on CPU ranks (gloo)."""
import pytest
import torch

from mp_util import run_ranks


def _data(world, steps, bs=8, d_in=16, d_out=4):
    g = torch.Generator().manual_seed(1234)
    xs = torch.randn(steps, world * bs, d_in, generator=g)
    ys = torch.randn(steps, world * bs, d_out, generator=g)
    return xs, ys


def _train(rank, world, algo_name, steps, opt_name):
    import bagua_core_b200.parallel as P
    from bagua_core_b200.models import MLP

    torch.manual_seed(7)  # same init everywhere (also broadcast from rank 0)
    model = MLP(16, 32, 4, depth=3)
    pg = P.init_process_group(torch.device("cpu"))
    if opt_name == "flat_sgd":
        opt = P.FlatSGD(model.parameters(), lr=0.05, momentum=0.9)
    elif opt_name == "qadam":
        opt = P.QAdamOptimizer(model.parameters(), lr=0.01, warmup_steps=3, eps=1e-2)
    else:
        opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    algo = {
        "allreduce": lambda: P.GradientAllReduceAlgorithm(),
        "allreduce_sg": lambda: P.GradientAllReduceAlgorithm(scattergather=True),
        "allreduce_hier": lambda: P.GradientAllReduceAlgorithm(hierarchical=True),
        "bytegrad": lambda: P.ByteGradAlgorithm(),
        "decentralized_all": lambda: P.DecentralizedAlgorithm(peer_selection_mode="all"),
        "decentralized_shift_one": lambda: P.DecentralizedAlgorithm(peer_selection_mode="shift_one"),
        "low_precision_decentralized": lambda: P.LowPrecisionDecentralizedAlgorithm(),
        "qadam": lambda: P.QAdamAlgorithm(opt),
    }[algo_name]()
    bm = P.with_bagua(model, [opt], algo, bucket_bytes=2048)
    xs, ys = _data(world, steps)
    bs = xs.shape[1] // world
    losses = []
    for s in range(steps):
        x = xs[s, rank * bs:(rank + 1) * bs]
        y = ys[s, rank * bs:(rank + 1) * bs]
        opt.zero_grad(set_to_none=False)
        loss = torch.nn.functional.mse_loss(bm(x), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    state = bm.bagua_state_dict()
    P.destroy_process_group()
    return flat, losses, state["step"]


def _single_process_reference(world, steps):
    from bagua_core_b200.models import MLP

    torch.manual_seed(7)
    model = MLP(16, 32, 4, depth=3)
    opt = torch.optim.SGD(model.parameters(), lr=0.05, momentum=0.9)
    xs, ys = _data(world, steps)
    for s in range(steps):
        opt.zero_grad()
        torch.nn.functional.mse_loss(model(xs[s]), ys[s]).backward()
        opt.step()
    return torch.cat([p.detach().reshape(-1) for p in model.parameters()])


@pytest.mark.parametrize("algo,opt", [("allreduce", "sgd"), ("allreduce", "flat_sgd"), ("allreduce_sg", "sgd"),
                                      ("allreduce_hier", "sgd")])
def test_gradient_allreduce_matches_large_batch(algo, opt):
    world, steps = 2, 4
    res = run_ranks(_train, world, args=(algo, steps, opt))
    ref = _single_process_reference(world, steps)
    for flat, _, step in res:
        assert step == steps
        assert torch.allclose(flat, ref, atol=1e-5), (flat - ref).abs().max()


def test_bytegrad_trains_and_ranks_agree():
    res = run_ranks(_train, 2, args=("bytegrad", 6, "sgd"))
    ref = _single_process_reference(2, 6)
    assert torch.equal(res[0][0], res[1][0])  # identical replicas
    assert (res[0][0] - ref).abs().max() < 0.05  # close to exact training despite 8-bit gradients
    assert res[0][1][-1] < res[0][1][0] * 1.5


@pytest.mark.parametrize("algo", ["decentralized_all", "decentralized_shift_one", "low_precision_decentralized"])
def test_decentralized_algorithms_run(algo):
    res = run_ranks(_train, 2, args=(algo, 5, "sgd"))
    # replicas stay close to each other and finite
    a, b = res[0][0], res[1][0]
    assert torch.isfinite(a).all() and torch.isfinite(b).all()
    assert (a - b).abs().max() < 0.2


def test_qadam_switches_to_compressed_momentum():
    res = run_ranks(_train, 2, args=("qadam", 6, "qadam"))
    a, b = res[0][0], res[1][0]
    assert torch.isfinite(a).all()
    assert torch.allclose(a, b, atol=1e-6)


def _two_groups(rank, world, steps):
    """Biases without weight decay and with their own learning rate, weights with decay: the flat
    optimizer must step every run of a bucket with its own group's hyperparameters."""
    import bagua_core_b200.parallel as P
    from bagua_core_b200.models import MLP

    torch.manual_seed(7)
    model = MLP(16, 32, 4, depth=3)
    pg = P.init_process_group(torch.device("cpu"))
    decay = [p for n, p in model.named_parameters() if not n.endswith("bias")]
    plain = [p for n, p in model.named_parameters() if n.endswith("bias")]
    opt = P.FlatSGD([{"params": decay, "weight_decay": 0.1}, {"params": plain, "weight_decay": 0.0, "lr": 0.2}],
                    lr=0.05, momentum=0.9)
    bm = P.with_bagua(model, [opt], P.GradientAllReduceAlgorithm(), bucket_bytes=2048)
    assert any(len(f["runs"]) > 1 for f in opt._flat), "the test needs a bucket that mixes both groups"
    xs, ys = _data(world, steps)
    bs = xs.shape[1] // world
    for s in range(steps):
        if s == 2:
            opt.param_groups[0]["lr"] = 0.01  # what a scheduler does
        opt.zero_grad()
        torch.nn.functional.mse_loss(bm(xs[s, rank * bs:(rank + 1) * bs]), ys[s, rank * bs:(rank + 1) * bs]).backward()
        opt.step()
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    P.destroy_process_group()
    return flat


def test_flat_sgd_honours_parameter_groups():
    from bagua_core_b200.models import MLP

    world, steps = 2, 4
    res = run_ranks(_two_groups, world, args=(steps,))
    torch.manual_seed(7)
    model = MLP(16, 32, 4, depth=3)
    decay = [p for n, p in model.named_parameters() if not n.endswith("bias")]
    plain = [p for n, p in model.named_parameters() if n.endswith("bias")]
    opt = torch.optim.SGD([{"params": decay, "weight_decay": 0.1}, {"params": plain, "weight_decay": 0.0, "lr": 0.2}],
                          lr=0.05, momentum=0.9)
    xs, ys = _data(world, steps)
    for s in range(steps):
        if s == 2:
            opt.param_groups[0]["lr"] = 0.01
        opt.zero_grad()
        torch.nn.functional.mse_loss(model(xs[s]), ys[s]).backward()
        opt.step()
    ref = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    for flat in res:
        assert torch.allclose(flat, ref, atol=1e-5), (flat - ref).abs().max()


class _TwoHeads(torch.nn.Module):
    def __init__(self):
        super().__init__()
        self.trunk = torch.nn.Linear(16, 32)
        self.aux = torch.nn.Linear(32, 4)
        self.main = torch.nn.Linear(32, 4)
        self.unused_aux = False

    def forward(self, x):
        h = torch.relu(self.trunk(x))
        if self.unused_aux:
            return self.aux(h), self.main(h)  # a loss on the second output leaves `aux` without gradients
        a = self.aux(h)
        return a * 2, self.main(h) + 0.5 * a  # the first output's own node still never receives a gradient


def _second_output_only(rank, world, steps, unused_aux):
    import bagua_core_b200.parallel as P

    torch.manual_seed(5)
    model = _TwoHeads()
    model.unused_aux = unused_aux
    pg = P.init_process_group(torch.device("cpu"))
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    bm = P.with_bagua(model, [opt], P.GradientAllReduceAlgorithm(), bucket_bytes=1 << 20)
    xs, ys = _data(world, steps)
    bs = xs.shape[1] // world
    for s in range(steps):
        opt.zero_grad(set_to_none=False)
        _aux, main = bm(xs[s, rank * bs:(rank + 1) * bs])
        torch.nn.functional.mse_loss(main, ys[s, rank * bs:(rank + 1) * bs]).backward()
        assert pg.backend.pending() == 0, "backward returned with communication still waiting to be collected"
        opt.step()
    flat = torch.cat([p.detach().reshape(-1) for n, p in model.named_parameters() if not n.startswith("aux")])
    step = bm.bagua_train_step_counter
    P.destroy_process_group()
    return flat, step


@pytest.mark.parametrize("unused_aux", [False, True])
def test_the_post_backward_step_runs_when_the_loss_uses_only_a_later_output(unused_aux):
    """unused_aux: one head's parameters get no gradient at all; their bucket must still be communicated."""
    world, steps = 2, 3
    res = run_ranks(_second_output_only, world, args=(steps, unused_aux))
    torch.manual_seed(5)
    model = _TwoHeads()
    model.unused_aux = unused_aux
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    xs, ys = _data(world, steps)
    for s in range(steps):
        opt.zero_grad()
        torch.nn.functional.mse_loss(model(xs[s])[1], ys[s]).backward()
        opt.step()
    ref = torch.cat([p.detach().reshape(-1) for n, p in model.named_parameters() if not n.startswith("aux")])
    for flat, step in res:
        assert step == steps
        assert torch.allclose(flat, ref, atol=1e-5), (flat - ref).abs().max()
