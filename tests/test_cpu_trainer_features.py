"""Trainer-layer features on CPU ranks: asynchronous model averaging, checkpointable op
state, `no_sync`, gradients replaced by `zero_grad(set_to_none=True)`."""
import time

import torch

from mp_util import run_ranks


def _async(rank, world):
    import bagua_core_b200.parallel as P
    from bagua_core_b200.models import MLP

    torch.manual_seed(100 + rank)  # different init per rank; with_bagua broadcasts rank 0's
    model = MLP(8, 16, 4, depth=2)
    pg = P.init_process_group(torch.device("cpu"))
    opt = torch.optim.SGD(model.parameters(), lr=0.0)  # lr 0: only averaging moves the weights
    algo = P.AsyncModelAverageAlgorithm(sync_interval_ms=20)
    bm = P.with_bagua(model, [opt], algo)
    with torch.no_grad():
        for p in model.parameters():
            p.add_(float(rank))  # make replicas differ after the broadcast
    x, y = torch.randn(4, 8), torch.randn(4, 4)
    for _ in range(3):
        opt.zero_grad(set_to_none=False)
        torch.nn.functional.mse_loss(bm(x), y).backward()
        opt.step()
    deadline = time.time() + 20
    while algo.rounds < 3 and time.time() < deadline:
        time.sleep(0.05)
    algo.abort(bm)
    rounds = algo.rounds
    flat = torch.cat([p.detach().reshape(-1) for p in model.parameters()])
    P.destroy_process_group()
    return flat, rounds


def test_async_model_average_converges_replicas():
    res = run_ranks(_async, 2)
    (a, ra), (b, rb) = res
    assert ra >= 3 and rb >= 3
    # after a few averaging rounds both replicas sit at the mean of the perturbed weights
    assert torch.allclose(a, b, atol=1e-5)


def _async_uneven_stop(rank, world):
    """Rank 0 stops averaging early and keeps training; the other ranks go on for a while.  Nobody may be
    left waiting inside a round for the rank that stopped: the threads agree before every round."""
    import bagua_core_b200.parallel as P
    from bagua_core_b200.models import MLP

    torch.manual_seed(7)
    model = MLP(8, 16, 4, depth=2)
    pg = P.init_process_group(torch.device("cpu"))
    pg.backend.set_watchdog_timeout(20.0)
    opt = torch.optim.SGD(model.parameters(), lr=0.01)
    algo = P.AsyncModelAverageAlgorithm(sync_interval_ms=10)
    bm = P.with_bagua(model, [opt], algo)
    x, y = torch.randn(4, 8), torch.randn(4, 4)
    t0 = time.time()
    for step in range(30 if rank == 0 else 120):
        opt.zero_grad(set_to_none=False)
        torch.nn.functional.mse_loss(bm(x), y).backward()
        opt.step()
        time.sleep(0.005)
        if rank == 0 and step == 10:
            algo.abort(bm)  # the other ranks' threads end at their next round
    algo.abort(bm)
    alive = algo._thread is not None
    elapsed = time.time() - t0
    rounds = algo.rounds
    P.destroy_process_group()
    return rounds, alive, elapsed


def test_async_model_average_stops_everywhere_when_one_rank_stops():
    res = run_ranks(_async_uneven_stop, 3, timeout=120)
    rounds = [r[0] for r in res]
    assert len(set(rounds)) == 1, rounds  # every rank ran exactly the rounds all of them agreed on
    assert not any(r[1] for r in res)
    assert all(r[2] < 60 for r in res)


def _state_and_nosync(rank, world):
    import bagua_core_b200.parallel as P
    from bagua_core_b200.models import MLP

    torch.manual_seed(5)
    model = MLP(8, 16, 4, depth=2)
    pg = P.init_process_group(torch.device("cpu"))
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    bm = P.with_bagua(model, [opt], P.DecentralizedAlgorithm(peer_selection_mode="shift_one"))
    x, y = torch.randn(4, 8) + rank, torch.randn(4, 4)
    for _ in range(3):
        opt.zero_grad(set_to_none=False)
        torch.nn.functional.mse_loss(bm(x), y).backward()
        opt.step()
    state = bm.bagua_state_dict()
    # restoring the state rewinds the gossip step counter
    bm.load_bagua_state_dict({"step": 1, "ops": [[[("step", 1)]] for _ in bm.bagua_buckets], "algorithm": {}})
    after = bm.bagua_state_dict()
    P.destroy_process_group()
    return state["step"], state["ops"], after["step"], after["ops"]


def test_op_state_can_be_saved_and_restored():
    res = run_ranks(_state_and_nosync, 2)
    for step, ops, step2, ops2 in res:
        assert step == 3
        assert all(op == [[("step", 3)]] for op in ops)
        assert step2 == 1 and all(op == [[("step", 1)]] for op in ops2)


def _no_sync_and_set_to_none(rank, world):
    import bagua_core_b200 as bb
    import bagua_core_b200.parallel as P
    from bagua_core_b200.models import MLP

    torch.manual_seed(9)
    model = MLP(8, 16, 4, depth=2)
    pg = P.init_process_group(torch.device("cpu"))
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    bm = P.with_bagua(model, [opt], P.GradientAllReduceAlgorithm(), bucket_bytes=256)
    g = torch.Generator().manual_seed(rank)
    x, y = torch.randn(4, 8, generator=g), torch.randn(4, 4, generator=g)
    bb._C.reset_stats()
    with bm.no_sync():
        opt.zero_grad(set_to_none=False)
        torch.nn.functional.mse_loss(bm(x), y).backward()
    local = torch.cat([p.grad.reshape(-1).clone() for p in model.parameters()])
    scheduled_in_no_sync = bb._C.stats()["buckets_scheduled"]
    # a user optimizer that drops the gradients: the hook must move the fresh ones into the bucket
    opt.zero_grad(set_to_none=True)
    torch.nn.functional.mse_loss(bm(x), y).backward()
    synced = torch.cat([p.grad.reshape(-1).clone() for p in model.parameters()])
    views_ok = all(p.grad.data_ptr() >= b.flattened.data_ptr() for b in bm.bagua_buckets for t in b.tensors
                   for p in [t.owner])
    P.destroy_process_group()
    return local, synced, scheduled_in_no_sync, views_ok


def test_no_sync_and_regrown_gradients():
    res = run_ranks(_no_sync_and_set_to_none, 2)
    mean_local = (res[0][0] + res[1][0]) / 2
    for local, synced, scheduled, views_ok in res:
        assert scheduled == 0  # nothing communicated under no_sync
        assert torch.allclose(synced, mean_local, atol=1e-6)  # same data → all-reduced mean of the local grads
        assert views_ok


def test_qadam_multi_tensor_step_equals_the_per_tensor_formulas():
    """`QAdamOptimizer.step` runs one multi-tensor call per operation; element by element it must be
    the sequence m = b1 m + (1-b1) g, v = b2 v + (1-b2) g², p -= lr/bc1 · m / (sqrt(v)/sqrt(bc2) + eps)
    applied tensor by tensor — through warm-up (parameters without a gradient left alone) and after it
    (second moment frozen, every parameter moves)."""
    import bagua_core_b200.parallel as P

    torch.manual_seed(0)
    shapes = [(7, 5), (33,), (4, 4, 3), (1,)]
    params = [torch.nn.Parameter(torch.randn(*s)) for s in shapes]
    ref_p = [p.detach().clone() for p in params]
    ref_m = [torch.zeros_like(p) for p in ref_p]
    ref_v = [torch.zeros_like(p) for p in ref_p]
    lr, b1, b2, eps, wd, warmup = 0.02, 0.9, 0.999, 1e-3, 0.01, 3
    opt = P.QAdamOptimizer(params, lr=lr, warmup_steps=warmup, betas=(b1, b2), eps=eps, weight_decay=wd)
    for step in range(1, 7):
        grads = [torch.randn(*s) for s in shapes]
        skip = 1 if step == 2 else None  # no gradient for one parameter in one warm-up step
        for i, p in enumerate(params):
            p.grad = None if i == skip else grads[i].clone()
        if step > warmup:  # the algorithm updates the momentum itself after warm-up
            for i, p in enumerate(params):
                opt.state[p]["exp_avg"].mul_(b1).add_(grads[i], alpha=1 - b1)
                ref_m[i].mul_(b1).add_(grads[i], alpha=1 - b1)
        opt.step()
        for i in range(len(shapes)):
            if step <= warmup:
                if i == skip:
                    continue
                g = grads[i].add(ref_p[i], alpha=wd)
                ref_m[i].mul_(b1).add_(g, alpha=1 - b1)
                ref_v[i].mul_(b2).addcmul_(g, g, value=1 - b2)
            bc1, bc2 = 1 - b1 ** step, 1 - b2 ** min(step, warmup)
            denom = (ref_v[i].sqrt() / (bc2 ** 0.5)).add_(eps)
            ref_p[i].addcdiv_(ref_m[i], denom, value=-lr / bc1)
        for i, p in enumerate(params):
            assert torch.equal(p.detach(), ref_p[i]), (step, i)
            assert torch.equal(opt.state[p]["exp_avg"], ref_m[i]) and torch.equal(opt.state[p]["exp_avg_sq"], ref_v[i])
