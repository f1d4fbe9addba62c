"""The functional collectives of the trainer layer (`bagua_core_b200.parallel.allreduce`, ...)
on CPU ranks (gloo): every call against its definition."""
import torch

from mp_util import run_ranks


def _worker(rank, world):
    import bagua_core_b200.parallel as P

    P.init_process_group(torch.device("cpu"))
    n = 6
    base = [torch.arange(n * world, dtype=torch.float32) * (r + 1) + r for r in range(world)]  # every rank's data
    mine = base[rank].clone()
    total = torch.stack(base).sum(0)
    done = []

    out = torch.zeros_like(mine)
    P.allreduce(mine, out, P.ReduceOp.SUM)
    assert torch.equal(out, total)
    t = mine.clone()
    P.allreduce_inplace(t, P.ReduceOp.AVG)
    assert torch.allclose(t, total / world)
    t = mine.clone()
    P.allreduce_inplace(t, P.ReduceOp.MAX)
    assert torch.equal(t, torch.stack(base).max(0).values)
    done.append("allreduce")

    t = mine.clone()
    P.broadcast(t, src=world - 1)
    assert torch.equal(t, base[world - 1])
    done.append("broadcast")

    out = torch.full_like(mine, -1.0)
    P.reduce(mine, out, dst=1, op=P.ReduceOp.SUM)
    if rank == 1:
        assert torch.equal(out, total)
    t = mine.clone()
    P.reduce_inplace(t, dst=0)
    if rank == 0:
        assert torch.equal(t, total)
    done.append("reduce")

    part = mine[:n].clone()
    out = torch.zeros(n * world)
    P.allgather(part, out)
    assert torch.equal(out, torch.cat([b[:n] for b in base]))
    t = torch.zeros(n * world)
    t[rank * n:(rank + 1) * n] = part
    P.allgather_inplace(t)
    assert torch.equal(t, out)
    done.append("allgather")

    out = torch.full((n * world,), -1.0)
    P.gather(part, out, dst=0)
    if rank == 0:
        assert torch.equal(out, torch.cat([b[:n] for b in base]))
    t = torch.zeros(n * world) if rank == world - 1 else part.clone()
    if rank == world - 1:
        t[rank * n:(rank + 1) * n] = part
    P.gather_inplace(t, n, dst=world - 1)
    if rank == world - 1:
        assert torch.equal(t, torch.cat([b[:n] for b in base]))
    done.append("gather")

    out = torch.zeros(n)
    P.scatter(mine, out, src=0)
    assert torch.equal(out, base[0][rank * n:(rank + 1) * n])
    t = mine.clone() if rank == 1 else torch.zeros(n)
    P.scatter_inplace(t, n, src=1)
    got = t[rank * n:(rank + 1) * n] if rank == 1 else t
    assert torch.equal(got, base[1][rank * n:(rank + 1) * n])
    done.append("scatter")

    out = torch.zeros(n)
    P.reduce_scatter(mine, out, P.ReduceOp.SUM)
    assert torch.equal(out, total[rank * n:(rank + 1) * n])
    t = mine.clone()
    P.reduce_scatter_inplace(t, P.ReduceOp.SUM)
    assert torch.equal(t[rank * n:(rank + 1) * n], total[rank * n:(rank + 1) * n])
    done.append("reduce_scatter")

    out = torch.zeros_like(mine)
    P.alltoall(mine, out)
    expect = torch.cat([b[rank * n:(rank + 1) * n] for b in base])
    assert torch.equal(out, expect)
    t = mine.clone()
    P.alltoall_inplace(t)
    assert torch.equal(t, expect)
    done.append("alltoall")

    # alltoall_v: rank r sends (q + 1) elements to rank q, taken from the front of its data
    send_counts = [q + 1 for q in range(world)]
    send_displs = [sum(send_counts[:q]) for q in range(world)]
    recv_counts = [rank + 1] * world
    recv_displs = [q * (rank + 1) for q in range(world)]
    out = torch.zeros((rank + 1) * world)
    P.alltoall_v(mine, send_counts, send_displs, out, recv_counts, recv_displs)
    lo = send_displs[rank]
    assert torch.equal(out, torch.cat([b[lo:lo + rank + 1] for b in base]))
    done.append("alltoall_v")

    if world >= 2:
        t = mine.clone()
        if rank == 0:
            P.send(t, dst=1)
        elif rank == 1:
            P.recv(t, src=0)
            assert torch.equal(t, base[0])
        done.append("send_recv")

    P.barrier()
    done.append("barrier")
    P.destroy_process_group()
    return done


def test_functional_collectives_match_their_definitions():
    res = run_ranks(_worker, 3)
    assert all(r[-1] == "barrier" and len(r) == 11 for r in res), res
