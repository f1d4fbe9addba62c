"""Helpers to run a function as several ranks (CPU/gloo or one GPU per rank/NCCL)."""
import os
import socket
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _to_np(o):
    """Tensors travel between processes as numpy arrays (no shared-memory handles to outlive the child)."""
    if isinstance(o, torch.Tensor):
        return ("__tensor__", o.detach().cpu().numpy() if o.dtype != torch.bfloat16 else o.detach().cpu().float().numpy(),
                str(o.dtype))
    if isinstance(o, dict):
        return {k: _to_np(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return type(o)(_to_np(v) for v in o)
    return o


def _from_np(o):
    if isinstance(o, tuple) and len(o) == 3 and o[0] == "__tensor__":
        t = torch.from_numpy(o[1].copy())
        return t.to(getattr(torch, o[2].split(".")[1]))
    if isinstance(o, dict):
        return {k: _from_np(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return type(o)(_from_np(v) for v in o)
    return o


def _check_pool_guards(device):
    """Every scratch block the engine took from its pools on this rank still has intact guard regions."""
    import bagua_core_b200 as bb

    damaged = bb._C.pool_check_guards(device)
    seen = bb._C.pool_stats(device)["guard_violations"]
    if damaged or seen:
        raise RuntimeError(f"pool guard regions overwritten on device {device}: {damaged} now, {seen} in total")


def _entry(rank, world, port, backend, fn, args, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["LOCAL_RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world)
    # CPU ranks always run with guard regions around the engine's pool blocks; GPU ranks when asked to
    guard = backend == "gloo" or os.environ.get("BAGUA_B200_POOL_GUARD") == "1"
    if guard:
        os.environ["BAGUA_B200_POOL_GUARD"] = "1"
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        dist.init_process_group(backend, rank=rank, world_size=world)
        out = fn(rank, world, *args)
        if guard:
            _check_pool_guards(rank if backend == "nccl" else -1)
        q.put((rank, "ok", _to_np(out)))
    except Exception:
        q.put((rank, "error", traceback.format_exc()))
    finally:
        try:
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:
            pass


def run_ranks(fn, world, backend="gloo", args=(), timeout=180):
    """Runs fn(rank, world, *args) in `world` processes; returns the list of results by rank."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, backend, fn, args, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, out = q.get(timeout=timeout)
            if status != "ok":
                raise RuntimeError(f"rank {rank} failed:\n{out}")
            results[rank] = _from_np(out)
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world)]
