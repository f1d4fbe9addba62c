#!/usr/bin/env python
"""The engine's own API — the four classes of the `bagua_core` module — without the trainer layer.

This is the call sequence a framework integration makes (reference: bagua-core-py/src/lib.rs:21-38,
203-233, 308-349, 359-485):

1. one `BaguaSingleCommunicatorPy(rank, nranks, device_id, stream_ptr, id_str)` per rank; the id string
   comes from `generate_nccl_unique_id_str()` on one rank and is handed to the others out of band
   (GPU), or names a torch.distributed group, `"c10d:<group name>"`, with `device_id = -1` (host);
2. `BaguaTensorPy(torch_tensor, name)` for every tensor to communicate, grouped into `BaguaBucketPy`s;
3. communication ops appended to each bucket (here: gradient average, then ByteGrad);
4. `BaguaCommBackendPy.register_ordered_buckets`, then per step `mark_communication_ready(tensor,
   cuda_event)` as tensors become final and `wait_pending_comm_ops()` before they are used.

Run it as it is (two host ranks are spawned), or under a launcher on GPUs:

    python examples/low_level_api.py
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 examples/low_level_api.py
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run(rank: int, world: int) -> float:
    import bagua_core as bc

    use_gpu = torch.cuda.is_available() and torch.cuda.device_count() >= world
    if use_gpu:
        device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
        torch.cuda.set_device(device)
    else:
        device = torch.device("cpu")
    if not dist.is_initialized():
        dist.init_process_group("nccl" if use_gpu else "gloo", rank=rank, world_size=world)

    # 1. communicator
    if use_gpu:
        stream = torch.cuda.Stream(device)
        ids = [bc.BaguaSingleCommunicatorPy.generate_nccl_unique_id_str() if rank == 0 else None]
        dist.broadcast_object_list(ids, src=0)
        comm = bc.BaguaSingleCommunicatorPy(rank, world, device.index, stream.cuda_stream, ids[0])
    else:
        comm = bc.BaguaSingleCommunicatorPy(rank, world, -1, 0, "c10d:" + dist.group.WORLD.group_name)

    # 2. tensors in one flat storage (contiguous tensors are communicated in place), one bucket
    g = torch.Generator().manual_seed(rank)
    shapes = [(256, 64), (1024,), (32, 32)]
    flat = torch.empty(sum(torch.Size(s).numel() for s in shapes), device=device)
    tensors, off = [], 0
    for s in shapes:
        n = torch.Size(s).numel()
        view = flat[off:off + n].view(*s)
        view.copy_(torch.randn(*s, generator=g))
        tensors.append(view)
        off += n
    mine = flat.clone()
    handles = [bc.BaguaTensorPy(t, f"grad_{i}") for i, t in enumerate(tensors)]
    bucket = bc.BaguaBucketPy("bucket_0", handles)

    # 3 + 4. average the bucket over all ranks
    backend = bc.BaguaCommBackendPy(100, device.index if use_gpu else -1)
    bucket.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True)
    backend.register_ordered_buckets([bucket])

    def communicate():
        for h in handles:
            event = torch.cuda.current_stream().record_event().cuda_event if use_gpu else 0
            backend.mark_communication_ready(h, event)
        done = backend.wait_pending_comm_ops()
        if use_gpu:
            torch.cuda.current_stream().wait_stream(stream)
            torch.cuda.synchronize()
        return done

    assert communicate() == 1
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    mean = sum(gathered) / world
    err_avg = (flat - mean).abs().max().item()

    # the same bucket with another algorithm: ops can be replaced after registration
    flat.copy_(mine)
    bucket.clear_ops()
    bucket.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True, scattergather=True,
                                             compression="MinMaxUInt8")
    assert communicate() == 1
    err_q = (flat - mean).abs().max().item()
    bound = 2 * max((t.max() - t.min()).item() for t in gathered) / 255

    if rank == 0:
        print(f"average over {world} ranks: max error {err_avg:.2e}; ByteGrad: max error {err_q:.2e} (bound {bound:.2e})")
    assert err_avg < 1e-6 and err_q <= bound
    if hasattr(backend, "close"):
        backend.close()
    dist.barrier()
    return err_q


def _spawned(rank: int, world: int, port: int):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    run(rank, world)
    dist.destroy_process_group()


if __name__ == "__main__":
    if "RANK" in os.environ:  # under a launcher
        run(int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]))
        dist.destroy_process_group()
    else:
        import socket

        import torch.multiprocessing as mp

        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            free_port = s.getsockname()[1]
        mp.spawn(_spawned, args=(2, free_port), nprocs=2, join=True)
