"""Single-GPU end-to-end: the flagship training step through `with_bagua` (world size 1)
and the engine scheduler driving GPU buckets with CUDA events."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_smoke_entry():
    import __graft_entry__ as g

    g.smoke()


def test_scheduler_with_cuda_events_single_rank():
    import bagua_core as bc

    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream()
    uid = bc.BaguaSingleCommunicatorPy.generate_nccl_unique_id_str()
    comm = bc.BaguaSingleCommunicatorPy(0, 1, 0, stream.cuda_stream, uid)
    backend = bc.BaguaCommBackendPy(10, 0)
    flat = torch.randn(3 * 4096, device=dev)
    views = [flat[i * 4096:(i + 1) * 4096] for i in range(3)]
    ts = [bc.BaguaTensorPy(v, f"t{i}") for i, v in enumerate(views)]
    bucket = bc.BaguaBucketPy("b", ts)
    bucket.append_centralized_synchronous_op(comm, None, hierarchical=False, average=True, scattergather=True,
                                             compression="MinMaxUInt8")
    backend.register_ordered_buckets([bucket])
    orig = flat.clone()
    events = []  # the engine borrows the handles: keep the events alive until the wait returns
    for t in ts:
        ev = torch.cuda.Event()
        ev.record()
        events.append(ev)
        backend.mark_communication_ready(t, ev.cuda_event)
    assert backend.wait_pending_comm_ops() == 1
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    # one rank: ByteGrad = quantise/dequantise twice
    assert (flat - orig).abs().max() <= 2 * (orig.max() - orig.min()) / 255
    backend.close()
