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


def test_bert_trains_with_a_bf16_residual_stream():
    """A two-layer BERT through `with_bagua` with ByteGrad under bf16 autocast: the encoder's LayerNorms
    take and return bf16 (statistics in fp32 inside the library kernel), so every projection sees a
    bf16 input; losses stay finite and close to the model with stock fp32-in/fp32-out LayerNorms."""
    import copy
    import os

    import bagua_core_b200.parallel as P
    from bagua_core_b200.models import BertConfig, BertForQuestionAnswering

    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29547")
    dev = torch.device("cuda", 0)
    losses = []
    for stock in (False, True):
        torch.manual_seed(0)
        cfg = BertConfig.tiny()
        cfg.dropout = 0.0
        cfg = copy.copy(cfg)
        cfg.fp32_layernorm_io = stock
        model = BertForQuestionAnswering(cfg).to(dev)
        seen = []
        model.layers[1].qkv.register_forward_hook(lambda m, i, o: seen.append(i[0].dtype))
        P.init_process_group(dev)
        opt = P.FlatSGD(model.parameters(), lr=0.05, momentum=0.9)
        bm = P.with_bagua(model, [opt], P.ByteGradAlgorithm(), bucket_bytes=64 << 10)
        g = torch.Generator().manual_seed(3)
        run = []
        for _ in range(4):
            ids = torch.randint(0, cfg.vocab_size, (4, 32), generator=g).to(dev)
            span = torch.randint(0, 32, (4, 2), generator=g).to(dev)
            opt.zero_grad()
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = bm(ids, span[:, 0], span[:, 1])
            loss.backward()
            opt.step()
            run.append(loss.item())
        torch.cuda.synchronize()
        P.destroy_process_group()
        assert all(d == (torch.float32 if stock else torch.bfloat16) for d in seen), seen
        assert all(torch.isfinite(torch.tensor(run)))
        losses.append(run)
    assert all(abs(a - b) < 5e-2 for a, b in zip(*losses)), losses
