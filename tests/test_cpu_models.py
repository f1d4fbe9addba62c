"""Model definitions: the BERT encoder keeps its residual stream in the autocast dtype (its LayerNorm
takes and returns low precision, statistics still in fp32) and is unchanged outside autocast."""
import copy

import torch

from bagua_core_b200.models import BertConfig, BertForQuestionAnswering


def _pair():
    torch.manual_seed(0)
    cfg = BertConfig.tiny()
    cfg.dropout = 0.0
    new = BertForQuestionAnswering(cfg)
    cfg_old = copy.copy(cfg)
    cfg_old.fp32_layernorm_io = True
    old = BertForQuestionAnswering(cfg_old)
    old.load_state_dict(new.state_dict())  # same parameter names and shapes
    return cfg, new, old


def test_bert_layernorm_outside_autocast_is_nn_layernorm():
    cfg, new, old = _pair()
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    for a, b in zip(new(ids), old(ids)):
        assert torch.equal(a, b)


def test_bert_residual_stream_stays_in_bf16_under_autocast_and_training_agrees():
    cfg, new, old = _pair()
    seen = {"new": [], "old": []}
    for name, model in (("new", new), ("old", old)):
        for layer in model.layers:
            layer.ln2.register_forward_hook(lambda m, i, o, k=name: seen[k].append((i[0].dtype, o.dtype)))
            layer.qkv.register_forward_hook(lambda m, i, o, k=name: seen[k].append((i[0].dtype,)))
    g = torch.Generator().manual_seed(1)
    opts = [torch.optim.SGD(m.parameters(), lr=0.05) for m in (new, old)]
    losses = [[], []]
    for _ in range(5):
        ids = torch.randint(0, cfg.vocab_size, (2, 16), generator=g)
        span = torch.randint(0, 16, (2, 2), generator=g)
        for k, (model, opt) in enumerate(zip((new, old), opts)):
            opt.zero_grad()
            with torch.autocast("cpu", dtype=torch.bfloat16):
                loss = model(ids, span[:, 0], span[:, 1])
            loss.backward()
            opt.step()
            losses[k].append(loss.item())
    # every projection of the second layer on gets a bf16 input; the stock module hands it fp32
    assert all(d == (torch.bfloat16, torch.bfloat16) for d in seen["new"] if len(d) == 2)
    assert all(d == (torch.bfloat16,) for d in seen["new"] if len(d) == 1)
    assert all(d == (torch.float32, torch.float32) for d in seen["old"] if len(d) == 2)
    assert all(abs(a - b) < 3e-2 for a, b in zip(*losses)), losses
