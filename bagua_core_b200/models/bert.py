"""BERT-large encoder with a span-prediction (SQuAD-style) head: 24 layers, hidden 1024,
16 heads, FFN 4096, vocabulary 30522, post-LayerNorm, learned positions.  Attention goes
through `torch.nn.functional.scaled_dot_product_attention` (library kernel).  Random
initialisation only.

The encoder's projections are `ShadowLinear` modules: `nn.Linear` (same parameter names, same
math) unless an optimizer keeps bf16 copies of the weights (`FlatSGD(bf16_shadow=True)`) or
in-place weight-gradient accumulation is on (`bagua_core_b200.ops.wgrad.enabled`), in which case
they skip the per-forward weight casts and the cast-and-add of every weight gradient."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops.fused_linear import ShadowLinear


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden: int = 1024
    layers: int = 24
    heads: int = 16
    ffn: int = 4096
    max_pos: int = 512
    type_vocab: int = 2
    dropout: float = 0.1
    eps: float = 1e-12
    # True: LayerNorm as autocast runs it, fp32 in and out, which turns the whole residual stream
    # into fp32 and adds a cast before every projection.
    fp32_layernorm_io: bool = False

    @staticmethod
    def large():
        return BertConfig()

    @staticmethod
    def tiny():
        return BertConfig(vocab_size=1000, hidden=64, layers=2, heads=4, ffn=128, max_pos=128)


class _LayerNorm(nn.LayerNorm):
    """LayerNorm whose output stays in the autocast dtype.

    Autocast runs `layer_norm` in fp32: a bf16 activation is cast up, normalised, and leaves as
    fp32, so the residual sum that follows is fp32 too and every projection casts its input down
    again: per site about five times the bytes of a bf16-in, bf16-out normalisation.  The library
    kernel accumulates its statistics in fp32 whatever the input type, so here a low-precision
    input is normalised as it is (parameters cast to its type: 2·hidden values) and an fp32 input
    (the embedding sum) is normalised in fp32 and cast once.  Outside autocast this is
    `nn.LayerNorm`."""

    def forward(self, x):
        dev = x.device.type
        if not torch.is_autocast_enabled(dev):
            return super().forward(x)
        dtype = torch.get_autocast_dtype(dev)
        with torch.autocast(dev, enabled=False):
            if x.dtype == torch.float32:
                return F.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps).to(dtype)
            return F.layer_norm(x, self.normalized_shape, self.weight.to(x.dtype), self.bias.to(x.dtype), self.eps)


def _layer_norm(c: "BertConfig") -> nn.LayerNorm:
    return (nn.LayerNorm if c.fp32_layernorm_io else _LayerNorm)(c.hidden, eps=c.eps)


class _Layer(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.heads = c.heads
        self.qkv = ShadowLinear(c.hidden, 3 * c.hidden)
        self.proj = ShadowLinear(c.hidden, c.hidden)
        self.ln1 = _layer_norm(c)
        self.fc1 = ShadowLinear(c.hidden, c.ffn)
        self.fc2 = ShadowLinear(c.ffn, c.hidden)
        self.ln2 = _layer_norm(c)
        self.drop = nn.Dropout(c.dropout)
        self.p = c.dropout

    def forward(self, x):
        b, s, h = x.shape
        q, k, v = self.qkv(x).view(b, s, 3, self.heads, h // self.heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, dropout_p=self.p if self.training else 0.0)
        a = a.transpose(1, 2).reshape(b, s, h)
        x = self.ln1(x + self.drop(self.proj(a)))
        f = self.fc2(F.gelu(self.fc1(x)))
        return self.ln2(x + self.drop(f))


class BertForQuestionAnswering(nn.Module):
    def __init__(self, config: BertConfig = None):
        super().__init__()
        c = config or BertConfig.large()
        self.config = c
        self.tok = nn.Embedding(c.vocab_size, c.hidden)
        self.pos = nn.Embedding(c.max_pos, c.hidden)
        self.typ = nn.Embedding(c.type_vocab, c.hidden)
        self.ln = _layer_norm(c)
        self.drop = nn.Dropout(c.dropout)
        self.layers = nn.ModuleList([_Layer(c) for _ in range(c.layers)])
        self.qa = nn.Linear(c.hidden, 2)
        self.apply(self._init)

    @staticmethod
    def _init(m):
        if isinstance(m, (nn.Linear, nn.Embedding)):
            nn.init.normal_(m.weight, 0.0, 0.02)
            if isinstance(m, nn.Linear) and m.bias is not None:
                nn.init.zeros_(m.bias)

    def forward(self, input_ids, start_positions=None, end_positions=None):
        b, s = input_ids.shape
        pos = torch.arange(s, device=input_ids.device)
        x = self.tok(input_ids) + self.pos(pos)[None] + self.typ.weight[0][None, None]
        x = self.drop(self.ln(x))
        for layer in self.layers:
            x = layer(x)
        logits = self.qa(x).float()
        start, end = logits[..., 0], logits[..., 1]
        if start_positions is None:
            return start, end
        return (F.cross_entropy(start, start_positions) + F.cross_entropy(end, end_positions)) / 2
