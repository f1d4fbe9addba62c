"""Flat buckets: contiguous storage shared by a group of tensors, registered with the engine.

A bucket is what the engine communicates in one fused kernel.  Tensors (gradients or
weights) are re-pointed at slices of one flat buffer so the engine can alias the bucket in
place (no staging copy); a padding tensor named ``bagua_padding_tensor_bucket_<i>`` rounds
the bucket up so that it splits into equal, 16-byte-aligned chunks per rank — the layout
the fused kernels need (the engine treats tensors with that name prefix as always ready;
reference: bagua-core-internal/src/datatypes/mod.rs:810-813).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .. import BaguaBucketPy, BaguaTensorPy

# 16 uint8 values per 16-byte vector of compressed data, per rank chunk
ALIGN_ELEMS_PER_RANK = 16


class BaguaTensor:
    """A named tensor registered with the engine (its live storage is `tensor`)."""

    def __init__(self, tensor: torch.Tensor, name: str, owner=None, kind: str = "grad"):
        self.tensor = tensor
        self.name = name
        self.owner = owner  # the nn.Parameter this tensor belongs to (if any)
        self.kind = kind
        self.backend_tensor = BaguaTensorPy(tensor, name)


class BaguaBucket:
    def __init__(self, tensors: Sequence[BaguaTensor], name: str, flatten: bool = True, alignment: int = 1,
                 allocator=None):
        self.name = name
        self.tensors: List[BaguaTensor] = list(tensors)
        self.flattened: Optional[torch.Tensor] = None
        self.padding: Optional[BaguaTensor] = None
        self._alignment = max(1, alignment)
        # allocator(numel, dtype, device, tensors) -> 1-D tensor or None (e.g. symmetric memory); it may hand
        # back the buffer these very tensors already live in, in this order (a re-bucketing with an unchanged layout)
        self._allocator = allocator
        if flatten:
            self._flatten()
        backend_tensors = [t.backend_tensor for t in self.tensors]
        if self.padding is not None:
            backend_tensors.append(self.padding.backend_tensor)
        self.backend_bucket = BaguaBucketPy(name, backend_tensors)

    # ---- layout -------------------------------------------------------------------
    def _flatten(self):
        first = self.tensors[0].tensor
        total = sum(t.tensor.numel() for t in self.tensors)
        padded = (total + self._alignment - 1) // self._alignment * self._alignment
        flat = self._allocator(padded, first.dtype, first.device, self.tensors) if self._allocator is not None else None
        if flat is None:
            flat = torch.zeros(padded, dtype=first.dtype, device=first.device)
        off = 0
        with torch.no_grad():
            for t in self.tensors:
                n = t.tensor.numel()
                shape, stride = tuple(t.tensor.shape), tuple(t.tensor.stride())
                # keep the tensor's own (dense) layout, e.g. channels_last conv weights
                view = flat[off:off + n].as_strided(shape, stride)
                view.copy_(t.tensor)
                # re-point the registered tensor at the bucket storage (same TensorImpl, new storage)
                t.tensor.set_(flat.untyped_storage(), off, shape, stride)
                off += n
        if padded > total:
            pad = flat[total:padded]
            self.padding = BaguaTensor(pad, f"bagua_padding_tensor_{self.name}", kind="padding")
        self.flattened = flat

    @property
    def numel(self) -> int:
        return self.flattened.numel() if self.flattened is not None else sum(t.tensor.numel() for t in self.tensors)

    def bytes(self) -> int:
        return self.numel * self.tensors[0].tensor.element_size()

    # ---- ops (thin forwards to the engine; same names as the reference bindings) -----
    def clear_ops(self):
        self.backend_bucket.clear_ops()
        return self

    def append_python_op(self, fn):
        self.backend_bucket.append_python_op(fn)
        return self

    def append_centralized_synchronous_op(self, pg, hierarchical=False, average=True, scattergather=False,
                                          compression=None):
        inter, intra = _comms(pg, hierarchical)
        self.backend_bucket.append_centralized_synchronous_op(inter, intra, hierarchical=hierarchical, average=average,
                                                              scattergather=scattergather, compression=compression)
        return self

    def append_decentralized_synchronous_op(self, pg, peer_weight: torch.Tensor, hierarchical=False,
                                            peer_selection_mode="all"):
        inter, intra = _comms(pg, hierarchical)
        self._peer_weight = BaguaTensorPy(peer_weight, f"{self.name}_peer_weight")
        self.backend_bucket.append_decentralized_synchronous_op(inter, intra, hierarchical=hierarchical,
                                                                peer_selection_mode=peer_selection_mode,
                                                                peer_weight=self._peer_weight)
        return self

    def append_low_precision_decentralized_synchronous_op(self, pg, weight, left_peer_weight, right_peer_weight,
                                                          hierarchical=False, compression="MinMaxUInt8"):
        inter, intra = _comms(pg, hierarchical)
        self._lp = [BaguaTensorPy(weight, f"{self.name}_weight"),
                    BaguaTensorPy(left_peer_weight, f"{self.name}_left"),
                    BaguaTensorPy(right_peer_weight, f"{self.name}_right")]
        self.backend_bucket.append_low_precision_decentralized_synchronous_op(
            inter, intra, hierarchical=hierarchical, peer_selection_mode="ring", compression=compression,
            weight=self._lp[0], left_peer_weight=self._lp[1], right_peer_weight=self._lp[2])
        return self

    def append_asynchronous_model_average_op(self, pg, peer_selection_mode="all"):
        torch_stream = torch.cuda.current_stream().cuda_stream if pg.is_cuda else 0
        self.backend_bucket.append_decentralized_asynchronous_op(pg.global_comm, None,
                                                                 peer_selection_mode=peer_selection_mode,
                                                                 torch_stream=torch_stream)
        return self


def _comms(pg, hierarchical: bool):
    if not hierarchical:
        return pg.global_comm, None
    pg.ensure_hierarchical()
    if pg.intra_comm is None:
        raise RuntimeError("hierarchical communication needs intra-node / inter-node communicators")
    return pg.inter_comm, pg.intra_comm


def split_into_buckets(tensors: Sequence[BaguaTensor], bucket_bytes: int) -> List[List[BaguaTensor]]:
    """Greedy split in the given order; every bucket holds one dtype and at most
    `bucket_bytes` (a single larger tensor gets a bucket of its own)."""
    groups: List[List[BaguaTensor]] = []
    cur: List[BaguaTensor] = []
    cur_bytes = 0
    for t in tensors:
        nbytes = t.tensor.numel() * t.tensor.element_size()
        if cur and (cur_bytes + nbytes > bucket_bytes or cur[0].tensor.dtype != t.tensor.dtype):
            groups.append(cur)
            cur, cur_bytes = [], 0
        cur.append(t)
        cur_bytes += nbytes
    if cur:
        groups.append(cur)
    return groups
