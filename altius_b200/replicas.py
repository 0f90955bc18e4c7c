"""Batch-sharded replicas: the only multi-GPU mode of this backend.

Inference on one image depends on that image and the weights only, so the
global batch is cut along its first axis into one shard per rank, each rank
runs a full session replica on its own GPU, and the outputs are concatenated
on the host. There is no collective per inference. The weights are sent once
at load: rank 0 packs the f32 initializers into one blob and broadcasts it
(`torch.distributed`, NCCL over NVLink on GPUs, gloo on CPU); each rank hands
the landed device addresses to `altius_cuda_create` (`AcInitDesc.location = 1`).

The reference has no counterpart: it is a single-process CPU runtime.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np


def shard_bounds(global_batch: int, world_size: int) -> List[Tuple[int, int]]:
    """Contiguous [lo, hi) per rank; the first `global_batch % world_size` ranks
    take one extra item. Covers every item exactly once."""
    base, extra = divmod(global_batch, world_size)
    out, lo = [], 0
    for r in range(world_size):
        hi = lo + base + (1 if r < extra else 0)
        out.append((lo, hi))
        lo = hi
    return out


def shard_batch(array: np.ndarray, rank: int, world_size: int) -> np.ndarray:
    lo, hi = shard_bounds(array.shape[0], world_size)[rank]
    return array[lo:hi]


def pack_layout(model, min_bytes: int = 1024) -> List[Tuple[int, int, int]]:
    """(value id, element offset, element count) of every f32 initializer that
    travels in the blob, 64-element aligned so each lands 256-byte aligned.
    Small and integer initializers (shape tensors) stay host-side on every rank."""
    layout, off = [], 0
    for vid in sorted(model.graph.inits):
        arr = model.graph.inits[vid]
        if arr.dtype != np.float32 or arr.nbytes < min_bytes:
            continue
        layout.append((vid, off, arr.size))
        off += (arr.size + 63) // 64 * 64
    return layout


def pack_weights(model, layout) -> np.ndarray:
    total = (layout[-1][1] + (layout[-1][2] + 63) // 64 * 64) if layout else 0
    blob = np.zeros(total, np.float32)
    for vid, off, cnt in layout:
        blob[off:off + cnt] = model.graph.inits[vid].reshape(-1)
    return blob


def broadcast_weights(model, device, src: int = 0):
    """Broadcasts rank `src`'s packed f32 initializers to every rank. Returns
    (blob tensor, {value id: address}) -- the tensor must stay alive until the
    session has been created. `device` is a torch device ("cuda:N" or "cpu")."""
    import torch
    import torch.distributed as dist
    layout = pack_layout(model)
    blob_np = pack_weights(model, layout)
    if dist.get_rank() != src:
        blob_np = np.zeros_like(blob_np)   # receivers start from zeros: the bytes come from src
    blob = torch.from_numpy(blob_np).to(device)
    dist.broadcast(blob, src=src)
    base = blob.data_ptr()
    return blob, {vid: base + 4 * off for vid, off, _ in layout}


def unpack_into(model, blob_np: np.ndarray) -> None:
    """Host-side counterpart (CPU ranks): writes the blob back into the initializers."""
    for vid, off, cnt in pack_layout(model):
        arr = model.graph.inits[vid]
        model.graph.inits[vid] = blob_np[off:off + cnt].reshape(arr.shape).copy()


def gather_outputs(local: Sequence[np.ndarray], world_size: int) -> List[np.ndarray]:
    """Concatenates every rank's outputs along the batch axis on all ranks."""
    import torch
    import torch.distributed as dist
    outs = []
    for a in local:
        bucket = [None] * world_size
        dist.all_gather_object(bucket, np.ascontiguousarray(a))
        outs.append(np.concatenate(bucket, axis=0))
    return outs
