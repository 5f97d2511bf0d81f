"""Host logic for the only natural shard of the token loop: independent
sequences.  Nothing couples sequences inside the forward pass (every op is per
row; the batch is only the leading axis, src/ops/matmul.rs:65-70), so each rank
owns a contiguous slice of the batch, a full copy of the weights and a private
KV cache, and no collective runs inside the loop.  The generated ids are
gathered once at the end."""
from __future__ import annotations

from typing import Tuple

import numpy as np


def shard_range(n_sequences: int, rank: int, world: int) -> Tuple[int, int]:
    """[lo, hi) of the sequences rank owns; the first n % world ranks get one more."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(n_sequences, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def gather_ids(local_ids: np.ndarray, n_sequences: int, rank: int, world: int, device=None) -> np.ndarray:
    """All-gather of the per-rank id arrays [n_local, G] into [n_sequences, G] (same
    on every rank).  Uses torch.distributed's default group (NCCL on GPUs, gloo in
    the CPU tests); ragged shards are padded to the largest."""
    if world == 1:
        return np.ascontiguousarray(local_ids)
    import torch
    import torch.distributed as dist
    G = local_ids.shape[1]
    most = max(shard_range(n_sequences, r, world)[1] - shard_range(n_sequences, r, world)[0] for r in range(world))
    buf = torch.zeros((most, G), dtype=torch.int64, device=device)
    if local_ids.shape[0]:
        buf[: local_ids.shape[0]] = torch.from_numpy(local_ids.astype(np.int64)).to(buf.device)
    out = [torch.empty_like(buf) for _ in range(world)]
    dist.all_gather(out, buf)
    rows = []
    for r in range(world):
        lo, hi = shard_range(n_sequences, r, world)
        rows.append(out[r][: hi - lo].cpu().numpy())
    return np.concatenate(rows, 0).astype(np.uint32)


def max_over_ranks(value: float, world: int, device=None) -> float:
    """Slowest rank's time: the figure every multi-GPU number is reported on."""
    if world == 1:
        return float(value)
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())
