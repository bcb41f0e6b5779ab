"""Data-parallel plumbing: images are independent units, so ranks only need a deterministic
partition of the batch and one gather of the embeddings.  No kernel reads another GPU's memory."""
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n_items: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [start, stop) slice of ``n_items`` owned by ``rank``; sizes differ by at most one and
    earlier ranks take the remainder (empty slices are allowed when n_items < world)."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    base, rem = divmod(n_items, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def gather_embeddings(local: torch.Tensor, group: Optional[dist.ProcessGroup] = None,
                      out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """All ranks hold ``local [b, C, h, w]`` (same shape); returns ``[world*b, C, h, w]`` in rank order
    on every rank.  One ``all_gather_into_tensor`` (NCCL on GPUs, gloo in the CPU tests)."""
    world = dist.get_world_size(group)
    local = local.contiguous()
    if out is None:
        out = local.new_empty((world * local.shape[0],) + tuple(local.shape[1:]))
    dist.all_gather_into_tensor(out, local, group=group)
    return out


def gather_ragged(local: torch.Tensor, counts: List[int], group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Gather slices whose leading sizes differ per rank (``counts[r]`` items on rank r): pad to the
    largest slice, gather, and drop the padding."""
    world = dist.get_world_size(group)
    if len(counts) != world or counts[dist.get_rank(group)] != local.shape[0]:
        raise ValueError("counts must list every rank's slice size")
    mx = max(counts)
    padded = local.new_zeros((mx,) + tuple(local.shape[1:]))
    padded[: local.shape[0]] = local
    full = gather_embeddings(padded, group)
    return torch.cat([full[r * mx: r * mx + c] for r, c in enumerate(counts)], dim=0)
