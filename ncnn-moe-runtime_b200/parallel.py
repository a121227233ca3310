"""Host-side plumbing for running the sampler on several GPUs of one box.

Two partitions, chosen by shape:

* rows     — large batches: every rank samples a contiguous block of rows.  Rows
             are independent, so there is no data-path collective.
* vocab    — very large vocabularies: every rank owns a contiguous slice of the
             vocabulary, extracts the stable Top-K of its slice
             (moe_sample_local_candidates), the k records per row are all-gathered
             (NCCL over NVLink) and every rank finishes the rows it is responsible
             for with moe_sample_merge_candidates.  The reference normalises over
             the k selected candidates only (src/engine/session.cpp:86-101), so no
             partial softmax sums have to cross GPUs.

The functions here only compute ranges and move tensors; torch.distributed is
the transport.
"""
from __future__ import annotations


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous [begin, end) of `total` items owned by `rank`; sizes differ by at most one."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def vocab_shard_range(vocab: int, world: int, rank: int, align: int = 16) -> tuple[int, int]:
    """Like shard_range, but interior boundaries fall on multiples of `align` logits
    so that every slice of a 32-byte aligned row starts 32-byte aligned."""
    blocks = (vocab + align - 1) // align
    begin_block, end_block = shard_range(blocks, world, rank)
    return min(vocab, begin_block * align), min(vocab, end_block * align)


def all_gather_candidates(local_candidates, group=None):
    """[rows, k] int64 records of this rank -> [world, rows, k] on every rank."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    rows = local_candidates.shape[0]
    # concatenated along dim 0 (the form every backend accepts), then viewed per rank
    gathered = torch.empty((world * rows,) + tuple(local_candidates.shape[1:]), dtype=local_candidates.dtype, device=local_candidates.device)
    dist.all_gather_into_tensor(gathered, local_candidates.contiguous(), group=group)
    return gathered.view((world, rows) + tuple(local_candidates.shape[1:]))


def agree_on_maximum(value: int, device="cpu", group=None) -> int:
    """The largest `value` any rank holds, on every rank (one all-reduce).

    For decisions every rank must take alike although each derives them from its own
    measurement — e.g. how often a timed CUDA graph that holds a collective is replayed:
    ranks that replay it a different number of times leave the collective unmatched and hang."""
    import torch
    import torch.distributed as dist

    holder = torch.tensor([int(value)], dtype=torch.int64, device=device)
    dist.all_reduce(holder, op=dist.ReduceOp.MAX, group=group)
    return int(holder.item())
