"""Partitioning decode sequences across the GPUs of one node.

Sequences are independent on this path: every CTA touches one sequence's pages
and nothing else.  Each rank therefore owns whole sequences together with their
KV pages (local page ids, its own pools), and no collective runs on the hot
path.  A gather to rank 0 exists for verification only.

Host-side integer logic; works with any torch.distributed backend (tests run it
under gloo on CPU).
"""

from __future__ import annotations


def partition_sequences(lengths, world_size, policy="snake"):
    """Assign sequence indices to ranks.

    policy "block": contiguous blocks of ceil(B / world) sequences, in order.
    policy "snake": sort by length (longest first) and deal 0..w-1, w-1..0, ...
    so every rank receives nearly the same number of KV pages; a log-uniform
    length mix dealt in blocks leaves the heaviest rank bounding the step time.
    Within a rank the sequences keep their order in the batch: a rank's batch sorted
    by length would put all its shortest sequences in the shares of a few CTAs of
    the persistent attention kernels, which pay a fixed cost per sequence.
    Returns a list of `world_size` lists of indices into `lengths`; every index
    appears exactly once.
    """
    if world_size < 1:
        raise ValueError("world_size must be positive")
    count = len(lengths)
    if policy == "block":
        per_rank = -(-count // world_size) if count else 0
        return [list(range(r * per_rank, min(count, (r + 1) * per_rank))) for r in range(world_size)]
    if policy != "snake":
        raise ValueError("policy must be 'block' or 'snake'")
    order = sorted(range(count), key=lambda i: (-int(lengths[i]), i))
    shards = [[] for _ in range(world_size)]
    for position, index in enumerate(order):
        lap, offset = divmod(position, world_size)
        rank = offset if lap % 2 == 0 else world_size - 1 - offset
        shards[rank].append(index)
    return [sorted(shard) for shard in shards]


def shard_pages(lengths, shards, page_size=16):
    """KV pages each rank must hold for its sequences."""
    return [sum(-(-int(lengths[i]) // page_size) for i in shard) for shard in shards]


def imbalance(lengths, shards):
    """max over ranks of attended tokens divided by the mean (1.0 = perfect)."""
    loads = [sum(int(lengths[i]) for i in shard) for shard in shards]
    mean = sum(loads) / max(1, len(loads))
    return max(loads) / mean if mean else 1.0


def gather_rows(local_rows, local_indices, total_rows, *, group=None, dst=0):
    """Verification helper: collect per-rank output rows on `dst` in global order.

    local_rows: tensor [n_local, ...] on any device; local_indices: the global
    sequence index of each row.  Returns the [total_rows, ...] tensor on `dst`
    (CPU) and None elsewhere.  Uses gather_object, so it is not for the hot path.
    """
    import torch
    import torch.distributed as dist

    payload = (list(map(int, local_indices)), local_rows.detach().cpu())
    if not (dist.is_available() and dist.is_initialized()):
        gathered = [payload]
        rank = dst
    else:
        rank = dist.get_rank(group)
        world = dist.get_world_size(group)
        gathered = [None] * world if rank == dst else None
        dist.gather_object(payload, gathered, dst=dst, group=group)
    if rank != dst:
        return None
    sample = next(rows for _, rows in gathered if rows.shape[0] > 0)
    full = torch.zeros((total_rows, *sample.shape[1:]), dtype=sample.dtype)
    seen = torch.zeros(total_rows, dtype=torch.bool)
    for indices, rows in gathered:
        if indices:
            index = torch.tensor(indices, dtype=torch.long)
            if seen[index].any():
                raise RuntimeError("a sequence was produced by more than one rank")
            full[index] = rows
            seen[index] = True
    if not seen.all():
        raise RuntimeError("some sequences were produced by no rank")
    return full


def localize_block_table(block_table, seq_lens, page_size=16):
    """Re-number the pages one rank's sequences use as 0..n-1.

    block_table: int tensor [b, width] with GLOBAL page ids (padding ignored);
    seq_lens: int tensor [b].  Returns (local_table, global_pages): local_table has
    the same shape with local ids (padding zero); global_pages[i] is the global id
    of local page i, so `pool[global_pages]` is the rank's own pool.
    """
    import torch

    local = torch.zeros_like(block_table)
    pages = []
    for row in range(block_table.shape[0]):
        count = -(-int(seq_lens[row]) // page_size)
        for column in range(count):
            local[row, column] = len(pages)
            pages.append(int(block_table[row, column]))
    if len(set(pages)) != len(pages):
        raise ValueError("a page is shared by two sequences; sequences cannot be sharded independently")
    return local, torch.tensor(pages, dtype=torch.long)
