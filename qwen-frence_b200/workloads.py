"""Seeded synthetic decode workloads with the shapes, sizes and value
distributions of the five benchmark configurations.  No dataset or checkpoint
is involved: the reference measures this path on synthetic tensors too
(experiments/decode/grouped_splitk_validation.py:6-40,
experiments/decode/benchmark_native_grouped_decode.py:112-135).

A workload is host-side data only (torch CPU tensors); DecodeStep places it on a
device.  Values are N(0,1) * 0.5 in fp16; RoPE theta 1e6; positions = context
length; seq_lens = context + 1 (the new token attends to itself).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from . import kv_layout, sharding

WORKLOADS = {
    # name: (layers, batch, context sampler, fp8, description)
    "cpu_single_layer_b8": dict(layers=1, batch=8, fp8=False,
                                doc="1 layer, batch 8, context 512, 512-page pool"),
    "decode_b64": dict(layers=28, batch=64, fp8=False,
                       doc="28 layers, batch 64, context uniform in [128, 4096]"),
    "sweep_b256": dict(layers=28, batch=256, fp8=False,
                       doc="28 layers, batch 256, context log-uniform in [64, 8192], "
                           "pool of 8192*256/16 pages filled to ~90%"),
    "long_skew_b4": dict(layers=28, batch=4, fp8=False,
                         doc="28 layers, batch 4, contexts 32768/16384/4096/512"),
    "fp8_b128": dict(layers=28, batch=128, fp8=True,
                     doc="28 layers, batch 128, context 2048, e4m3 pools with per-page scales"),
    # not one of the five benchmark configurations: the many-short-sequences regime
    "short_b512": dict(layers=28, batch=512, fp8=False,
                       doc="28 layers, batch 512, context 100 (seven pages per sequence)"),
}


def context_lengths(name, seed=0, batch=None):
    """Context length (tokens already cached) of every sequence of a workload."""
    spec = WORKLOADS[name]
    batch = spec["batch"] if batch is None else batch
    generator = torch.Generator().manual_seed(1000 + seed)
    if name == "cpu_single_layer_b8":
        return [512] * batch
    if name == "decode_b64":
        return torch.randint(128, 4097, (batch,), generator=generator).tolist()
    if name == "sweep_b256":
        u = torch.rand(batch, generator=generator, dtype=torch.float64)
        lengths = torch.exp(math.log(64) + u * (math.log(8192) - math.log(64)))
        return lengths.round().clamp(64, 8192).long().tolist()
    if name == "long_skew_b4":
        base = [32768, 16384, 4096, 512]
        return [base[i % 4] for i in range(batch)]
    if name == "fp8_b128":
        return [2048] * batch
    if name == "short_b512":
        return [100] * batch
    raise KeyError(name)


@dataclass
class Workload:
    """Host-side description of one rank's share of a decode step."""

    name: str
    layers: int
    fp8: bool
    contexts: list            # context length per local sequence
    global_indices: list      # index of each local sequence in the global batch
    num_pages: int            # pool pages per layer on this rank
    block_table: torch.Tensor  # int32 [B, max_blocks], zero padded, LOCAL page ids
    seq_lens: torch.Tensor     # int32 [B] = context + 1
    positions: torch.Tensor    # int32 [B] = context
    slot_mapping: torch.Tensor  # int64 [B]
    live_pages: torch.Tensor   # int64 [n]: pages that hold cached tokens
    seed: int = 0
    meta: dict = field(default_factory=dict)

    @property
    def value_seed(self):
        """Seed of the K/V and packed-row values: differs between ranks."""
        return self.seed + 7919 * int(self.meta.get("rank", 0))

    @property
    def batch(self):
        return len(self.contexts)

    @property
    def max_context(self):
        return max(self.contexts) + 1 if self.contexts else 1


def build_workload(name, *, rank=0, world_size=1, scaling="weak", seed=0, layers=None,
                   batch=None, pool_pages=None, shard_policy="snake", reserve_tokens=0):
    """Build rank `rank`'s share of workload `name`.

    scaling "weak": every rank gets its own full-size batch with the SAME context
    lengths in the same order (equal cost per rank, so a scaling curve measures the
    machine and not the draw) but its own page permutation and values.  scaling "strong": the global batch is partitioned by sequence with
    `sharding.partition_sequences`; each rank owns its sequences' pages.
    Page ids are local to the rank.  The pool is filled through a PagePool whose
    free list is randomly permuted first, so block tables are a seeded random
    permutation of the pool.  `reserve_tokens` > 0 reserves pages for that many
    further tokens per sequence at admission (block tables then cover the tokens
    that consecutive decode steps will append, as the reference's engine does for a
    stable cohort, engine/cpp/src/iteration_loop.cpp:512-514).
    """
    spec = WORKLOADS[name]
    layers = spec["layers"] if layers is None else layers
    if scaling == "weak":
        contexts = context_lengths(name, seed=seed, batch=batch)
        global_indices = [rank * len(contexts) + i for i in range(len(contexts))]
    elif scaling == "strong":
        everyone = context_lengths(name, seed=seed, batch=batch)
        shards = sharding.partition_sequences([c + 1 for c in everyone], world_size, shard_policy)
        global_indices = shards[rank]
        contexts = [everyone[i] for i in global_indices]
    else:
        raise ValueError("scaling must be 'weak' or 'strong'")

    local_batch = len(contexts)
    lengths = [c + 1 for c in contexts]
    reserved = [n + int(reserve_tokens) for n in lengths]
    needed = sum(-(-n // kv_layout.PAGE_SIZE) for n in reserved)
    if pool_pages is None:
        if name == "cpu_single_layer_b8":
            pool_pages = 512
        elif name == "sweep_b256":
            pool_pages = (8192 * 256 // kv_layout.PAGE_SIZE) // (world_size if scaling == "strong" else 1)
        else:
            pool_pages = needed + 64
    pool_pages = max(pool_pages, needed, 1)

    generator = torch.Generator().manual_seed(2000 + seed + 104729 * rank)
    pool = kv_layout.PagePool(max(local_batch, 1), pool_pages, max_seq_len=1 << 20)
    order = torch.randperm(pool_pages, generator=generator).tolist()
    pool.free_pages = order  # allocation pops from the end of a shuffled list
    filler = 0
    if name == "sweep_b256":
        # ~90% of the pool is allocated: live sequences plus filler allocations that
        # the step never reads, scattered among them by the permutation.
        filler = max(0, int(0.9 * pool_pages) - needed)
        del pool.free_pages[:filler]
    if local_batch:
        pool.allocate(reserved)
    max_blocks = max([len(t) for t in pool.block_tables] + [1])
    if local_batch:
        positions, seq_lens, table, slots = kv_layout.decode_step_inputs(
            lengths, pool.block_tables, max_blocks)
    else:
        import numpy as np

        positions = np.zeros(0, dtype=np.int32)
        seq_lens = np.zeros(0, dtype=np.int32)
        table = np.zeros((0, max_blocks), dtype=np.int32)
        slots = np.zeros(0, dtype=np.int64)
    live = sorted({page for t in pool.block_tables for page in t})
    return Workload(
        name=name, layers=layers, fp8=spec["fp8"], contexts=contexts,
        global_indices=global_indices, num_pages=pool_pages,
        block_table=torch.from_numpy(table), seq_lens=torch.from_numpy(seq_lens),
        positions=torch.from_numpy(positions), slot_mapping=torch.from_numpy(slots),
        live_pages=torch.tensor(live, dtype=torch.long), seed=seed,
        meta=dict(scaling=scaling, world_size=world_size, rank=rank, filler_pages=filler,
                  reserve_tokens=int(reserve_tokens),
                  doc=spec["doc"]),
    )


def packed_qkv_rows(workload, layer, device, dtype=torch.float16):
    """The packed [B, 2048] QKV row of `layer`: random hidden states [B, 1536]
    through a random [2048, 1536] * 0.02 projection with bias, as in the
    reference's fusion benchmark (experiments/model/... random-weight geometry;
    no checkpoint is available offline).  Setup work, never timed."""
    generator = torch.Generator(device="cpu").manual_seed(3000 + workload.value_seed * 131 + layer)
    hidden = torch.randn(workload.batch, kv_layout.HIDDEN, generator=generator)
    weight = torch.randn(2048, kv_layout.HIDDEN, generator=generator) * 0.02
    bias = torch.randn(2048, generator=generator) * 0.1
    packed = hidden.to(device) @ weight.to(device).T + bias.to(device)
    # bring the projection to the N(0,1)*0.5 scale of the cached K/V
    packed = packed / packed.std().clamp_min(1e-6) * 0.5
    return packed.to(dtype)
