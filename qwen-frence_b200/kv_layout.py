"""Host-side layout of the paged KV cache: page allocator, per-step metadata and
the split-K policy.  Integer work only; nothing here touches a GPU.

Pool layout (engine/kvcache/paged_kv_cache.py:31-37,
experiments/integration/model_adapter.py:14-20): per layer two tensors
[num_pages, 16, kv_heads, 128]; token `p` of a sequence lives in page
`table[p // 16]` at row `p % 16`, i.e. flat slot `table[p // 16] * 16 + p % 16`.
"""

from __future__ import annotations

import numpy as np

PAGE_SIZE = 16
Q_HEADS, KV_HEADS, HEAD_DIM, LAYERS, HIDDEN = 12, 2, 128, 28, 1536
MAX_SEQ_LEN = 32768

# Frozen split-K action of the reference engine
# (engine/kvcache/paged_decode_attention.py:34-40).
SPLITK_PAGE_THRESHOLD = 80
SPLITK_ACTIONS = {"short": {"split_k": 8, "num_stages": 2},
                  "long": {"split_k": 22, "num_stages": 3}}


class CacheFullError(RuntimeError):
    """The page pool is exhausted: a capacity signal for a scheduler, not a bug
    (engine/kvcache/paged_kv_cache.py:6-8)."""


class PagePool:
    """Page allocator with the reference's semantics
    (engine/kvcache/paged_kv_cache.py:56-111): LIFO free list popped from the
    end, all-or-nothing growth of every sequence at once, free / truncate /
    reset.  Owns no tensors: pools are allocated by the caller per layer."""

    def __init__(self, batch_size, num_pages, page_size=PAGE_SIZE, max_seq_len=MAX_SEQ_LEN):
        self.batch_size = batch_size
        self.num_pages = num_pages
        self.page_size = page_size
        self.max_seq_len = max_seq_len
        self.reset()

    def reset(self):
        self.free_pages = list(range(self.num_pages))
        self.block_tables = [[] for _ in range(self.batch_size)]
        self.cur_lens = [0] * self.batch_size

    def pages_needed(self, length):
        return (length - 1) // self.page_size + 1 if length > 0 else 0

    def allocate(self, new_tokens):
        """Grow every sequence b by new_tokens[b]; raises before mutating anything."""
        if len(new_tokens) != self.batch_size:
            raise ValueError("one token count per sequence is required")
        total = 0
        for b, extra in enumerate(new_tokens):
            new_len = self.cur_lens[b] + extra
            if new_len > self.max_seq_len:
                raise ValueError(
                    f"sequence {b} would reach {new_len} tokens, exceeds "
                    f"max_seq_len={self.max_seq_len}")
            total += max(0, self.pages_needed(new_len) - len(self.block_tables[b]))
        if total > len(self.free_pages):
            raise CacheFullError(f"need {total} new blocks, only {len(self.free_pages)} free")
        for b, extra in enumerate(new_tokens):
            new_len = self.cur_lens[b] + extra
            table = self.block_tables[b]
            while len(table) < self.pages_needed(new_len):
                table.append(self.free_pages.pop())
            self.cur_lens[b] = new_len

    def free(self, b):
        self.free_pages.extend(self.block_tables[b])
        self.block_tables[b] = []
        self.cur_lens[b] = 0

    def truncate(self, b, new_len):
        if not 0 <= new_len <= self.cur_lens[b]:
            raise ValueError(f"cannot truncate slot {b} from {self.cur_lens[b]} to {new_len}")
        keep = (new_len + self.page_size - 1) // self.page_size
        self.free_pages.extend(self.block_tables[b][keep:])
        self.block_tables[b] = self.block_tables[b][:keep]
        self.cur_lens[b] = new_len


def decode_step_inputs(cur_lens, block_tables, max_blocks, page_size=PAGE_SIZE):
    """Metadata of one decode step, as the engine builds it
    (engine/graph/paged_graph_decoder.py:392-417; C++ twin
    engine/cpp/src/iteration_loop.cpp:402-473).

    cur_lens[b] already counts the token being decoded.  Returns numpy arrays
    positions int32 [B] (= cur-1), seq_lens int32 [B] (= cur),
    block_table int32 [B, max_blocks] zero padded, slot_mapping int64 [B].
    """
    batch = len(cur_lens)
    positions = np.empty(batch, dtype=np.int32)
    seq_lens = np.empty(batch, dtype=np.int32)
    slot_mapping = np.empty(batch, dtype=np.int64)
    table = np.zeros((batch, max_blocks), dtype=np.int32)
    for b, (cur, pages) in enumerate(zip(cur_lens, block_tables)):
        if cur < 1:
            raise ValueError(f"sequence {b} has no token to decode")
        if len(pages) > max_blocks:
            raise ValueError(f"sequence {b} holds {len(pages)} pages, more than max_blocks={max_blocks}")
        position = cur - 1
        positions[b] = position
        seq_lens[b] = cur
        slot_mapping[b] = pages[position // page_size] * page_size + position % page_size
        table[b, :len(pages)] = pages
    return positions, seq_lens, table, slot_mapping


def select_splitk_config(max_context_length, page_size=PAGE_SIZE):
    """The reference engine's frozen split-K action for a host context bound
    (engine/kvcache/paged_decode_attention.py:62-73)."""
    if max_context_length is None or max_context_length < 1:
        raise ValueError("split-K configuration requires a positive host context length")
    pages = -(-max_context_length // page_size)
    action = SPLITK_ACTIONS["short" if pages <= SPLITK_PAGE_THRESHOLD else "long"]
    return {**action, "heads_per_program": 1, "num_warps": 4}


def plan_split_k(batch, max_context_length, *, kv_heads=KV_HEADS, page_size=PAGE_SIZE,
                 sm_count=148, ctas_per_sm=2, waves=4, min_pages_per_split=8):
    """Split count for the B200 kernels from host-known bounds only (capture safe).

    Aim for `waves` full waves of resident CTAs (sm_count * ctas_per_sm each)
    over the batch * kv_heads (sequence, KV head) pairs, but never cut a
    sequence into partitions shorter than `min_pages_per_split` pages: each CTA
    pays a fixed merge cost worth about two pages of work.
    """
    if batch < 1 or max_context_length < 1:
        raise ValueError("batch and context bound must be positive")
    pages = -(-max_context_length // page_size)
    wanted = -(-(sm_count * ctas_per_sm * waves) // (batch * kv_heads))
    cap = max(1, pages // min_pages_per_split)
    split_k = int(max(1, min(wanted, cap, 65535)))
    # Many short sequences: the persistent kernel (which needs split_k >= 2; a slot it does not
    # fill costs nothing) instead of one CTA per sequence and KV head.
    if pages <= SHORT_TABLE_PAGES and batch >= SHORT_MIN_BATCH:
        split_k = max(split_k, 3)
    return split_k


# Widest block table (pages) and smallest batch for which plan_split_k keeps a batch of short
# sequences on the persistent kernel (split_k >= 3) instead of one CTA per sequence and KV head
# (split_k 1): measured per layer, attention call alone, 256 x 200 tokens 15.4 against 26.1 us,
# 512 x 100 15.7 against 30.2, 1 024 x 60 19.8 against 40.6; 64 x 200 13.1 against 10.9.
SHORT_TABLE_PAGES = 64
SHORT_MIN_BATCH = 256


# Empty units the tensor-core persistent kernel counts per sequence when it cuts the
# shares: min(TENSOR_CORE_PIECE_OVERHEAD, pages // 4) (kPieceOverhead and
# sequence_overhead() in csrc/; the per-CTA timeline test pins the two).
TENSOR_CORE_PIECE_OVERHEAD = 6


def sequence_overhead(data_units, overhead_units):
    """Empty units in front of a sequence of `data_units` in a persistent kernel's list."""
    return min(overhead_units, data_units // 4)


def persistent_schedule(seq_lens, *, split_k, ctas_per_head, unit_tokens=PAGE_SIZE, overhead_units=0):
    """Host restatement of how the persistent partial kernels cut one KV head's work.

    A sequence with tokens is `sequence_overhead(units, overhead_units)` empty units
    (the fixed cost a CTA pays per sequence; 0 for the CUDA-core kernel) followed by
    its data units (pages for
    the tensor-core kernel, page pairs for the CUDA-core one).  The sequences are
    concatenated; CTA c takes units [c*share, (c+1)*share) with
    share = max(ceil(total / ctas_per_head), ceil(longest / (split_k - 1))), so no
    sequence is cut into more than split_k pieces.  Returns (share, pieces) where a
    piece is (cta, sequence, first data unit within the sequence, data units, split
    slot); slots count from the CTA that holds the sequence's first data unit.
    """
    if split_k < 2 or ctas_per_head < 1:
        raise ValueError("the persistent kernels need split_k >= 2 and at least one CTA per head")
    data = [-(-max(int(t), 0) // unit_tokens) for t in seq_lens]
    empty = [sequence_overhead(count, overhead_units) for count in data]
    units = [count + extra for count, extra in zip(data, empty)]
    total, longest = sum(units), max(units, default=0)
    if total == 0:
        return 0, []
    share = max(-(-total // ctas_per_head), -(-longest // (split_k - 1)))
    pieces, first = [], 0
    for sequence, count in enumerate(data):
        if count:
            start = first + empty[sequence]  # the sequence's first data unit
            position = start
            while position < start + count:
                cta = position // share
                stop = min(start + count, (cta + 1) * share)
                pieces.append((cta, sequence, position - start, stop - position, cta - start // share))
                position = stop
        first += units[sequence]
    return share, pieces


def solo_schedule(seq_lens, *, split_k, ctas_per_head, unit_tokens=PAGE_SIZE):
    """Host restatement of how the tensor-core kernel's solo variant cuts one KV head's work.

    The unit list and the CTAs' shares are those of persistent_schedule with
    TENSOR_CORE_PIECE_OVERHEAD empty units per sequence.  Inside a CTA the eight warps stream
    consecutive blocks of share // 8 (the first share % 8 of them one more) units on their own,
    and what they hold of one sequence is merged at the CTA's end into ONE piece, which goes to
    split slot (the CTA) - (the CTA that holds the sequence's first page): the pieces are those
    of the variant whose warps interleave over the units.  Returns (share, pieces), a piece
    being (cta, sequence, first page within the sequence, pages, split slot)."""
    return persistent_schedule(seq_lens, split_k=split_k, ctas_per_head=ctas_per_head, unit_tokens=unit_tokens,
                               overhead_units=TENSOR_CORE_PIECE_OVERHEAD)


def kv_bytes_per_layer(seq_lens, *, kv_heads=KV_HEADS, head_dim=HEAD_DIM, elem_bytes=2):
    """Unique K+V bytes one layer's attention must read: sum_b T_b * 2 * kv * D * e
    (same count as unique_bytes in
    experiments/decode/benchmark_native_grouped_decode.py:177)."""
    return int(sum(int(t) for t in seq_lens)) * 2 * kv_heads * head_dim * elem_bytes


def algorithmic_bytes_per_layer(seq_lens, *, split_k, page_size=PAGE_SIZE, q_heads=Q_HEADS,
                                kv_heads=KV_HEADS, head_dim=HEAD_DIM, fp8=False):
    """All bytes one layer of the hot path must move (KV write + attention):
    K/V pages, block table, FP8 scales, Q in/out, the packed QKV row read and the
    Q / K / V row writes, and the split-K partials (written, then read)."""
    elem = 1 if fp8 else 2
    batch = len(seq_lens)
    total = kv_bytes_per_layer(seq_lens, kv_heads=kv_heads, head_dim=head_dim, elem_bytes=elem)
    pages = sum(-(-int(t) // page_size) for t in seq_lens)
    total += pages * 4
    if fp8:
        total += pages * 2 * kv_heads * 4
    width = (q_heads + 2 * kv_heads) * head_dim
    total += batch * (2 * q_heads * head_dim * 2)  # attention: Q in, out
    total += batch * (width * 2 + q_heads * head_dim * 2 + 2 * kv_heads * head_dim * elem + 12)
    if split_k > 1:
        total += 2 * batch * split_k * q_heads * (head_dim + 2) * 4
    return int(total)
