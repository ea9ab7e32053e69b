"""Device-side advance of the decode-step metadata of a stable cohort.

The reference keeps positions, lengths, slot mapping and block table in fixed
device buffers and, while the cohort of decoding requests does not change, moves
them on by one token with torch ops instead of rebuilding them on the host
(IterationLoop::advance_decode_state, engine/cpp/src/iteration_loop.cpp:500-528;
the K-step unrolled graph decoder holds the same sequence of tensors,
engine/graph/unrolled_graph_decoder.py:92-130).  `advance_decode_state` does that
update with one small kernel of libqf_hotpath.so, in place, and orders the
library's next launch after it.
"""

from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

PAGE_SIZE = 16


def _cabi():
    """The ctypes binding, loaded by path so this file works under any module name."""
    module = sys.modules.get("qf_hotpath_cabi")
    if module is None:
        path = Path(__file__).resolve().parents[1] / "_cabi.py"
        spec = importlib.util.spec_from_file_location("qf_hotpath_cabi", path)
        module = importlib.util.module_from_spec(spec)
        sys.modules["qf_hotpath_cabi"] = module
        spec.loader.exec_module(module)
    return module


def _require(condition, message):
    if not condition:
        raise ValueError(message)


def advance_decode_state(positions, seq_lens, slot_mapping, block_table, *,
                         block_size=PAGE_SIZE, num_pages=None):
    """positions += 1, seq_lens += 1, slot_mapping = slot of the new position, in place.

    positions, seq_lens, slot_mapping: (n,) contiguous CUDA int32 / int64 tensors
    (the reference holds int64, int32, int64); block_table: (n, max_blocks) int32 /
    int64, immutable for the cohort.  `num_pages` bounds the page ids (default: no
    bound beyond the int32 range of the table).  A position that leaves its table
    gets slot -1, which the KV-write kernel skips, and status 4 in
    `cabi.device_status()`; the reference's `gather` would raise there.
    Returns None, like the in-place torch ops it replaces.
    """
    import torch

    cabi = _cabi()
    n = positions.shape[0] if positions.ndim == 1 else -1
    _require(n >= 0 and tuple(seq_lens.shape) == (n,) and tuple(slot_mapping.shape) == (n,),
             "positions, seq_lens and slot_mapping must be 1-D with one entry per sequence")
    _require(block_table.ndim == 2 and block_table.shape[0] == n,
             "block_table must be (sequences, max_blocks)")
    _require(int(block_size) > 0, "block_size must be positive")
    tensors = (positions, seq_lens, slot_mapping, block_table)
    _require(all(t.is_cuda for t in tensors), "decode state must live on a CUDA device")
    _require(len({t.device for t in tensors}) == 1, "decode state must share one device")
    _require(all(t.dtype in (torch.int32, torch.int64) for t in tensors),
             "decode state must be int32 or int64")
    _require(all(t.is_contiguous() for t in tensors[:3]),
             "positions, seq_lens and slot_mapping must be contiguous")
    if num_pages is None:
        num_pages = 1 << 31
    with cabi.device_of(positions):
        cabi.check(cabi.library().qf_advance_decode_metadata(
            positions.data_ptr(), cabi.torch_index_code(positions.dtype),
            seq_lens.data_ptr(), cabi.torch_index_code(seq_lens.dtype),
            slot_mapping.data_ptr(), cabi.torch_index_code(slot_mapping.dtype),
            block_table.data_ptr(), cabi.torch_index_code(block_table.dtype),
            block_table.stride(0), block_table.stride(1), block_table.shape[1], int(num_pages),
            n, int(block_size), cabi.stream_pointer(positions.device)))
