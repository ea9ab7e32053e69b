"""Packed-QKV post-GEMM epilogue: RoPE Q/K and direct paged K/V writes.

Drop-in for custom_kernels/packed_qkv_rope_cache.py: same function name,
signature and ValueError behaviour, so baseline/kernel_dispatch.py:141-143 and
engine/graph/paged_graph_decoder.py:234-241 call it unchanged.  A packed row is
[Q0..Q11 | K0 K1 | V0 V1], sixteen 128-wide segments; K and V each restart their
cache-head index at zero.  Rows at or beyond `*valid_tokens` return zero queries
and never touch the cache (token-bucket CUDA graphs replay with fewer live rows
than they captured).  The work is done by `qf_rope_kv_write` in
libqf_hotpath.so, pointed at the three column ranges of the packed row.
"""

from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

Q_HEADS, KV_HEADS, HEAD_DIM, PAGE_SIZE = 12, 2, 128, 16
PACKED_WIDTH = (Q_HEADS + 2 * KV_HEADS) * HEAD_DIM  # 2048


def _sibling(name):
    """Load a sibling module by path so this file works under any module name."""
    key = f"qf_hotpath_{name}"
    module = sys.modules.get(key)
    if module is None:
        path = Path(__file__).resolve().parent / f"{name}.py"
        spec = importlib.util.spec_from_file_location(key, path)
        module = importlib.util.module_from_spec(spec)
        sys.modules[key] = module
        spec.loader.exec_module(module)
    return module


def _require(condition, message):
    if not condition:
        raise ValueError(message)


def packed_qkv_rope_cache(
    packed, positions, slot_mapping, k_pool, v_pool,
    *, base=1_000_000.0, num_warps=4, valid_tokens=None,
):
    """Consume packed QKV GEMM output without split/transpose/materialisation.

    packed: (rows, 2048) or (rows, 1, 2048); positions, slot_mapping: (rows,);
    pools: (pages, 16, 2, 128); valid_tokens: optional CUDA int32 scalar.
    Returns q (rows, 12, 128), contiguous.  Mirrors
    custom_kernels/packed_qkv_rope_cache.py:91-133.
    """
    import torch

    if packed.ndim == 3:
        _require(packed.shape[1] == 1, "packed QKV must have one decode token per row")
        packed = packed[:, 0, :]
    _require(packed.ndim == 2 and packed.shape[1] == PACKED_WIDTH,
             "expected packed QKV shape (batch, 2048)")
    rows = packed.shape[0]
    _require(tuple(positions.shape) == (rows,) and tuple(slot_mapping.shape) == (rows,),
             "positions and slots must contain one value per row")
    _require(k_pool.shape == v_pool.shape
             and tuple(k_pool.shape[1:]) == (PAGE_SIZE, KV_HEADS, HEAD_DIM),
             "expected matching page-16 Qwen K/V pools")
    if valid_tokens is not None:
        _require(valid_tokens.ndim == 0 and valid_tokens.dtype == torch.int32
                 and valid_tokens.is_cuda and valid_tokens.device == packed.device,
                 "valid_tokens must be a CUDA int32 scalar")
    operands = (packed, positions, slot_mapping, k_pool, v_pool)
    _require(all(t.is_cuda and t.device == packed.device for t in operands),
             "packed QKV epilogue tensors must share one CUDA device")
    _require(packed.dtype in (torch.float16, torch.bfloat16),
             "packed QKV epilogue supports FP16 and BF16")
    _require(all(t.dtype == packed.dtype for t in (k_pool, v_pool)),
             "packed QKV and KV pools must share a dtype")
    _require(positions.dtype in (torch.int32, torch.int64, torch.float32),
             "positions must be int32, int64, or float32")
    _require(slot_mapping.dtype in (torch.int32, torch.int64),
             "slots must use an integer dtype")

    q = torch.empty(rows, Q_HEADS, HEAD_DIM, device=packed.device, dtype=packed.dtype)
    if rows == 0:
        return q
    row_stride, col_stride = packed.stride()
    segment = (row_stride, HEAD_DIM * col_stride, col_stride)  # (row, head, d) strides
    _sibling("rope_kv_write")._launch(
        packed[:, : Q_HEADS * HEAD_DIM],
        packed[:, Q_HEADS * HEAD_DIM: (Q_HEADS + KV_HEADS) * HEAD_DIM],
        packed[:, (Q_HEADS + KV_HEADS) * HEAD_DIM:],
        q, segment, segment, segment, tuple(q.stride()),
        positions, slot_mapping, k_pool, v_pool,
        rows=rows, q_heads=Q_HEADS, kv_heads=KV_HEADS, head_dim=HEAD_DIM,
        rotate_q=True, base=base, valid_tokens=valid_tokens,
    )
    return q
