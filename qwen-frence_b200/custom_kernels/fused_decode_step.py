"""One layer's decode step in two launches: RoPE + paged KV write folded into the
attention partial pass, then the split-K combine.

The reference runs this as two operators on one stream -- packed_qkv_rope_cache
(custom_kernels/packed_qkv_rope_cache.py:91-133) and then
grouped_splitk_decode_attention (custom_kernels/paged_decode_grouped_splitk.py:228-334),
engine/graph/paged_graph_decoder.py:234-289 -- and `packed_qkv_rope_attention` returns
exactly what that pair returns and leaves the pools exactly as it leaves them.  When
the tensor-core persistent kernel does not apply to the arguments (FP8 pools, split_k
1, an unusual layout) it runs the pair itself.
"""

from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

Q_HEADS, KV_HEADS, HEAD_DIM = 12, 2, 128
PACKED_WIDTH = (Q_HEADS + 2 * KV_HEADS) * HEAD_DIM


def _sibling(name, directory=None):
    key = f"qf_hotpath_{name.lstrip('_')}"
    module = sys.modules.get(key)
    if module is None:
        base = Path(__file__).resolve().parent if directory is None else directory
        spec = importlib.util.spec_from_file_location(key, base / f"{name}.py")
        module = importlib.util.module_from_spec(spec)
        sys.modules[key] = module
        spec.loader.exec_module(module)
    return module


def _require(condition, message):
    if not condition:
        raise ValueError(message)


_tables = {}


def build_rope_table(positions, *, base=1_000_000.0, device=None):
    """(cos, sin) fp32 pairs [positions, 64, 2] of every position and rotary frequency, with
    the expressions of the RoPE / KV-write kernel (so the fused step rotates to the same
    bits).  Cached per (device, base, positions); 512 bytes per position."""
    import torch

    cabi = _sibling("_cabi", Path(__file__).resolve().parents[1])
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (device.index, float(base), int(positions))
    table = _tables.get(key)
    if table is None:
        table = torch.empty((int(positions), HEAD_DIM // 2, 2), dtype=torch.float32, device=device)
        with cabi.device_of(table):
            cabi.check(cabi.library().qf_build_rope_table(
                table.data_ptr(), int(positions), float(base), cabi.stream_pointer(device)))
        _tables[key] = table
    return table


def packed_qkv_rope_attention(packed, positions, slot_mapping, k_pool, v_pool, block_table, seq_lens, *,
                              split_k, scale=None, base=1_000_000.0, partials=None, rope_table=None,
                              require_fused=False, check_slots=False):
    """RoPE Q/K of the packed rows, write K/V at token seq_lens - 1, attend over `block_table`.

    packed: (B, 2048) or (B, 1, 2048) fp16 / bf16, rows of [Q0..Q11 | K0 K1 | V0 V1];
    positions, slot_mapping, seq_lens: (B,); pools (pages, 16, 2, 128); block_table
    (B, max_blocks).  `slot_mapping[b]` must name token seq_lens[b] - 1 of sequence b in
    `block_table` (what the engine builds, engine/graph/paged_graph_decoder.py:392-417):
    the fused kernel derives the slot from the table and never reads `slot_mapping`, so a
    row whose slot is -1 or names another place is still written at the table's slot
    (the operator pair would skip it, or write elsewhere) -- such batches belong to the
    pair.  `check_slots=True` compares the two on the host first and raises ValueError on
    a difference (it synchronises: for debugging, not under graph capture).  It is a decode
    step: every attended token but the newest of each sequence must already be in the
    pools, written before the kernel in front of this call started (the kernel requests
    those older pages early).  Returns the attention output
    (B, 12, 128); the rotated queries are not materialised.  `rope_table`: the result of
    `build_rope_table` covering every position (default: a cached table of as many
    positions as the block table can hold -- build it before capturing a graph; positions
    must then be int32 / int64).  `require_fused=True` raises
    instead of running the two operators when the fused kernel does not apply.
    """
    import ctypes

    import torch

    cabi = _sibling("_cabi", Path(__file__).resolve().parents[1])
    attention = _sibling("paged_decode_grouped_splitk")
    if packed.ndim == 3:
        _require(packed.shape[1] == 1, "packed QKV must have one decode token per row")
        packed = packed[:, 0, :]
    _require(packed.ndim == 2 and packed.shape[1] == PACKED_WIDTH, "expected packed QKV shape (batch, 2048)")
    batch = packed.shape[0]
    _require(tuple(positions.shape) == (batch,) and tuple(slot_mapping.shape) == (batch,) and
             tuple(seq_lens.shape) == (batch,), "positions, slot_mapping and seq_lens must hold one entry per row")
    _require(packed.is_cuda, "packed QKV must live on a CUDA device")

    def pair():
        if require_fused:
            raise RuntimeError("the fused step does not apply to these arguments")
        q = _sibling("packed_qkv_rope_cache").packed_qkv_rope_cache(
            packed, positions, slot_mapping, k_pool, v_pool, base=base)
        return attention.grouped_splitk_decode_attention(
            q, k_pool, v_pool, block_table, seq_lens, split_k=split_k, scale=scale, partials=partials)

    fused_ok = (batch > 0 and int(split_k) >= 2 and k_pool.dtype == packed.dtype and packed.stride(1) == 1
                and tuple(k_pool.shape[1:]) == (16, KV_HEADS, HEAD_DIM)
                and k_pool.shape == v_pool.shape and block_table.ndim == 2 and block_table.shape[1] > 0
                and positions.dtype in (torch.int32, torch.int64))
    if not fused_ok:
        return pair()
    if check_slots:
        rows = torch.arange(batch, device=packed.device)
        last = (seq_lens.long() - 1).clamp_min(0)
        derived = block_table[rows, last // 16].long() * 16 + last % 16
        wrong = ((slot_mapping.long() != derived) & (seq_lens.long() > 0)).nonzero().flatten().tolist()
        _require(not wrong, f"slot_mapping differs from the block table's slot for rows {wrong[:8]}; "
                            "run packed_qkv_rope_cache and grouped_splitk_decode_attention instead")
    q_view = packed.as_strided((batch, Q_HEADS, HEAD_DIM), (packed.stride(0), HEAD_DIM, 1))
    out = torch.empty((batch, Q_HEADS, HEAD_DIM), dtype=packed.dtype, device=packed.device)
    if partials is None:
        shape = (batch, int(split_k), Q_HEADS, HEAD_DIM)
        partials = (torch.empty(shape, dtype=torch.float32, device=packed.device),
                    torch.empty(shape[:3], dtype=torch.float32, device=packed.device),
                    torch.empty(shape[:3], dtype=torch.float32, device=packed.device))
    args = attention.fill_attention_args(
        cabi, q_view, k_pool, v_pool, block_table, seq_lens, split_k=int(split_k),
        scale=HEAD_DIM ** -0.5 if scale is None else scale, partials=partials, out=out)
    if not cabi.fused_kernel_plan(args)[0].startswith("decode_mma_kernel"):
        return pair()
    positions = positions.contiguous()
    if rope_table is None:
        rope_table = build_rope_table(block_table.shape[1] * 16, base=base, device=packed.device)
    _require(rope_table.is_cuda and rope_table.dtype == torch.float32 and rope_table.is_contiguous()
             and tuple(rope_table.shape[1:]) == (HEAD_DIM // 2, 2), "rope_table must come from build_rope_table")
    with cabi.device_of(packed):
        cabi.check(cabi.library().qf_packed_rope_decode_attention(
            ctypes.byref(args), positions.data_ptr(), cabi.torch_index_code(positions.dtype),
            1, rope_table.data_ptr(), rope_table.shape[0], cabi.STAGE_PARTIAL | cabi.STAGE_COMBINE,
            cabi.stream_pointer(packed.device)))
    return out
