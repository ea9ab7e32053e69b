"""FP8-e4m3 paged KV cache with one fp32 scale per (page, KV head).

The reference has no per-page-scale paged FP8 cache; its nearest pieces are the
e4m3 codec (experiments/quant/attention.py:27-50) and the fixed-scale cache
write (experiments/quant/kernels/staged_cache.py:39-55).  This module defines
the layout and keeps the conventions of the 16-bit entry points:

    k8_pool, v8_pool : uint8 (or torch.float8_e4m3fn) [pages, 16, Hkv, 128]
    k_scale, v_scale : float32 [pages, Hkv]
    byte  = e4m3_rn_satfinite(clamp(x / scale, -448, 448))
    x_hat = float(byte) * scale

Attention dequantises in-kernel: the K scale multiplies the reduced score and
the V scale multiplies the probability, once per page, so no dequantised copy
of the cache is ever written.  Queries and outputs stay fp16/bf16.
"""

from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

E4M3_MAX = 448.0


def _sibling(name, directory=None):
    """Load a module of this package by path, under a stable private name."""
    key = f"qf_hotpath_{name.lstrip('_')}"
    module = sys.modules.get(key)
    if module is None:
        base = Path(__file__).resolve().parent if directory is None else directory
        spec = importlib.util.spec_from_file_location(key, base / f"{name}.py")
        module = importlib.util.module_from_spec(spec)
        sys.modules[key] = module
        spec.loader.exec_module(module)
    return module


def _cabi():
    return _sibling("_cabi", Path(__file__).resolve().parents[1])


def _require(condition, message):
    if not condition:
        raise ValueError(message)


def _as_bytes(torch, pool):
    if pool.dtype == torch.uint8:
        return pool
    _require(pool.dtype == torch.float8_e4m3fn, "FP8 pools must be uint8 or float8_e4m3fn")
    return pool.view(torch.uint8)


def _check_fp8_pools(torch, k8_pool, v8_pool, k_scale, v_scale):
    _require(k8_pool.ndim == 4 and k8_pool.shape == v8_pool.shape,
             "K/V pools must have matching rank-four shapes")
    pages, _, kv_heads, _ = k8_pool.shape
    for scale in (k_scale, v_scale):
        _require(tuple(scale.shape) == (pages, kv_heads) and scale.dtype == torch.float32
                 and scale.is_contiguous(),
                 "scales must be contiguous float32 [pages, kv_heads]")
    operands = (k8_pool, v8_pool, k_scale, v_scale)
    _require(all(t.is_cuda and t.device == k8_pool.device for t in operands),
             "FP8 pools and scales must share one CUDA device")


def quantize_kv_pool_e4m3(pool):
    """Quantise a contiguous fp16/bf16 pool [pages, page, Hkv, D] page by page.

    Returns (bytes uint8 [pages, page, Hkv, D], scales float32 [pages, Hkv]) with
    scale = max(amax(page, head) / 448, 1e-12).
    """
    import torch

    _require(pool.ndim == 4 and pool.is_contiguous(), "pool must be a contiguous rank-four tensor")
    _require(pool.is_cuda, "pool must be a CUDA tensor")
    _require(pool.dtype in (torch.float16, torch.bfloat16), "pool must be float16 or bfloat16")
    cabi = _cabi()
    pages, page_size, kv_heads, dim = pool.shape
    pool8 = torch.empty(pool.shape, dtype=torch.uint8, device=pool.device)
    scales = torch.empty((pages, kv_heads), dtype=torch.float32, device=pool.device)
    with cabi.device_of(pool):
        cabi.check(cabi.library().qf_quantize_kv_pages_e4m3(
            pool.data_ptr(), cabi.torch_dtype_code(pool.dtype), pages, page_size, kv_heads, dim,
            pool8.data_ptr(), scales.data_ptr(), cabi.stream_pointer(pool.device)))
    return pool8, scales


def dequantize_kv_pool_e4m3(pool8, scales, dtype=None):
    """x_hat = float(byte) * scale, rounded to `dtype` (default float16).

    A verification helper built from torch ops; attention never calls it.
    """
    import torch

    dtype = torch.float16 if dtype is None else dtype
    values = _as_bytes(torch, pool8).view(torch.float8_e4m3fn).float()
    return (values * scales[:, None, :, None]).to(dtype)


def native_decode_rope_kv_write_fp8(
    q, k, v, positions, slot_mapping, k8_pool, v8_pool, k_scale, v_scale,
    *, base=1_000_000.0, rotate_q=True,
):
    """RoPE Q/K for (B, H, 1, D) decode tensors; quantise K (rotated) and V with the
    page's fixed scale into the FP8 pools.  Returns rotated Q (or q when rotate_q=False)."""
    import torch

    _require(all(t.ndim == 4 and t.shape[2] == 1 for t in (q, k, v)),
             "decode Q/K/V must have shape (batch, heads, 1, dim)")
    batch, q_heads, _, dim = q.shape
    kv_heads = k.shape[1]
    _require(k.shape == v.shape and k.shape[0] == batch and k.shape[-1] == dim,
             "decode K/V shapes do not match Q")
    _require(tuple(positions.shape) == (batch,) and tuple(slot_mapping.shape) == (batch,),
             "positions and slots must contain one entry per batch row")
    _check_fp8_pools(torch, k8_pool, v8_pool, k_scale, v_scale)
    _require(tuple(k8_pool.shape[2:]) == (kv_heads, dim) and k8_pool.is_contiguous()
             and v8_pool.is_contiguous(),
             "K/V pools must be contiguous with matching KV dimensions")
    _require(q.dtype in (torch.float16, torch.bfloat16)
             and k.dtype == q.dtype and v.dtype == q.dtype,
             "Q/K/V must share FP16 or BF16 dtype")
    _require(dim % 16 == 0 and dim <= 256,
             "head dimension must be a multiple of 16 no larger than 256")
    out = torch.empty_like(q) if rotate_q else q
    _sibling("rope_kv_write")._launch(
        q if rotate_q else None, k, v, out if rotate_q else None,
        (q.stride(0), q.stride(1), q.stride(3)),
        (k.stride(0), k.stride(1), k.stride(3)),
        (v.stride(0), v.stride(1), v.stride(3)),
        (out.stride(0), out.stride(1), out.stride(3)),
        positions, slot_mapping, _as_bytes(torch, k8_pool), _as_bytes(torch, v8_pool),
        rows=batch, q_heads=q_heads, kv_heads=kv_heads, head_dim=dim, rotate_q=rotate_q,
        base=base, fp8_scales=(k_scale, v_scale), page_size=k8_pool.shape[1],
    )
    return out


def packed_qkv_rope_cache_fp8(
    packed, positions, slot_mapping, k8_pool, v8_pool, k_scale, v_scale,
    *, base=1_000_000.0, valid_tokens=None,
):
    """packed_qkv_rope_cache for FP8 pools: packed (rows, 2048) -> q (rows, 12, 128)."""
    import torch

    if packed.ndim == 3:
        _require(packed.shape[1] == 1, "packed QKV must have one decode token per row")
        packed = packed[:, 0, :]
    _require(packed.ndim == 2 and packed.shape[1] == 2048, "expected packed QKV shape (batch, 2048)")
    rows = packed.shape[0]
    _require(tuple(positions.shape) == (rows,) and tuple(slot_mapping.shape) == (rows,),
             "positions and slots must contain one value per row")
    _check_fp8_pools(torch, k8_pool, v8_pool, k_scale, v_scale)
    _require(tuple(k8_pool.shape[1:]) == (16, 2, 128), "expected matching page-16 Qwen K/V pools")
    _require(packed.dtype in (torch.float16, torch.bfloat16),
             "packed QKV epilogue supports FP16 and BF16")
    q = torch.empty(rows, 12, 128, device=packed.device, dtype=packed.dtype)
    if rows == 0:
        return q
    row_stride, col_stride = packed.stride()
    segment = (row_stride, 128 * col_stride, col_stride)
    _sibling("rope_kv_write")._launch(
        packed[:, :1536], packed[:, 1536:1792], packed[:, 1792:], q,
        segment, segment, segment, tuple(q.stride()),
        positions, slot_mapping, _as_bytes(torch, k8_pool), _as_bytes(torch, v8_pool),
        rows=rows, q_heads=12, kv_heads=2, head_dim=128, rotate_q=True, base=base,
        valid_tokens=valid_tokens, fp8_scales=(k_scale, v_scale), page_size=16,
    )
    return q


def grouped_splitk_decode_attention_fp8(
    q, k8_pool, v8_pool, k_scale, v_scale, block_table, seq_lens,
    *, split_k, scale=None, partials=None,
):
    """Split-K paged GQA decode attention over FP8 pools; q and the result are fp16/bf16.

    Same contract as grouped_splitk_decode_attention otherwise: explicit split_k,
    optional preallocated fp32 partials, capture-safe.
    """
    import ctypes

    import torch

    _require(q.ndim == 3 and all(size >= 1 for size in q.shape),
             "q must have non-empty shape [batch, query_heads, head_dim]")
    _check_fp8_pools(torch, k8_pool, v8_pool, k_scale, v_scale)
    batch, query_heads, head_dim = q.shape
    kv_heads = k8_pool.shape[2]
    _require(k8_pool.shape[-1] == head_dim, "head dimensions must match")
    _require(query_heads % kv_heads == 0, "query heads must be divisible by KV heads")
    _require(block_table.ndim == 2 and seq_lens.ndim == 1
             and block_table.shape[0] == batch and seq_lens.numel() == batch,
             "batch dimensions must match")
    _require(q.dtype in (torch.float16, torch.bfloat16), "q must be float16 or bfloat16")
    _require(all(t.dtype in (torch.int32, torch.int64) for t in (block_table, seq_lens)),
             "page table and lengths must use integer tensors")
    _require(isinstance(split_k, int) and not isinstance(split_k, bool) and split_k >= 1,
             "split_k must be a positive integer")
    if scale is None:
        scale = head_dim ** -0.5
    expected = (batch, split_k, query_heads, head_dim)
    if partials is None:
        partials = (
            torch.empty(expected, dtype=torch.float32, device=q.device),
            torch.empty(expected[:3], dtype=torch.float32, device=q.device),
            torch.empty(expected[:3], dtype=torch.float32, device=q.device),
        )
    else:
        _require(tuple(partials[0].shape) == expected and tuple(partials[1].shape) == expected[:3]
                 and tuple(partials[2].shape) == expected[:3]
                 and all(t.dtype == torch.float32 and t.is_contiguous() for t in partials),
                 "preallocated partials do not match this launch shape")
    cabi = _cabi()
    splitk = _sibling("paged_decode_grouped_splitk")
    out = torch.empty_like(q)
    args = splitk.fill_attention_args(
        cabi, q, _as_bytes(torch, k8_pool), _as_bytes(torch, v8_pool), block_table, seq_lens,
        split_k=split_k, scale=scale, partials=partials, out=out, kv_scales=(k_scale, v_scale))
    with cabi.device_of(q):
        cabi.check(cabi.library().qf_grouped_splitk_decode_attention(
            ctypes.byref(args), cabi.stream_pointer(q.device)))
    return out


def packed_qkv_rope_attention_fp8(
    packed, positions, slot_mapping, k8_pool, v8_pool, k_scale, v_scale, block_table, seq_lens,
    *, split_k, scale=None, base=1_000_000.0, partials=None, rope_table=None, require_fused=False,
):
    """The decode step on FP8 pools in two launches: packed_qkv_rope_attention (RoPE + KV write
    folded into the attention partial pass, then the combine) with the new K / V rows quantised
    at their page's scales, byte for byte what packed_qkv_rope_cache_fp8 stores.  Same contract
    as the 16-bit call: `slot_mapping[b]` names token seq_lens[b] - 1 of sequence b in
    `block_table` and is not read, every older token is already in the pools; positions are
    int32 / int64; `rope_table` from build_rope_table (default: a cached table as long as the
    block table can hold).  Falls back to the two operators when the fused kernel does not apply
    (`require_fused=True`: raises instead)."""
    import ctypes

    import torch

    fused = _sibling("fused_decode_step")
    if packed.ndim == 3:
        _require(packed.shape[1] == 1, "packed QKV must have one decode token per row")
        packed = packed[:, 0, :]
    _require(packed.ndim == 2 and packed.shape[1] == 2048, "expected packed QKV shape (batch, 2048)")
    batch = packed.shape[0]
    _require(tuple(positions.shape) == (batch,) and tuple(slot_mapping.shape) == (batch,) and
             tuple(seq_lens.shape) == (batch,), "positions, slot_mapping and seq_lens must hold one entry per row")
    _check_fp8_pools(torch, k8_pool, v8_pool, k_scale, v_scale)
    _require(packed.dtype in (torch.float16, torch.bfloat16), "packed QKV must be float16 or bfloat16")

    def pair():
        if require_fused:
            raise RuntimeError("the fused step does not apply to these arguments")
        q = packed_qkv_rope_cache_fp8(packed, positions, slot_mapping, k8_pool, v8_pool, k_scale, v_scale, base=base)
        return grouped_splitk_decode_attention_fp8(q, k8_pool, v8_pool, k_scale, v_scale, block_table, seq_lens,
                                                   split_k=split_k, scale=scale, partials=partials)

    fused_ok = (batch > 0 and int(split_k) >= 2 and packed.stride(1) == 1
                and tuple(k8_pool.shape[1:]) == (16, 2, 128) and block_table.ndim == 2 and block_table.shape[1] > 0
                and positions.dtype in (torch.int32, torch.int64))
    if not fused_ok:
        return pair()
    cabi = _cabi()
    splitk = _sibling("paged_decode_grouped_splitk")
    q_view = packed.as_strided((batch, 12, 128), (packed.stride(0), 128, 1))
    out = torch.empty((batch, 12, 128), dtype=packed.dtype, device=packed.device)
    if partials is None:
        shape = (batch, int(split_k), 12, 128)
        partials = (torch.empty(shape, dtype=torch.float32, device=packed.device),
                    torch.empty(shape[:3], dtype=torch.float32, device=packed.device),
                    torch.empty(shape[:3], dtype=torch.float32, device=packed.device))
    args = splitk.fill_attention_args(
        cabi, q_view, _as_bytes(torch, k8_pool), _as_bytes(torch, v8_pool), block_table, seq_lens,
        split_k=int(split_k), scale=128 ** -0.5 if scale is None else scale, partials=partials, out=out,
        kv_scales=(k_scale, v_scale))
    if cabi.fused_kernel_plan(args)[0] != "decode_mma_kernel (solo)":
        return pair()
    positions = positions.contiguous()
    if rope_table is None:
        rope_table = fused.build_rope_table(block_table.shape[1] * 16, base=base, device=packed.device)
    with cabi.device_of(packed):
        cabi.check(cabi.library().qf_packed_rope_decode_attention(
            ctypes.byref(args), positions.data_ptr(), cabi.torch_index_code(positions.dtype),
            1, rope_table.data_ptr(), rope_table.shape[0], cabi.STAGE_PARTIAL | cabi.STAGE_COMBINE,
            cabi.stream_pointer(packed.device)))
    return out
