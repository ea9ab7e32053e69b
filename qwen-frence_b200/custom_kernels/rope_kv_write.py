"""Fused Q/K RoPE with direct K/V placement into paged cache slots.

Drop-in for the reference module of the same name
(custom_kernels/rope_kv_write.py): same function names, signatures, argument
meaning and ValueError behaviour, so baseline/kernel_dispatch.py:121-133 and
engine/graph/paged_graph_decoder.py:249-265 call it unchanged.  The work is done
by `qf_rope_kv_write` in libqf_hotpath.so (hand-written sm_100a CUDA); the
Triton launch knobs `num_warps` / `num_stages` are validated like the reference
validates them and otherwise ignored.
"""

from __future__ import annotations

import importlib.util
import sys
from pathlib import Path


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


def _ELEMENT_DTYPES(torch):
    return (torch.float16, torch.bfloat16)


def _launch(q, k, v, q_out, q_strides, k_strides, v_strides, o_strides, positions,
            slot_mapping, k_pool, v_pool, *, rows, q_heads, kv_heads, head_dim, rotate_q,
            base, valid_tokens=None, fp8_scales=None, page_size=0):
    """Fill qf_rope_kv_write_args and enqueue on the current stream of q's device."""
    import ctypes

    cabi = _cabi()
    lib = cabi.library()
    flat_k = k_pool.view(-1, k_pool.shape[2], k_pool.shape[3])
    flat_v = v_pool.view(-1, v_pool.shape[2], v_pool.shape[3])
    args = cabi.RopeKvWriteArgs()
    args.q = q.data_ptr() if q is not None else None
    args.k = k.data_ptr()
    args.v = v.data_ptr()
    args.q_out = q_out.data_ptr() if q_out is not None else None
    args.q_stride_row, args.q_stride_head, args.q_stride_d = q_strides
    args.k_stride_row, args.k_stride_head, args.k_stride_d = k_strides
    args.v_stride_row, args.v_stride_head, args.v_stride_d = v_strides
    args.o_stride_row, args.o_stride_head, args.o_stride_d = o_strides
    args.positions = positions.data_ptr()
    args.positions_dtype = cabi.torch_index_code(positions.dtype, allow_float=True)
    args.positions_stride = positions.stride(0)
    args.slot_mapping = slot_mapping.data_ptr()
    args.slot_dtype = cabi.torch_index_code(slot_mapping.dtype)
    args.slot_stride = slot_mapping.stride(0)
    args.k_pool = flat_k.data_ptr()
    args.v_pool = flat_v.data_ptr()
    args.kp_stride_slot, args.kp_stride_head, args.kp_stride_d = flat_k.stride()
    args.vp_stride_slot, args.vp_stride_head, args.vp_stride_d = flat_v.stride()
    args.num_slots = flat_k.shape[0]
    args.valid_tokens = valid_tokens.data_ptr() if valid_tokens is not None else None
    args.rows, args.q_heads, args.kv_heads, args.head_dim = rows, q_heads, kv_heads, head_dim
    args.dtype = cabi.torch_dtype_code(k.dtype)
    args.rotate_q = 1 if rotate_q else 0
    args.base = float(base)
    with cabi.device_of(k):
        stream = cabi.stream_pointer(k.device)
        if fp8_scales is None:
            cabi.check(lib.qf_rope_kv_write(ctypes.byref(args), stream))
        else:
            k_scale, v_scale = fp8_scales
            cabi.check(lib.qf_rope_kv_write_fp8(
                ctypes.byref(args), k_scale.data_ptr(), v_scale.data_ptr(), page_size, stream))


def rope_kv_write(
    q,
    k,
    v,
    positions,
    slot_mapping,
    k_pool,
    v_pool,
    *,
    base=1_000_000.0,
    num_warps=4,
    num_stages=2,
):
    """Rotate packed-layout Q/K and write rotated K plus raw V to paged slots.

    q: (1, Hq, T, D); k, v: (1, Hkv, T, D); positions: (T,) or (1, T);
    slot_mapping: (T,); pools: (pages, page_size, Hkv, D).  Returns rotated Q
    shaped like q.  Mirrors custom_kernels/rope_kv_write.py:89-162.
    """
    import torch

    _require(q.ndim == 4 and k.ndim == 4 and v.ndim == 4, "q, k, and v must be rank-four tensors")
    _require(q.shape[0] == 1 and k.shape[0] == 1 and v.shape[0] == 1,
             "packed q, k, and v must have batch dimension one")
    _require(k.shape == v.shape, "k and v must have matching shapes")
    _require(q.shape[2:] == k.shape[2:], "q and k token/head dimensions are incompatible")
    tokens, dim = q.shape[2], q.shape[-1]
    _require(dim % 2 == 0, "head dimension must be even")
    _require(k_pool.ndim == 4 and k_pool.shape == v_pool.shape,
             "K/V pools must have matching rank-four shapes")
    _require(tuple(k_pool.shape[2:]) == (k.shape[1], dim),
             "pool KV-head and head dimensions must match k/v")
    if positions.ndim == 2:
        _require(tuple(positions.shape) == (1, tokens), "positions must have shape (1, tokens)")
        positions = positions[0]
    _require(positions.ndim == 1 and positions.numel() == tokens,
             "positions must contain one entry per token")
    _require(slot_mapping.ndim == 1 and slot_mapping.numel() == tokens,
             "slot mapping must contain one entry per token")
    operands = (q, k, v, positions, slot_mapping, k_pool, v_pool)
    _require(all(t.is_cuda for t in operands), "fused RoPE/KV placement requires CUDA tensors")
    _require(len({t.device for t in operands}) == 1, "all tensors must share a device")
    _require(q.dtype in _ELEMENT_DTYPES(torch), "q, k, and v must use float16 or bfloat16")
    _require(k.dtype == q.dtype and v.dtype == q.dtype, "q, k, and v dtypes must match")
    _require(k_pool.dtype == q.dtype and v_pool.dtype == q.dtype,
             "Q/K/V and pool dtypes must match")
    _require(slot_mapping.dtype in (torch.int32, torch.int64),
             "slot mapping must use an integer dtype")
    _require(positions.dtype in (torch.int32, torch.int64, torch.float32),
             "positions must be int32, int64, or float32")
    _require(num_warps in (1, 2, 4, 8) and num_stages >= 1, "unsupported warp or stage count")
    _require(dim % 16 == 0 and dim <= 256,
             "head dimension must be a multiple of 16 no larger than 256")

    q_out = torch.empty_like(q)
    _launch(
        q, k, v, q_out,
        (q.stride(2), q.stride(1), q.stride(3)),
        (k.stride(2), k.stride(1), k.stride(3)),
        (v.stride(2), v.stride(1), v.stride(3)),
        (q_out.stride(2), q_out.stride(1), q_out.stride(3)),
        positions, slot_mapping, k_pool, v_pool,
        rows=tokens, q_heads=q.shape[1], kv_heads=k.shape[1], head_dim=dim,
        rotate_q=True, base=base,
    )
    return q_out


def native_decode_rope_kv_write(
    q, k, v, positions, slot_mapping, k_pool, v_pool,
    *, base=1_000_000.0, num_warps=4, rotate_q=True,
):
    """Rotate native-layout decode Q/K and place K/V without layout copies.

    Inputs are (B, H, 1, D) views of the packed projection output.  With
    rotate_q=False only the KV heads are processed and q is returned untouched.
    Mirrors custom_kernels/rope_kv_write.py:223-276.
    """
    import torch

    _require(all(t.ndim == 4 and t.shape[2] == 1 for t in (q, k, v)),
             "decode Q/K/V must have shape (batch, heads, 1, dim)")
    batch, q_heads, _, dim = q.shape
    kv_heads = k.shape[1]
    _require(k.shape == v.shape and k.shape[0] == batch and k.shape[-1] == dim,
             "decode K/V shapes do not match Q")
    _require(dim % 2 == 0 and q_heads >= kv_heads, "invalid query/KV head dimensions")
    _require(tuple(positions.shape) == (batch,) and tuple(slot_mapping.shape) == (batch,),
             "positions and slots must contain one entry per batch row")
    _require(k_pool.ndim == 4 and k_pool.shape == v_pool.shape,
             "K/V pools must have matching rank-four shapes")
    _require(tuple(k_pool.shape[2:]) == (kv_heads, dim) and k_pool.is_contiguous()
             and v_pool.is_contiguous(),
             "K/V pools must be contiguous with matching KV dimensions")
    operands = (q, k, v, positions, slot_mapping, k_pool, v_pool)
    _require(all(t.is_cuda and t.device == q.device for t in operands),
             "all inputs must share one CUDA device")
    _require(q.dtype in _ELEMENT_DTYPES(torch)
             and all(t.dtype == q.dtype for t in (k, v, k_pool, v_pool)),
             "Q/K/V and pools must share FP16 or BF16 dtype")
    _require(positions.dtype in (torch.int32, torch.int64, torch.float32),
             "positions must be int32, int64, or float32")
    _require(slot_mapping.dtype in (torch.int32, torch.int64), "slots must use an integer dtype")
    _require(num_warps in (1, 2, 4, 8), "num_warps must be 1, 2, 4, or 8")
    _require(dim % 16 == 0 and dim <= 256,
             "head dimension must be a multiple of 16 no larger than 256")

    out = torch.empty_like(q) if rotate_q else q
    _launch(
        q if rotate_q else None, k, v, out if rotate_q else None,
        (q.stride(0), q.stride(1), q.stride(3)),
        (k.stride(0), k.stride(1), k.stride(3)),
        (v.stride(0), v.stride(1), v.stride(3)),
        (out.stride(0), out.stride(1), out.stride(3)),
        positions, slot_mapping, k_pool, v_pool,
        rows=batch, q_heads=q_heads, kv_heads=kv_heads, head_dim=dim,
        rotate_q=rotate_q, base=base,
    )
    return out
