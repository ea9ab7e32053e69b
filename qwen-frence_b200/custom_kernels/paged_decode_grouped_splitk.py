"""Grouped split-K paged decode attention, CUDA-graph safe.

Drop-in for custom_kernels/paged_decode_grouped_splitk.py: same entry point,
signature, return contract and ValueError behaviour, so
baseline/kernel_dispatch.py:77-81 and
engine/kvcache/paged_decode_attention.py:219-227 call it unchanged.

`split_k` is always explicit: the caller resolves it once on the host, before
capture.  Validation reads shapes and dtypes only, nothing is read back from
the device, and every buffer (partials included) is a torch allocation, so the
call can be recorded into a CUDA graph exactly like the reference's
(custom_kernels/paged_decode_grouped_splitk.py:247-252).

The work is done by libqf_hotpath.so: `qf_grouped_splitk_decode_attention`
runs the partial pass (all query heads of a GQA group share each page load; for
split_k > 1 persistent CTAs share the batch's pages equally, and the partial
buffers are their private scratch) and the combine.  The Triton knobs `num_stages`, `heads_per_program` and `num_warps` are validated as
the reference validates them and otherwise ignored.
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


def _power_of_two(size):
    return size >= 1 and not size & (size - 1)


def fill_attention_args(cabi, q, k_pool, v_pool, block_table, seq_lens, *, split_k, scale,
                        partials, out, kv_scales=None):
    """Build qf_decode_attention_args from torch tensors (strides in elements)."""
    args = cabi.DecodeAttentionArgs()
    args.q = q.data_ptr()
    args.q_stride_b, args.q_stride_h, args.q_stride_d = q.stride()
    args.k_pool = k_pool.data_ptr()
    args.v_pool = v_pool.data_ptr()
    (args.k_stride_page, args.k_stride_tok, args.k_stride_head, args.k_stride_d) = k_pool.stride()
    (args.v_stride_page, args.v_stride_tok, args.v_stride_head, args.v_stride_d) = v_pool.stride()
    args.block_table = block_table.data_ptr()
    args.table_dtype = cabi.torch_index_code(block_table.dtype)
    args.table_stride_b, args.table_stride_p = block_table.stride()
    args.table_width = block_table.shape[1]
    args.seq_lens = seq_lens.data_ptr()
    args.lens_dtype = cabi.torch_index_code(seq_lens.dtype)
    args.lens_stride = seq_lens.stride(0)
    if kv_scales is not None:
        args.k_scale = kv_scales[0].data_ptr()
        args.v_scale = kv_scales[1].data_ptr()
        args.kv_fp8 = 1
    if partials is not None:
        args.partial_out = partials[0].data_ptr()
        args.partial_max = partials[1].data_ptr()
        args.partial_sum = partials[2].data_ptr()
    if out is not None:
        args.out = out.data_ptr()
        args.o_stride_b, args.o_stride_h, args.o_stride_d = out.stride()
    args.num_pages = k_pool.shape[0]
    args.batch, args.q_heads, args.head_dim = q.shape
    args.kv_heads = k_pool.shape[2]
    args.page_size = k_pool.shape[1]
    args.split_k = split_k
    args.dtype = cabi.torch_dtype_code(q.dtype)
    args.scale = float(scale)
    return args


def splitk_reduce(partial_out, partial_max, partial_sum, out):
    """Combine fp32 split-K partials into `out` (B, heads, D), skipping empty partitions.

    Stands in for launching the reference's `_splitk_reduce_kernel`
    (custom_kernels/paged_decode_grouped_splitk.py:165-226).
    """
    cabi = _cabi()
    batch, split_k, heads, dim = partial_out.shape
    with cabi.device_of(out):
        cabi.check(cabi.library().qf_splitk_reduce(
            partial_out.data_ptr(), partial_max.data_ptr(), partial_sum.data_ptr(),
            *partial_out.stride(), *partial_max.stride(),
            out.data_ptr(), *out.stride(),
            batch, heads, dim, split_k, cabi.torch_dtype_code(out.dtype),
            cabi.stream_pointer(out.device)))
    return out


def grouped_splitk_decode_attention(
    q,
    k_pool,
    v_pool,
    block_table,
    seq_lens,
    *,
    split_k,
    num_stages=2,
    heads_per_program=1,
    num_warps=4,
    scale=None,
    partials=None,
):
    """Explicit-configuration split-K decode attention.

    q: (B, n_heads, d_head). pools: (num_pages, page_size, n_kv_heads, d_head).
    block_table: (B, max_pages) int32/int64. seq_lens: (B,) int32/int64.
    Returns out (B, n_heads, d_head) in q's dtype; for split_k == 1 it is
    `partial_out.squeeze(1)` as in the reference.  `partials` optionally supplies
    preallocated (out, max, sum) buffers.
    """
    import ctypes

    import torch

    _require(q.ndim == 3 and all(size >= 1 for size in q.shape),
             "q must have non-empty shape [batch, query_heads, head_dim]")
    _require(k_pool.ndim == 4 and k_pool.shape == v_pool.shape,
             "K/V pools must have matching rank-four shapes")
    batch, query_heads, head_dim = q.shape
    page_size, kv_heads = k_pool.shape[1], k_pool.shape[2]
    _require(kv_heads >= 1 and k_pool.shape[-1] == head_dim,
             "KV heads must be positive and head dimensions must match")
    _require(query_heads % kv_heads == 0, "query heads must be divisible by KV heads")
    _require(block_table.ndim == 2 and seq_lens.ndim == 1,
             "block table and sequence lengths must be rank two and one")
    _require(block_table.shape[0] == batch and seq_lens.numel() == batch,
             "batch dimensions must match")
    _require(_power_of_two(head_dim) and _power_of_two(page_size),
             "head dimension and page size must be powers of two")
    _require(k_pool.dtype == q.dtype and v_pool.dtype == q.dtype, "Q/K/V dtypes must match")
    _require(all(t.dtype in (torch.int32, torch.int64) for t in (block_table, seq_lens)),
             "page table and lengths must use integer tensors")
    _require(isinstance(split_k, int) and not isinstance(split_k, bool) and split_k >= 1,
             "split_k must be a positive integer")
    _require(num_warps in (1, 2, 4, 8) and isinstance(num_stages, int) and num_stages >= 1,
             "num_warps must be 1, 2, 4, or 8 and num_stages a positive integer")
    group = query_heads // kv_heads
    _require(heads_per_program in (1, 2, 3, 6) and group % heads_per_program == 0,
             "heads_per_program must divide the query/KV head group evenly")
    _require(q.dtype in (torch.float16, torch.bfloat16), "Q/K/V must be float16 or bfloat16")
    _require(head_dim <= 256, "head dimension must not exceed 256")
    operands = (q, k_pool, v_pool, block_table, seq_lens)
    _require(all(t.is_cuda and t.device == q.device for t in operands),
             "all inputs must share one CUDA device")
    if scale is None:
        scale = head_dim ** -0.5

    expected = (batch, split_k, query_heads, head_dim)
    if partials is None:
        partial_out = torch.empty(expected, dtype=q.dtype if split_k == 1 else torch.float32,
                                  device=q.device)
        partial_max = torch.empty(expected[:3], dtype=torch.float32, device=q.device)
        partial_sum = torch.empty_like(partial_max)
    else:
        partial_out, partial_max, partial_sum = partials
        _require(tuple(partial_out.shape) == expected and tuple(partial_max.shape) == expected[:3],
                 "preallocated partials do not match this launch shape")
        _require(partial_max.dtype == torch.float32 and partial_sum.dtype == torch.float32
                 and partial_sum.shape == partial_max.shape
                 and partial_max.is_contiguous() and partial_sum.is_contiguous()
                 and partial_out.is_contiguous(),
                 "preallocated partials must be contiguous float32 statistics")

    cabi = _cabi()
    lib = cabi.library()
    with cabi.device_of(q):
        stream = cabi.stream_pointer(q.device)
        if split_k == 1 and partial_out.dtype == q.dtype:
            # Single pass: the kernel normalises in fp32 and stores the q dtype.
            out = partial_out[:, 0]
            args = fill_attention_args(cabi, q, k_pool, v_pool, block_table, seq_lens,
                                       split_k=1, scale=scale, partials=None, out=out)
            cabi.check(lib.qf_grouped_splitk_decode_attention(ctypes.byref(args), stream))
            return partial_out.squeeze(1)
        _require(partial_out.dtype == torch.float32,
                 "preallocated partial output must be float32 (or the q dtype when split_k is 1)")
        if split_k == 1:
            # fp32 buffer supplied for one partition: keep the reference's contract
            # (normalised values in the caller's buffer, returned squeezed).
            args = fill_attention_args(cabi, q, k_pool, v_pool, block_table, seq_lens,
                                       split_k=1, scale=scale,
                                       partials=(partial_out, partial_max, partial_sum), out=None)
            cabi.check(lib.qf_grouped_gqa_splitk_partial_out(ctypes.byref(args), stream))
            denominator = torch.where(partial_sum > 0, partial_sum, torch.ones_like(partial_sum))
            partial_out.div_(denominator[..., None])
            return partial_out.squeeze(1)
        out = torch.empty_like(q)
        args = fill_attention_args(cabi, q, k_pool, v_pool, block_table, seq_lens,
                                   split_k=split_k, scale=scale,
                                   partials=(partial_out, partial_max, partial_sum), out=out)
        cabi.check(lib.qf_grouped_splitk_decode_attention(ctypes.byref(args), stream))
    return out


def grouped_splitk_decode_attention_static(q, k_pool, v_pool, block_table, seq_lens, out, *,
                                           split_k, scale=None):
    """Split-K decode attention whose partial buffers come from the library's static
    device array instead of an allocation.

    For hosts that cannot allocate per call: a serving loop without a caching
    allocator (a raw cudaMalloc per decode step synchronises the device), or a
    process whose device memory was all handed to another allocator at start.  The
    caller passes the inputs and `out` (B, heads, D, q's dtype); this wrapper and
    the C entry point allocate nothing.  Limit: batch * split_k * heads * (D + 2)
    fp32 values must fit in 16 MiB, else RuntimeError.  The first call on a device
    resolves the array's address and should be made before any stream capture;
    calls that overlap on the GPU share the array and race.  No counterpart in the
    reference.
    """
    import ctypes

    import torch

    _require(q.ndim == 3 and k_pool.ndim == 4 and k_pool.shape == v_pool.shape,
             "expected Q rank three and matching rank-four K/V pools")
    _require(out.shape == q.shape and out.dtype == q.dtype and out.device == q.device,
             "out must match q in shape, dtype and device")
    _require(q.dtype in (torch.float16, torch.bfloat16) and k_pool.dtype == q.dtype
             and v_pool.dtype == q.dtype, "Q/K/V must share float16 or bfloat16")
    _require(block_table.ndim == 2 and seq_lens.ndim == 1 and block_table.shape[0] == q.shape[0]
             and seq_lens.numel() == q.shape[0], "batch dimensions must match")
    _require(all(t.dtype in (torch.int32, torch.int64) for t in (block_table, seq_lens)),
             "page table and lengths must use integer tensors")
    _require(isinstance(split_k, int) and not isinstance(split_k, bool) and split_k >= 1,
             "split_k must be a positive integer")
    _require(all(t.is_cuda and t.device == q.device for t in (k_pool, v_pool, block_table, seq_lens)),
             "all inputs must share one CUDA device")
    if scale is None:
        scale = q.shape[-1] ** -0.5
    cabi = _cabi()
    args = fill_attention_args(cabi, q, k_pool, v_pool, block_table, seq_lens, split_k=split_k,
                               scale=scale, partials=None, out=out)
    with cabi.device_of(q):
        cabi.check(cabi.library().qf_grouped_splitk_decode_attention_static(
            ctypes.byref(args), cabi.stream_pointer(q.device)))
    return out
