"""Native CUDA grouped-GQA split-K decode attention.

Drop-in for custom_kernels/paged_decode_native_grouped.py: same three entry
points and signatures, so baseline/kernel_dispatch.py:84-88 and
engine/kvcache/paged_decode_attention.py:228-234 call it unchanged.

The six query heads of a GQA group share every K/V page, which is copied once
into a shared-memory ring; the combine merges the numerically stable fp32
partials.  `native_grouped_splitk_decode_attention` runs the persistent kernel
(resident CTAs that share the batch's pages equally, then the combine);
`grouped_gqa_splitk_partial_out` runs one CTA per (request, KV head, split) and
returns the reference's balanced partitions.  Everything runs inside
libqf_hotpath.so (sm_100a); nothing here depends on Triton, on a torch C++
extension or on a CPU fallback.
"""

from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

GROUP, HEAD_DIM, PAGE_SIZE = 6, 128, 16


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


def _extension():
    """The loaded C ABI binding; raises with the one build command when it is missing."""
    cabi = _sibling("_cabi", Path(__file__).resolve().parents[1])
    try:
        cabi.library()
    except (RuntimeError, OSError) as exc:
        raise RuntimeError(
            "native grouped decode is not built; run: " + cabi.BUILD_COMMAND
        ) from exc
    return cabi


def _require(condition, message):
    if not condition:
        raise ValueError(message)


def _check_layout(q, k_pool, v_pool):
    _require(q.ndim == 3 and k_pool.ndim == 4 and k_pool.shape == v_pool.shape,
             "expected Q rank three and matching rank-four K/V pools")
    batch, query_heads, head_dim = q.shape
    _require(head_dim == HEAD_DIM and k_pool.shape[1] == PAGE_SIZE,
             "native grouped decode requires head_dim=128 and page_size=16")
    _require(query_heads == k_pool.shape[2] * GROUP,
             "native grouped decode requires six query heads per KV head")
    return batch, query_heads, head_dim


def _check_metadata(torch, q, k_pool, v_pool, block_table, seq_lens):
    _require(q.dtype in (torch.float16, torch.bfloat16), "Q/K/V must be float16 or bfloat16")
    _require(k_pool.dtype == q.dtype and v_pool.dtype == q.dtype, "Q/K/V dtypes must match")
    _require(block_table.dtype == seq_lens.dtype
             and block_table.dtype in (torch.int32, torch.int64),
             "block_table and seq_lens must both be int32 or int64")
    _require(block_table.ndim == 2 and seq_lens.ndim == 1,
             "block table and lengths must have rank two and one")
    _require(block_table.shape[0] == q.shape[0] and seq_lens.shape[0] == q.shape[0],
             "batch dimensions must match")
    operands = (q, k_pool, v_pool, block_table, seq_lens)
    _require(all(t.is_cuda and t.device == q.device for t in operands),
             "all inputs must share a device")


def native_grouped_splitk_decode_attention(
    q,
    k_pool,
    v_pool,
    block_table,
    seq_lens,
    *,
    split_k,
    scale=None,
    partials=None,
):
    """Run the CTA-shared grouped-GQA partial pass and the split-K combine.

    q: (B, 6*Hkv, 128); pools: (pages, 16, Hkv, 128); split_k >= 2.
    Mirrors custom_kernels/paged_decode_native_grouped.py:30-88.
    """
    batch, query_heads, head_dim = _check_layout(q, k_pool, v_pool)
    _require(isinstance(split_k, int) and not isinstance(split_k, bool) and split_k >= 2,
             "native grouped decode requires split_k >= 2")
    _require(split_k <= 65535, "split_k must be in [2, 65535]")
    if scale is None:
        scale = head_dim ** -0.5

    import ctypes

    import torch

    cabi = _extension()
    _check_metadata(torch, q, k_pool, v_pool, block_table, seq_lens)
    expected_out = (batch, split_k, query_heads, head_dim)
    expected_stats = expected_out[:3]
    if partials is None:
        partial_out = torch.empty(expected_out, dtype=torch.float32, device=q.device)
        partial_max = torch.empty(expected_stats, dtype=torch.float32, device=q.device)
        partial_sum = torch.empty_like(partial_max)
    else:
        partial_out, partial_max, partial_sum = partials
        _require(tuple(partial_out.shape) == expected_out,
                 "preallocated partial output has the wrong shape")
        _require(tuple(partial_max.shape) == expected_stats
                 and partial_sum.shape == partial_max.shape,
                 "preallocated partial statistics have the wrong shape")
        _require(all(t.dtype == torch.float32 and t.is_contiguous()
                     for t in (partial_out, partial_max, partial_sum)),
                 "partial outputs must be contiguous float32")

    splitk = _sibling("paged_decode_grouped_splitk")
    out = torch.empty_like(q)
    args = splitk.fill_attention_args(
        cabi, q, k_pool, v_pool, block_table, seq_lens, split_k=split_k, scale=scale,
        partials=(partial_out, partial_max, partial_sum), out=out)
    with cabi.device_of(q):
        cabi.check(cabi.library().qf_grouped_splitk_decode_attention(
            ctypes.byref(args), cabi.stream_pointer(q.device)))
    return out


def grouped_gqa_splitk_partial_out(q, k_pool, v_pool, block_table, seq_lens,
                                   partial_out, partial_max, partial_sum, scale):
    """The partial pass alone, into caller buffers, one partition per split slot.

    Same arguments as the extension op the reference binds
    (custom_kernels/native_grouped_decode.cu:329-403): partition s of a sequence
    covers pages [s*P/K, (s+1)*P/K); partial_out (B, K, H, 128) is unnormalised,
    partial_max an exponent offset in natural-log units, partial_sum the matching
    sum; an empty partition is (0, -inf, 0).  Returns None.
    """
    import ctypes

    import torch

    batch, query_heads, head_dim = _check_layout(q, k_pool, v_pool)
    cabi = _extension()
    _check_metadata(torch, q, k_pool, v_pool, block_table, seq_lens)
    _require(partial_out.ndim == 4 and partial_out.shape[0] == batch
             and tuple(partial_out.shape[2:]) == (query_heads, head_dim),
             "preallocated partial output has the wrong shape")
    split_k = partial_out.shape[1]
    _require(tuple(partial_max.shape) == (batch, split_k, query_heads)
             and partial_sum.shape == partial_max.shape,
             "preallocated partial statistics have the wrong shape")
    _require(all(t.dtype == torch.float32 and t.is_contiguous() and t.device == q.device
                 for t in (partial_out, partial_max, partial_sum)),
             "partial outputs must be contiguous float32")
    splitk = _sibling("paged_decode_grouped_splitk")
    args = splitk.fill_attention_args(
        cabi, q, k_pool, v_pool, block_table, seq_lens, split_k=split_k, scale=scale,
        partials=(partial_out, partial_max, partial_sum), out=None)
    with cabi.device_of(q):
        cabi.check(cabi.library().qf_grouped_gqa_splitk_partial_out(
            ctypes.byref(args), cabi.stream_pointer(q.device)))


def native_grouped_decode_diagnostics(q, block_table):
    """Compiled resources and occupancy of the partial kernel, without counters.

    Mirrors custom_kernels/paged_decode_native_grouped.py:91-93.
    """
    import ctypes

    import torch

    _require(q.is_cuda and block_table.is_cuda, "inputs must be CUDA")
    _require(q.dtype in (torch.float16, torch.bfloat16), "q must be float16 or bfloat16")
    _require(block_table.dtype in (torch.int32, torch.int64),
             "block table must be int32 or int64")
    cabi = _extension()
    info = (ctypes.c_int64 * len(cabi.KERNEL_INFO_FIELDS))()
    cabi.check(cabi.library().qf_grouped_gqa_splitk_diagnostics(
        q.device.index if q.device.index is not None else torch.cuda.current_device(),
        cabi.torch_dtype_code(q.dtype), 0, info))
    result = dict(zip(cabi.KERNEL_INFO_FIELDS, (int(v) for v in info)))
    threads = result["threads_per_block"]
    result["active_warps_per_sm"] = result["active_blocks_per_sm"] * (threads // 32)
    result["theoretical_occupancy"] = (
        result["active_warps_per_sm"] / result["max_warps_per_sm"]
        if result["max_warps_per_sm"] else 0.0)
    return result


def native_grouped_stage_cycles(
    q, k_pool, v_pool, block_table, seq_lens, *, split_k, scale=None
):
    """Run the instrumented partial once and return per-CTA stage cycles.

    Returns int64 [B, Hkv, split_k, 4]: clock64() cycles one warp of each CTA of
    the per-partition kernel spent {waiting for pages, in the whole page loop, in
    the set-up before it, in the merge after it} (loading overlaps the math, so
    there is no separate load or PV stage).
    Mirrors custom_kernels/paged_decode_native_grouped.py:96-119.
    """
    import ctypes

    import torch

    batch, query_heads, head_dim = q.shape
    _require(query_heads == k_pool.shape[2] * GROUP and head_dim == HEAD_DIM
             and k_pool.shape[1] == PAGE_SIZE,
             "stage profiler requires the native grouped-decode layout")
    _require(isinstance(split_k, int) and split_k >= 2, "split_k must exceed one")
    if scale is None:
        scale = head_dim ** -0.5
    cabi = _extension()
    _check_metadata(torch, q, k_pool, v_pool, block_table, seq_lens)
    partial_out = torch.empty((batch, split_k, query_heads, head_dim),
                              dtype=torch.float32, device=q.device)
    partial_max = torch.empty((batch, split_k, query_heads), dtype=torch.float32, device=q.device)
    partial_sum = torch.empty_like(partial_max)
    cycles = torch.zeros((batch, k_pool.shape[2], split_k, 4), dtype=torch.int64, device=q.device)
    splitk = _sibling("paged_decode_grouped_splitk")
    args = splitk.fill_attention_args(
        cabi, q, k_pool, v_pool, block_table, seq_lens, split_k=split_k, scale=scale,
        partials=(partial_out, partial_max, partial_sum), out=None)
    with cabi.device_of(q):
        cabi.check(cabi.library().qf_grouped_gqa_splitk_profile_out(
            ctypes.byref(args), cycles.data_ptr(), cabi.stream_pointer(q.device)))
    return cycles


def native_grouped_persistent_timeline(
    q, k_pool, v_pool, block_table, seq_lens, *, split_k, scale=None
):
    """Run the instrumented tensor-core persistent partial pass once.

    Returns int64 [Hkv * ctas_per_head, 10]: per CTA {ns at entry, ns when the work
    list was built, ns when its page ids were known, ns when its first K tile had
    landed, ns at exit (of its last warp), units in its share (pages plus the empty
    units the kernel counts per sequence), pieces that held
    pages of its warp 0, ns warp 0 spent depositing its piece states, ns warp 0
    spent merging pieces, pieces warp 0 merged} on the GPU's global timer (256 ns
    steps on B200); rows of CTAs without work stay zero.  Raises RuntimeError when these arguments
    would not run that kernel (batch above 1024, K and V pools with different strides).
    The counterpart of `native_grouped_stage_cycles` for a kernel whose CTAs are
    not tied to one (sequence, head, split).
    """
    import ctypes

    import torch

    batch, query_heads, head_dim = _check_layout(q, k_pool, v_pool)
    _require(isinstance(split_k, int) and split_k >= 2, "split_k must exceed one")
    if scale is None:
        scale = head_dim ** -0.5
    cabi = _extension()
    _check_metadata(torch, q, k_pool, v_pool, block_table, seq_lens)
    partial_out = torch.empty((batch, split_k, query_heads, head_dim),
                              dtype=torch.float32, device=q.device)
    partial_max = torch.empty((batch, split_k, query_heads), dtype=torch.float32, device=q.device)
    partial_sum = torch.empty_like(partial_max)
    splitk = _sibling("paged_decode_grouped_splitk")
    args = splitk.fill_attention_args(
        cabi, q, k_pool, v_pool, block_table, seq_lens, split_k=split_k, scale=scale,
        partials=(partial_out, partial_max, partial_sum), out=torch.empty_like(q))
    with cabi.device_of(q):
        _, ctas_per_head = cabi.fused_kernel_plan(args)
        timeline = torch.zeros((max(ctas_per_head, 1) * k_pool.shape[2], 10), dtype=torch.int64,
                               device=q.device)
        cabi.check(cabi.library().qf_grouped_splitk_persistent_timeline(
            ctypes.byref(args), timeline.data_ptr(), cabi.stream_pointer(q.device)))
    return timeline
