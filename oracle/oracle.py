"""Python face of the CPU oracle (oracle/qf_oracle.c).

TEST INFRASTRUCTURE, NOT PRODUCT.  Only tests/, __graft_entry__.smoke() and
bench.py's CPU-baseline legs may import this module; the product path
(qwen-frence_b200/) never does.

Parity pin: the functions here are checked against outputs of the reference's
own Python functions (tests/golden/*.npz, generated from the reference tree by
tests/golden/make_golden.py) and against the reference's known-answer tests,
in tests/test_oracle.py.

Everything takes and returns CPU torch tensors.  16-bit tensors cross into C as
bit patterns, so fp16 and bf16 share one code path.
"""

from __future__ import annotations

import ctypes
from ctypes import c_double, c_float, c_int, c_int64, c_void_p
from pathlib import Path

import numpy as np
import torch

ORACLE_DIR = Path(__file__).resolve().parent
_lib = None


def library():
    """Load (building on first use when gcc is present) oracle/libqf_oracle.so."""
    global _lib
    if _lib is not None:
        return _lib
    path = ORACLE_DIR / "libqf_oracle.so"
    if not path.is_file():
        import importlib.util

        spec = importlib.util.spec_from_file_location("qf_oracle_build", ORACLE_DIR / "build.py")
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        module.build_oracle()
    lib = ctypes.CDLL(str(path))
    lib.qfo_e4m3_decode.restype = c_float
    lib.qfo_e4m3_decode.argtypes = [ctypes.c_uint8]
    lib.qfo_e4m3_encode.restype = ctypes.c_uint8
    lib.qfo_e4m3_encode.argtypes = [c_float]
    lib.qfo_inv_freq.argtypes = [c_double, c_int, c_void_p]
    lib.qfo_rope.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_double, c_void_p]
    lib.qfo_rope_f32.argtypes = lib.qfo_rope.argtypes
    lib.qfo_packed_qkv_rope_cache.argtypes = [
        c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_double,
        c_void_p, c_void_p, c_void_p, c_int64]
    lib.qfo_paged_attention.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
        c_int, c_int64, c_float, c_void_p, c_void_p]
    lib.qfo_splitk_partial.argtypes = [
        c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
        c_int, c_int64, c_float, c_int, c_void_p, c_void_p, c_void_p]
    lib.qfo_splitk_reduce.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                      c_int, c_void_p]
    lib.qfo_quantize_pages.argtypes = [c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p,
                                       c_void_p]
    lib.qfo_dequantize_pages.argtypes = [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                                         c_void_p]
    lib.qfo_write_fixed_scale.argtypes = [c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          c_void_p, c_void_p, c_int64]
    _lib = lib
    return lib


def _code(dtype):
    if dtype == torch.float16:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise ValueError(f"oracle supports float16 and bfloat16, not {dtype}")


def _dense(tensor):
    """A contiguous CPU copy (strided or poisoned views become plain arrays)."""
    return tensor.detach().cpu().contiguous()


def _ptr(tensor):
    return c_void_p(tensor.data_ptr())


def _positions_f32(positions):
    # `.to(float32)`, the conversion the kernels apply to integer positions.
    return _dense(positions).to(torch.float32)


def inv_freq(base, half):
    out = torch.empty(half, dtype=torch.float32)
    library().qfo_inv_freq(float(base), int(half), _ptr(out))
    return out


def rope(x, positions, base=1_000_000.0):
    """fp32 single-rounding rotate-half RoPE of x [rows, heads, dim]."""
    x = _dense(x)
    rows, heads, dim = x.shape
    out = torch.empty_like(x)
    pos = _positions_f32(positions)
    library().qfo_rope(_ptr(x), _code(x.dtype), _ptr(pos), rows, heads, dim, float(base), _ptr(out))
    return out


def rope_f32(x, positions, base=1_000_000.0):
    """Same rotation, left in fp32 (what the FP8 write path quantises)."""
    x = _dense(x)
    rows, heads, dim = x.shape
    out = torch.empty(x.shape, dtype=torch.float32)
    pos = _positions_f32(positions)
    library().qfo_rope_f32(_ptr(x), _code(x.dtype), _ptr(pos), rows, heads, dim, float(base), _ptr(out))
    return out


def kv_write(k_pool, v_pool, slot_mapping, k_rows, v_rows):
    """Place rows [n, hkv, dim] at flat slots of pools [pages, page, hkv, dim], in
    place, like `index_copy_` on the flat view
    (engine/graph/paged_graph_decoder.py:271-274)."""
    flat_k = k_pool.view(-1, k_pool.shape[2], k_pool.shape[3])
    flat_v = v_pool.view(-1, v_pool.shape[2], v_pool.shape[3])
    slots = slot_mapping.detach().cpu().long()
    flat_k.index_copy_(0, slots, _dense(k_rows))
    flat_v.index_copy_(0, slots, _dense(v_rows))


def packed_qkv_rope_cache(packed, positions, slot_mapping, k_pool, v_pool, *, base=1_000_000.0,
                          valid_tokens=None, q_heads=12, kv_heads=2, head_dim=128):
    """Whole fused epilogue on CPU; mutates the (contiguous CPU) pools, returns q."""
    packed = _dense(packed)
    rows = packed.shape[0]
    assert k_pool.is_contiguous() and v_pool.is_contiguous() and k_pool.device.type == "cpu"
    live = rows if valid_tokens is None else min(rows, int(valid_tokens))
    q = torch.empty(rows, q_heads, head_dim, dtype=packed.dtype)
    pos = _positions_f32(positions)
    slots = _dense(slot_mapping).long()
    num_slots = k_pool.shape[0] * k_pool.shape[1]
    library().qfo_packed_qkv_rope_cache(
        _ptr(packed), _code(packed.dtype), _ptr(pos), _ptr(slots), rows, live, q_heads, kv_heads,
        head_dim, float(base), _ptr(q), _ptr(k_pool), _ptr(v_pool), num_slots)
    return q


def _attention_operands(q, k_pool, v_pool, block_table, seq_lens):
    q, k_pool, v_pool = _dense(q), _dense(k_pool), _dense(v_pool)
    table = _dense(block_table).long()
    lens = _dense(seq_lens).long()
    if table.shape[1] == 0:
        table = torch.zeros(table.shape[0], 1, dtype=torch.long)
    return q, k_pool, v_pool, table, lens


def paged_attention(q, k_pool, v_pool, block_table, seq_lens, *, scale=None, return_f32=False):
    """Dense fp32-accumulated paged GQA decode attention; empty rows are zero."""
    q, k_pool, v_pool, table, lens = _attention_operands(q, k_pool, v_pool, block_table, seq_lens)
    batch, hq, dim = q.shape
    _, page, hkv, _ = k_pool.shape
    scale = dim ** -0.5 if scale is None else scale
    out = torch.zeros_like(q)
    out32 = torch.zeros(q.shape, dtype=torch.float32) if return_f32 else None
    library().qfo_paged_attention(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _code(q.dtype), _ptr(table), _ptr(lens), batch, hq,
        hkv, dim, page, table.shape[1], float(scale), _ptr(out),
        _ptr(out32) if return_f32 else None)
    return (out, out32) if return_f32 else out


def splitk_partial(q, k_pool, v_pool, block_table, seq_lens, *, split_k, scale=None):
    q, k_pool, v_pool, table, lens = _attention_operands(q, k_pool, v_pool, block_table, seq_lens)
    batch, hq, dim = q.shape
    _, page, hkv, _ = k_pool.shape
    scale = dim ** -0.5 if scale is None else scale
    po = torch.empty(batch, split_k, hq, dim, dtype=torch.float32)
    pm = torch.empty(batch, split_k, hq, dtype=torch.float32)
    ps = torch.empty(batch, split_k, hq, dtype=torch.float32)
    library().qfo_splitk_partial(
        _ptr(q), _ptr(k_pool), _ptr(v_pool), _code(q.dtype), _ptr(table), _ptr(lens), batch, hq,
        hkv, dim, page, table.shape[1], float(scale), split_k, _ptr(po), _ptr(pm), _ptr(ps))
    return po, pm, ps


def splitk_reduce(partial_out, partial_max, partial_sum, dtype=torch.float16):
    po, pm, ps = (_dense(t).float() for t in (partial_out, partial_max, partial_sum))
    batch, split_k, hq, dim = po.shape
    out = torch.empty(batch, hq, dim, dtype=dtype)
    library().qfo_splitk_reduce(_ptr(po), _ptr(pm), _ptr(ps), batch, split_k, hq, dim,
                                _code(dtype), _ptr(out))
    return out


def splitk_attention(q, k_pool, v_pool, block_table, seq_lens, *, split_k, scale=None):
    po, pm, ps = splitk_partial(q, k_pool, v_pool, block_table, seq_lens, split_k=split_k,
                                scale=scale)
    return splitk_reduce(po, pm, ps, dtype=q.dtype)


# ---- FP8 e4m3 ---------------------------------------------------------------

def e4m3_decode_table():
    lib = library()
    return torch.tensor([lib.qfo_e4m3_decode(b) for b in range(256)], dtype=torch.float32)


def e4m3_encode(values):
    """Round-to-nearest-even e4m3 bytes of an fp32 tensor (saturating)."""
    lib = library()
    flat = _dense(values).float().flatten().tolist()
    return torch.tensor([lib.qfo_e4m3_encode(v) for v in flat], dtype=torch.uint8).view(values.shape)


def quantize_pages(pool):
    pool = _dense(pool)
    pages, page, hkv, dim = pool.shape
    pool8 = torch.empty(pool.shape, dtype=torch.uint8)
    scales = torch.empty(pages, hkv, dtype=torch.float32)
    library().qfo_quantize_pages(_ptr(pool), _code(pool.dtype), pages, page, hkv, dim, _ptr(pool8),
                                 _ptr(scales))
    return pool8, scales


def dequantize_pages(pool8, scales, dtype=torch.float16):
    pool8, scales = _dense(pool8), _dense(scales).float()
    if pool8.dtype != torch.uint8:
        pool8 = pool8.view(torch.uint8)
    pages, page, hkv, dim = pool8.shape
    out = torch.empty(pool8.shape, dtype=dtype)
    library().qfo_dequantize_pages(_ptr(pool8), _ptr(scales), pages, page, hkv, dim, _code(dtype),
                                   _ptr(out))
    return out


def write_fixed_scale(rows_f32, slot_mapping, pool8, scales, page_size=16):
    """Quantise fp32 rows [n, hkv, dim] into the (contiguous CPU uint8) pool in place."""
    rows_f32 = _dense(rows_f32).float()
    n, hkv, dim = rows_f32.shape
    slots = _dense(slot_mapping).long()
    scales = _dense(scales).float()
    assert pool8.is_contiguous() and pool8.dtype == torch.uint8
    library().qfo_write_fixed_scale(_ptr(rows_f32), _ptr(slots), n, hkv, dim, page_size,
                                    _ptr(scales), _ptr(pool8),
                                    pool8.shape[0] * pool8.shape[1])


# ---- metadata ---------------------------------------------------------------

def decode_step_inputs(cur_lens, block_tables, max_blocks, page_size=16):
    """Pure-Python restatement of build_decode_step_inputs
    (engine/graph/paged_graph_decoder.py:392-417): positions = cur-1, seq_lens =
    cur, slot = table[p // page] * page + p % page, table zero padded."""
    positions, seq_lens, slots, table = [], [], [], []
    for cur, pages in zip(cur_lens, block_tables):
        p = cur - 1
        positions.append(p)
        seq_lens.append(cur)
        slots.append(pages[p // page_size] * page_size + p % page_size)
        table.append(list(pages) + [0] * (max_blocks - len(pages)))
    return (np.asarray(positions, dtype=np.int32), np.asarray(seq_lens, dtype=np.int32),
            np.asarray(table, dtype=np.int32).reshape(len(cur_lens), max_blocks),
            np.asarray(slots, dtype=np.int64))


def advance_decode_state(positions, seq_lens, block_table, page_size=16):
    """numpy restatement of IterationLoop::advance_decode_state
    (engine/cpp/src/iteration_loop.cpp:500-528): positions + 1, lengths + 1, and
    slot = table[b, p // page] * page + p % page at the NEW position p (the same
    relation engine/cpp/tests/test_iteration_loop.py:545-551 asserts between
    consecutive decode rows).  Returns new (positions, seq_lens, slot_mapping int64);
    a position beyond the table is an IndexError, as the reference's gather."""
    positions = np.asarray(positions).astype(np.int64) + 1
    seq_lens = np.asarray(seq_lens).astype(np.int64) + 1
    table = np.asarray(block_table).astype(np.int64)
    logical = positions // page_size
    if len(positions) and (logical.max() >= table.shape[1] or positions.min() < 0):
        raise IndexError("position beyond the block table")
    pages = table[np.arange(len(positions)), logical] if len(positions) else np.zeros(0, np.int64)
    return positions, seq_lens, pages * page_size + positions % page_size


# ---- QKV projection with the RoPE / cache epilogue ---------------------------------

def qkv_projection(x, weight, bias=None):
    """x @ weight.T + bias with a float64 sum, rounded once to x's dtype: the model-dtype
    output of nn.Linear that the reference's epilogue rotates
    (custom_kernels/gemm_epilogue/fused_gemm.cu:262-267: accumulator + bias, then
    __float2half_rn)."""
    packed = x.detach().cpu().double() @ weight.detach().cpu().double().T
    if bias is not None:
        packed = packed + bias.detach().cpu().double()
    return packed.float().to(x.dtype)


def qkv_rope_cache(x, weight, bias, positions, slot_mapping, k_pool, v_pool, *, base=1_000_000.0,
                   valid_tokens=None):
    """The fused projection restated as its two steps: qkv_projection, then the packed
    epilogue (custom_kernels/fused_gemm.py:271-278).  Mutates the CPU pools, returns q."""
    return packed_qkv_rope_cache(qkv_projection(x, weight, bias), positions, slot_mapping, k_pool, v_pool,
                                 base=base, valid_tokens=valid_tokens)


# ---- RMSNorm -------------------------------------------------------------------

def rms_norm(x, weight, epsilon=1e-6):
    """RMSNorm of the last dimension in fp32, one rounding to x's dtype: restates
    rms_norm_reference (custom_kernels/fused_rms.py:137-140), whose arithmetic is the
    Triton kernel's (:38-42): weight * x / sqrt(mean(x^2) + epsilon).  The mean is
    accumulated in float64 and rounded once to fp32."""
    values = x.detach().cpu().float().numpy()
    mean = np.mean(values.astype(np.float64) ** 2, axis=-1, keepdims=True).astype(np.float32)
    rms = np.sqrt(mean + np.float32(epsilon), dtype=np.float32)
    scaled = (weight.detach().cpu().float().numpy() * values) / rms
    return torch.from_numpy(scaled.astype(np.float32)).to(x.dtype)


def residual_add_rms_norm(residual, branch, weight, epsilon=1e-6):
    """(residual + branch rounded to the model dtype, RMSNorm of that rounded sum):
    restates _residual_add_rms_norm_kernel (custom_kernels/fused_rms.py:78-104)."""
    summed = (residual.detach().cpu().float() + branch.detach().cpu().float()).to(residual.dtype)
    return summed, rms_norm(summed, weight, epsilon)


def ulp_distance(actual, expected):
    """|actual - expected| in units of the spacing of expected's own 16-bit format."""
    a, e = actual.detach().cpu(), expected.detach().cpu()
    fraction_bits = 10 if e.dtype == torch.float16 else 7
    smallest = -14 if e.dtype == torch.float16 else -126
    magnitude = e.float().abs().clamp_min(2.0 ** smallest)
    spacing = torch.exp2(torch.floor(torch.log2(magnitude)) - fraction_bits)
    return (a.float() - e.float()).abs() / spacing


def ulp_distance_fp16(actual, expected, reference_magnitude=None):
    """|actual - expected| in units of the fp16 spacing at max(|expected|,
    reference_magnitude): cancellation in x1*c - x2*s can leave a result far
    smaller than its operands, where one ulp of the result is not a meaningful
    yardstick."""
    a = actual.detach().cpu().float()
    e = expected.detach().cpu().float()
    magnitude = e.abs()
    if reference_magnitude is not None:
        magnitude = torch.maximum(magnitude, reference_magnitude.detach().cpu().float().abs())
    magnitude = magnitude.clamp_min(2.0 ** -14)
    spacing = torch.exp2(torch.floor(torch.log2(magnitude)) - 10)
    return (a - e).abs() / spacing
