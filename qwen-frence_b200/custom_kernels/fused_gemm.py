"""QKV projection with RoPE + paged KV-cache write as its epilogue (decode), sm_100a.

Drop-in for the one entry of custom_kernels/fused_gemm.py that sits on the decode
attention path: `qkv_rope_cache` (:271-278; CUTLASS source
custom_kernels/gemm_epilogue/fused_gemm.cu:223-310), which the graph decoder calls as

    q = fused.qkv_rope_cache(h.reshape(B, d_model), qkv_proj.weight, qkv_proj.bias, None,
                             positions=positions.to(torch.long), slots=slot_mapping,
                             k_pool=cache.k_pool[i], v_pool=cache.v_pool[i], theta=cfg.rope_theta)

(engine/graph/paged_graph_decoder.py:218-224).  The result equals
packed_qkv_rope_cache(qkv_proj(h), ...): the projection is rounded to the model dtype
before the rotation, as in the reference's epilogue.  The norm-folding variant
(`partials` given: per-row RMS scale applied inside the GEMM) is a separate
experiment of the reference and is not offered; passing partials raises.
"""

from __future__ import annotations

import importlib.util
import sys
from pathlib import Path

Q_HEADS, KV_HEADS, HEAD_DIM = 12, 2, 128
QKV_WIDTH = (Q_HEADS + 2 * KV_HEADS) * HEAD_DIM  # 2048


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


def qkv_rope_cache_timeline(x, weight, bias, partials, *, positions, slots, k_pool, v_pool,
                            valid_tokens=None, theta=1_000_000.0):
    """The same call, also returning per-CTA %globaltimer stamps [CTAs, 10] (int64,
    nanoseconds): entry, barriers and TMEM ready, previous kernel complete, first operand
    tiles landed, last MMA issued, accumulator complete, partial sums sent, peers' sums
    arrived, outputs stored, TMEM released.  CTAs that do not exist for this shape stay 0."""
    return qkv_rope_cache(x, weight, bias, partials, positions=positions, slots=slots, k_pool=k_pool,
                          v_pool=v_pool, valid_tokens=valid_tokens, theta=theta, _timeline=True)


def qkv_rope_cache(x, weight, bias, partials, *, positions, slots, k_pool, v_pool,
                   valid_tokens=None, hidden=None, eps=1e-6, theta=1_000_000.0, config=-1,
                   _timeline=False):
    """QKV + bias, rotate-half RoPE, K/V into the paged cache; returns Q [M, 12, 128].

    x: (M, K) fp16 / bf16 with unit stride inside a row; weight: (2048, K), the
    nn.Linear layout; bias: (2048,) or None; positions, slots: (M,) int32 / int64;
    pools: contiguous (pages, page, 2, 128).  Padded rows (>= valid_tokens) get zero Q
    and never touch the cache.  `hidden`, `eps` and `config` belong to the reference's
    norm folding and CUTLASS tile choice; they are accepted and ignored.
    """
    import torch

    _require(partials is None, "norm folding (partials) is not offered by this kernel")
    _require(x.ndim == 2 and weight.ndim == 2 and weight.shape[0] == QKV_WIDTH and
             weight.shape[1] == x.shape[1], "expected x (M, K) and weight (2048, K)")
    _require(x.dtype in (torch.float16, torch.bfloat16) and weight.dtype == x.dtype,
             "x and weight must share an FP16 or BF16 dtype")
    _require(bias is None or (tuple(bias.shape) == (QKV_WIDTH,) and bias.dtype == x.dtype),
             "bias must be (2048,) in the dtype of x")
    rows, width = x.shape
    _require(width % 64 == 0, "the input width must be a multiple of 64")
    _require(tuple(positions.shape) == (rows,) and tuple(slots.shape) == (rows,),
             "positions and slots must hold one entry per row")
    _require(k_pool.ndim == 4 and k_pool.shape == v_pool.shape and k_pool.shape[2] == KV_HEADS and
             k_pool.shape[3] == HEAD_DIM, "expected paged K/V pools shaped (pages, page, 2, 128)")
    _require(k_pool.dtype == x.dtype and v_pool.dtype == x.dtype, "pools must share the dtype of x")
    _require(k_pool.is_contiguous() and v_pool.is_contiguous(), "pools must be contiguous")
    tensors = [x, weight, positions, slots, k_pool, v_pool] + ([bias] if bias is not None else [])
    _require(all(t.is_cuda for t in tensors), "every tensor must live on a CUDA device")
    _require(len({t.device for t in tensors}) == 1, "every tensor must share one device")
    _require(x.stride(1) == 1 and weight.stride(1) == 1, "x and weight rows must have unit stride")
    if valid_tokens is not None:
        _require(valid_tokens.is_cuda and valid_tokens.dtype == torch.int32 and valid_tokens.numel() == 1,
                 "valid_tokens must be a CUDA int32 scalar")
    cabi = _cabi()
    positions, slots = positions.contiguous(), slots.contiguous()
    bias = bias.contiguous() if bias is not None else None
    q = torch.empty((rows, Q_HEADS, HEAD_DIM), dtype=x.dtype, device=x.device)
    if rows == 0:
        return q
    args = cabi.QkvRopeCacheArgs()
    args.hidden, args.hidden_stride_row = x.data_ptr(), x.stride(0)
    args.weight, args.weight_stride_row = weight.data_ptr(), weight.stride(0)
    args.bias = bias.data_ptr() if bias is not None else None
    args.q_out, args.q_stride_row = q.data_ptr(), Q_HEADS * HEAD_DIM
    args.positions, args.positions_dtype = positions.data_ptr(), cabi.torch_index_code(positions.dtype, allow_float=True)
    args.slot_mapping, args.slot_dtype = slots.data_ptr(), cabi.torch_index_code(slots.dtype)
    args.k_pool, args.v_pool = k_pool.data_ptr(), v_pool.data_ptr()
    args.num_slots = k_pool.shape[0] * k_pool.shape[1]
    args.valid_tokens = valid_tokens.data_ptr() if valid_tokens is not None else None
    args.rows, args.in_features, args.dtype = rows, width, cabi.torch_dtype_code(x.dtype)
    args.base = float(theta)
    import ctypes

    with cabi.device_of(x):
        if _timeline:
            ctas = 32 * (-(-rows // 128)) * 4
            timeline = torch.zeros((ctas, cabi.GEMM_TIMELINE_COLUMNS), dtype=torch.int64, device=x.device)
            cabi.check(cabi.library().qf_qkv_rope_cache_timeline(
                ctypes.byref(args), timeline.data_ptr(), cabi.stream_pointer(x.device)))
            return q, timeline
        cabi.check(cabi.library().qf_qkv_rope_cache(ctypes.byref(args), cabi.stream_pointer(x.device)))
    return q
