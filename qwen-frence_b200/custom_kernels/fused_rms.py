"""RMSNorm and residual-add + RMSNorm of the decode layer, as sm_100a kernels.

Drop-in for custom_kernels/fused_rms.py: `rms_norm` (:52-75) and
`residual_add_rms_norm` (:107-135) keep their names, signatures and error
behaviour, so baseline/kernel_dispatch.py and the graph decoder
(engine/graph/paged_graph_decoder.py:303-309, :325-331) call them unchanged.
The residual sum is materialised once, rounded to the model dtype, and the
normalisation reads that rounded value:

    summed     = (residual + branch)                     in fp16 / bf16
    normalized = (weight * float(summed) / sqrt(mean(float(summed)^2) + epsilon))

The work is done by qf_rms_norm / qf_residual_add_rms_norm in libqf_hotpath.so;
there is no Triton and no PyTorch fallback.
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


def _assert(condition, message):
    """The reference's rms_norm checks its arguments with assert statements."""
    if not condition:
        raise AssertionError(message)


def rms_norm(x, weight, epsilon=1e-6):
    """RMSNorm of every row of a contiguous (rows, N) fp16 / bf16 matrix; returns a new
    tensor.  Mirrors custom_kernels/fused_rms.py:52-75 (assertions included)."""
    import torch

    _assert(x.ndim == 2, "expected a (rows, N) input")
    _assert(x.is_contiguous(), "kernel assumes row-major contiguous input")
    _assert(weight.ndim == 1 and weight.shape[0] == x.shape[1], "weight must be (N,)")
    if not x.is_cuda or weight.device != x.device:
        raise ValueError("x and weight must live on one CUDA device")
    if x.dtype not in (torch.float16, torch.bfloat16) or weight.dtype != x.dtype:
        raise ValueError("expected FP16 or BF16 input and a weight of the same dtype")
    cabi = _cabi()
    weight = weight.contiguous()
    out = torch.empty_like(x)
    rows, hidden = x.shape
    with cabi.device_of(x):
        cabi.check(cabi.library().qf_rms_norm(
            x.data_ptr(), x.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0),
            rows, hidden, cabi.torch_dtype_code(x.dtype), float(epsilon),
            cabi.stream_pointer(x.device)))
    return out


def residual_add_rms_norm(residual, branch, weight, epsilon=1e-6):
    """Return ``(residual + branch, RMSNorm(residual + branch))`` from one kernel.
    Mirrors custom_kernels/fused_rms.py:107-135, ValueError wording included."""
    import torch

    if residual.shape != branch.shape or residual.dtype != branch.dtype:
        raise ValueError("residual and branch must have matching shapes and dtypes")
    if residual.ndim < 2 or residual.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("expected rank >= 2 FP16 or BF16 residual tensors")
    if not residual.is_contiguous() or not branch.is_contiguous():
        raise ValueError("residual and branch must be contiguous")
    if weight.ndim != 1 or weight.shape[0] != residual.shape[-1]:
        raise ValueError("RMSNorm weight must match the hidden dimension")
    if weight.device != residual.device or weight.dtype != residual.dtype:
        raise ValueError("weight must share the residual device and dtype")
    if not residual.is_cuda or branch.device != residual.device:
        raise ValueError("residual and branch must live on one CUDA device")
    cabi = _cabi()
    weight = weight.contiguous()
    hidden = residual.shape[-1]
    rows = residual.numel() // hidden if hidden else 0
    summed = torch.empty_like(residual)
    normalized = torch.empty_like(residual)
    if rows == 0 or hidden == 0:
        return summed, normalized
    with cabi.device_of(residual):
        cabi.check(cabi.library().qf_residual_add_rms_norm(
            residual.data_ptr(), hidden, branch.data_ptr(), hidden, weight.data_ptr(),
            summed.data_ptr(), hidden, normalized.data_ptr(), hidden,
            rows, hidden, cabi.torch_dtype_code(residual.dtype), float(epsilon),
            cabi.stream_pointer(residual.device)))
    return summed, normalized
