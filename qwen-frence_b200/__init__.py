"""B200-native decode-step attention hot path of Qwen-frence.

The directory is named `qwen-frence_b200`, which is not an importable
identifier; load it with `__graft_entry__.load_package()` (module name
`qwen_frence_b200`) or point the reference's `kernel_dispatch._KERNEL_DIR` at
`qwen-frence_b200/custom_kernels/`, whose files carry the reference's module
and function names.

Public operators (all enqueue sm_100a kernels from libqf_hotpath.so on the
current torch stream; none has a CPU fallback):

    rope_kv_write, native_decode_rope_kv_write            custom_kernels/rope_kv_write.py
    packed_qkv_rope_cache                                  custom_kernels/packed_qkv_rope_cache.py
    grouped_splitk_decode_attention, splitk_reduce         custom_kernels/paged_decode_grouped_splitk.py
    native_grouped_splitk_decode_attention,
    grouped_gqa_splitk_partial_out,
    native_grouped_decode_diagnostics,
    native_grouped_stage_cycles,
    native_grouped_persistent_timeline                     custom_kernels/paged_decode_native_grouped.py
    quantize_kv_pool_e4m3, dequantize_kv_pool_e4m3,
    native_decode_rope_kv_write_fp8, packed_qkv_rope_cache_fp8,
    grouped_splitk_decode_attention_fp8,
    packed_qkv_rope_attention_fp8                          custom_kernels/fp8_paged_kv.py
    advance_decode_state                                   custom_kernels/decode_state.py
    rms_norm, residual_add_rms_norm                        custom_kernels/fused_rms.py
    qkv_rope_cache, qkv_rope_cache_timeline                custom_kernels/fused_gemm.py
    packed_qkv_rope_attention, build_rope_table            custom_kernels/fused_decode_step.py
"""

from __future__ import annotations

import importlib
import importlib.util
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
KERNEL_DIR = PACKAGE_DIR / "custom_kernels"

_EXPORTS = {
    "rope_kv_write": "rope_kv_write",
    "native_decode_rope_kv_write": "rope_kv_write",
    "packed_qkv_rope_cache": "packed_qkv_rope_cache",
    "grouped_splitk_decode_attention": "paged_decode_grouped_splitk",
    "splitk_reduce": "paged_decode_grouped_splitk",
    "grouped_splitk_decode_attention_static": "paged_decode_grouped_splitk",
    "native_grouped_splitk_decode_attention": "paged_decode_native_grouped",
    "grouped_gqa_splitk_partial_out": "paged_decode_native_grouped",
    "native_grouped_decode_diagnostics": "paged_decode_native_grouped",
    "native_grouped_stage_cycles": "paged_decode_native_grouped",
    "native_grouped_persistent_timeline": "paged_decode_native_grouped",
    "quantize_kv_pool_e4m3": "fp8_paged_kv",
    "dequantize_kv_pool_e4m3": "fp8_paged_kv",
    "native_decode_rope_kv_write_fp8": "fp8_paged_kv",
    "packed_qkv_rope_cache_fp8": "fp8_paged_kv",
    "grouped_splitk_decode_attention_fp8": "fp8_paged_kv",
    "packed_qkv_rope_attention_fp8": "fp8_paged_kv",
    "advance_decode_state": "decode_state",
    "rms_norm": "fused_rms",
    "residual_add_rms_norm": "fused_rms",
    "qkv_rope_cache": "fused_gemm",
    "qkv_rope_cache_timeline": "fused_gemm",
    "packed_qkv_rope_attention": "fused_decode_step",
    "build_rope_table": "fused_decode_step",
}
_LOCAL = {"cabi": "_cabi", "build": "build", "kv_layout": "kv_layout", "workloads": "workloads",
          "decode_step": "decode_step", "sharding": "sharding"}


def _load(key, path):
    module = sys.modules.get(key)
    if module is None:
        spec = importlib.util.spec_from_file_location(key, path)
        module = importlib.util.module_from_spec(spec)
        sys.modules[key] = module
        spec.loader.exec_module(module)
    return module


def kernel_module(name):
    """One of the drop-in modules under custom_kernels/, loaded by path."""
    return _load(f"qf_hotpath_{name}", KERNEL_DIR / f"{name}.py")


def __getattr__(name):
    if name in _EXPORTS:
        return getattr(kernel_module(_EXPORTS[name]), name)
    if name == "cabi":
        # one shared instance with the drop-in modules, which load it by path
        return _load("qf_hotpath_cabi", PACKAGE_DIR / "_cabi.py")
    if name in _LOCAL:
        return importlib.import_module(f"{__name__}.{_LOCAL[name]}")
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")


__all__ = sorted(_EXPORTS) + sorted(_LOCAL) + ["kernel_module", "KERNEL_DIR", "PACKAGE_DIR"]
