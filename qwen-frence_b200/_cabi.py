"""ctypes binding of libqf_hotpath.so (declared in include/qf_hotpath.h).

This is the only place that touches the shared library.  There is no CPU or
PyTorch fallback: when the library is missing every operator raises with the
one command that builds it, like the reference's native wrapper does
(custom_kernels/paged_decode_native_grouped.py:17-27).
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_double, c_float, c_int32, c_int64, c_void_p
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
LIBRARY_PATH = PACKAGE_DIR / "libqf_hotpath.so"
BUILD_COMMAND = "python qwen-frence_b200/build.py"

ABI_VERSION = 1
DTYPE_F16, DTYPE_BF16 = 0, 1
INDEX_I32, INDEX_I64, INDEX_F32 = 0, 1, 2
KERNEL_INFO_FIELDS = (
    "registers_per_thread", "static_shared_bytes", "dynamic_shared_bytes",
    "local_bytes_per_thread", "max_threads_per_block", "binary_version", "ptx_version",
    "threads_per_block", "active_blocks_per_sm", "max_warps_per_sm", "pipeline_stages",
    "multiprocessor_count",
)

EXPORTED_SYMBOLS = (
    "qf_abi_version", "qf_last_error", "qf_rope_kv_write", "qf_rope_kv_write_fp8",
    "qf_quantize_kv_pages_e4m3", "qf_grouped_gqa_splitk_partial_out", "qf_splitk_reduce",
    "qf_grouped_splitk_decode_attention", "qf_grouped_gqa_splitk_diagnostics",
    "qf_grouped_gqa_splitk_profile_out", "qf_device_status", "qf_set_tuning",
    "qf_grouped_splitk_decode_attention_static", "qf_grouped_splitk_decode_attention_stages",
    "qf_grouped_splitk_decode_attention_plan", "qf_grouped_splitk_persistent_timeline",
    "qf_set_dependent_launch", "qf_order_next_launch", "qf_advance_decode_metadata",
    "qf_rms_norm", "qf_residual_add_rms_norm", "qf_qkv_rope_cache",
    "qf_qkv_rope_cache_timeline", "qf_packed_rope_decode_attention",
    "qf_build_rope_table",
)
KERNEL_NAMES = ("decode_partial_kernel", "decode_stream_kernel", "decode_mma_kernel", "decode_mma_kernel (solo)")
STAGE_PARTIAL, STAGE_COMBINE = 1, 2
GEMM_TIMELINE_COLUMNS = 10
STATIC_SCRATCH_BYTES = 16 << 20


class RopeKvWriteArgs(Structure):
    """Mirror of qf_rope_kv_write_args."""

    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("q_out", c_void_p),
        ("q_stride_row", c_int64), ("q_stride_head", c_int64), ("q_stride_d", c_int64),
        ("k_stride_row", c_int64), ("k_stride_head", c_int64), ("k_stride_d", c_int64),
        ("v_stride_row", c_int64), ("v_stride_head", c_int64), ("v_stride_d", c_int64),
        ("o_stride_row", c_int64), ("o_stride_head", c_int64), ("o_stride_d", c_int64),
        ("positions", c_void_p), ("positions_dtype", c_int32), ("positions_stride", c_int64),
        ("slot_mapping", c_void_p), ("slot_dtype", c_int32), ("slot_stride", c_int64),
        ("k_pool", c_void_p), ("v_pool", c_void_p),
        ("kp_stride_slot", c_int64), ("kp_stride_head", c_int64), ("kp_stride_d", c_int64),
        ("vp_stride_slot", c_int64), ("vp_stride_head", c_int64), ("vp_stride_d", c_int64),
        ("num_slots", c_int64),
        ("valid_tokens", c_void_p),
        ("rows", c_int32), ("q_heads", c_int32), ("kv_heads", c_int32), ("head_dim", c_int32),
        ("dtype", c_int32), ("rotate_q", c_int32),
        ("base", c_double),
    ]


class DecodeAttentionArgs(Structure):
    """Mirror of qf_decode_attention_args."""

    _fields_ = [
        ("q", c_void_p),
        ("q_stride_b", c_int64), ("q_stride_h", c_int64), ("q_stride_d", c_int64),
        ("k_pool", c_void_p), ("v_pool", c_void_p),
        ("k_stride_page", c_int64), ("k_stride_tok", c_int64), ("k_stride_head", c_int64),
        ("k_stride_d", c_int64),
        ("v_stride_page", c_int64), ("v_stride_tok", c_int64), ("v_stride_head", c_int64),
        ("v_stride_d", c_int64),
        ("block_table", c_void_p), ("table_dtype", c_int32),
        ("table_stride_b", c_int64), ("table_stride_p", c_int64), ("table_width", c_int64),
        ("seq_lens", c_void_p), ("lens_dtype", c_int32), ("lens_stride", c_int64),
        ("k_scale", c_void_p), ("v_scale", c_void_p),
        ("partial_out", c_void_p), ("partial_max", c_void_p), ("partial_sum", c_void_p),
        ("out", c_void_p),
        ("o_stride_b", c_int64), ("o_stride_h", c_int64), ("o_stride_d", c_int64),
        ("num_pages", c_int64),
        ("batch", c_int32), ("q_heads", c_int32), ("kv_heads", c_int32), ("head_dim", c_int32),
        ("page_size", c_int32), ("split_k", c_int32), ("dtype", c_int32), ("kv_fp8", c_int32),
        ("scale", c_float),
    ]


class QkvRopeCacheArgs(Structure):
    """Mirror of qf_qkv_rope_cache_args."""

    _fields_ = [
        ("hidden", c_void_p), ("hidden_stride_row", c_int64),
        ("weight", c_void_p), ("weight_stride_row", c_int64),
        ("bias", c_void_p),
        ("q_out", c_void_p), ("q_stride_row", c_int64),
        ("positions", c_void_p), ("positions_dtype", c_int32),
        ("slot_mapping", c_void_p), ("slot_dtype", c_int32),
        ("k_pool", c_void_p), ("v_pool", c_void_p),
        ("num_slots", c_int64),
        ("valid_tokens", c_void_p),
        ("rows", c_int32), ("in_features", c_int32), ("dtype", c_int32),
        ("base", c_double),
    ]


_library = None


def library():
    """Load libqf_hotpath.so once; fail loudly when it has not been built."""
    global _library
    if _library is not None:
        return _library
    if not LIBRARY_PATH.is_file():
        raise RuntimeError(
            f"libqf_hotpath.so is not built ({LIBRARY_PATH}); run: {BUILD_COMMAND}"
        )
    try:
        lib = ctypes.CDLL(str(LIBRARY_PATH))
    except OSError as exc:
        raise RuntimeError(
            f"libqf_hotpath.so could not be loaded ({exc}); rebuild it with: {BUILD_COMMAND}"
        ) from exc
    lib.qf_abi_version.restype = c_int32
    lib.qf_last_error.restype = ctypes.c_char_p
    if lib.qf_abi_version() != ABI_VERSION:
        raise RuntimeError(
            f"libqf_hotpath.so has ABI {lib.qf_abi_version()}, expected {ABI_VERSION}; "
            f"rebuild it with: {BUILD_COMMAND}"
        )
    lib.qf_rope_kv_write.argtypes = [POINTER(RopeKvWriteArgs), c_void_p]
    lib.qf_rope_kv_write_fp8.argtypes = [POINTER(RopeKvWriteArgs), c_void_p, c_void_p, c_int32, c_void_p]
    lib.qf_quantize_kv_pages_e4m3.argtypes = [
        c_void_p, c_int32, c_int64, c_int32, c_int32, c_int32, c_void_p, c_void_p, c_void_p]
    lib.qf_grouped_gqa_splitk_partial_out.argtypes = [POINTER(DecodeAttentionArgs), c_void_p]
    lib.qf_grouped_gqa_splitk_profile_out.argtypes = [POINTER(DecodeAttentionArgs), c_void_p, c_void_p]
    lib.qf_grouped_splitk_decode_attention.argtypes = [POINTER(DecodeAttentionArgs), c_void_p]
    lib.qf_grouped_splitk_decode_attention_static.argtypes = [POINTER(DecodeAttentionArgs), c_void_p]
    lib.qf_grouped_splitk_decode_attention_plan.argtypes = [
        POINTER(DecodeAttentionArgs), POINTER(c_int32), POINTER(c_int32)]
    lib.qf_grouped_splitk_persistent_timeline.argtypes = [
        POINTER(DecodeAttentionArgs), c_void_p, c_void_p]
    lib.qf_grouped_splitk_decode_attention_stages.argtypes = [
        POINTER(DecodeAttentionArgs), c_int32, c_void_p]
    lib.qf_splitk_reduce.argtypes = (
        [c_void_p] * 3 + [c_int64] * 7 + [c_void_p] + [c_int64] * 3 + [c_int32] * 5 + [c_void_p])
    lib.qf_grouped_gqa_splitk_diagnostics.argtypes = [c_int32, c_int32, c_int32, POINTER(c_int64)]
    lib.qf_device_status.argtypes = [POINTER(c_int32), c_int32]
    lib.qf_set_tuning.argtypes = [c_int32, c_int32]
    lib.qf_set_dependent_launch.argtypes = [c_int32]
    lib.qf_order_next_launch.argtypes = []
    lib.qf_advance_decode_metadata.argtypes = (
        [c_void_p, c_int32] * 4 + [c_int64] * 4 + [c_int32, c_int32, c_void_p])
    lib.qf_rms_norm.argtypes = [
        c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_int64, c_int32, c_int32, c_float, c_void_p]
    lib.qf_residual_add_rms_norm.argtypes = [
        c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_void_p, c_int64,
        c_int64, c_int32, c_int32, c_float, c_void_p]
    lib.qf_qkv_rope_cache.argtypes = [POINTER(QkvRopeCacheArgs), c_void_p]
    lib.qf_qkv_rope_cache_timeline.argtypes = [POINTER(QkvRopeCacheArgs), c_void_p, c_void_p]
    lib.qf_packed_rope_decode_attention.argtypes = [
        POINTER(DecodeAttentionArgs), c_void_p, c_int32, c_int64, c_void_p, c_int32, c_int32, c_void_p]
    lib.qf_build_rope_table.argtypes = [c_void_p, c_int32, c_double, c_void_p]
    for name in EXPORTED_SYMBOLS:
        if name not in ("qf_last_error",):
            getattr(lib, name).restype = c_int32
    _library = lib
    return lib


def check(status):
    """Turn a negative C status into RuntimeError carrying qf_last_error()."""
    if status != 0:
        message = library().qf_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"libqf_hotpath: {message} (status {status})")


# ---------------------------------------------------------------------------
# torch helpers (torch is imported lazily: the binding itself needs only ctypes)
# ---------------------------------------------------------------------------

def torch_dtype_code(dtype):
    import torch

    if dtype == torch.float16:
        return DTYPE_F16
    if dtype == torch.bfloat16:
        return DTYPE_BF16
    raise ValueError(f"unsupported element dtype {dtype}")


def torch_index_code(dtype, allow_float=False):
    import torch

    if dtype == torch.int32:
        return INDEX_I32
    if dtype == torch.int64:
        return INDEX_I64
    if allow_float and dtype == torch.float32:
        return INDEX_F32
    raise ValueError(f"unsupported index dtype {dtype}")


def stream_pointer(device):
    """The current torch stream of `device`, as the void* the C ABI takes."""
    import torch

    return torch.cuda.current_stream(device).cuda_stream


class device_of:
    """Make `tensor.device` current for the duration of a library call."""

    def __init__(self, tensor):
        import torch

        self._torch = torch
        self._index = tensor.device.index
        self._guard = None

    def __enter__(self):
        torch = self._torch
        if self._index is not None and torch.cuda.current_device() != self._index:
            self._guard = torch.cuda.device(self._index)
            self._guard.__enter__()
        return self

    def __exit__(self, *exc):
        if self._guard is not None:
            self._guard.__exit__(*exc)
        return False


def set_dependent_launch(enabled=True):
    """Programmatic dependent launch of the hot kernels on (default) or off."""
    check(library().qf_set_dependent_launch(1 if enabled else 0))


def order_next_launch():
    """The next kernel of the library starts only after everything earlier on its
    stream has completed (needed after a foreign kernel rewrote step metadata)."""
    check(library().qf_order_next_launch())


def fused_kernel_plan(args):
    """(kernel name, resident CTAs per KV head) the fused attention call would use."""
    kernel, ctas = c_int32(0), c_int32(0)
    check(library().qf_grouped_splitk_decode_attention_plan(
        ctypes.byref(args), ctypes.byref(kernel), ctypes.byref(ctas)))
    return KERNEL_NAMES[kernel.value], ctas.value


def device_status(reset=True):
    """Status word of the kernels on the current device (0 = clean, 2 = bad page id,
    3 = merge poll gave up, 4 = a position advanced past its block table)."""
    value = c_int32(0)
    check(library().qf_device_status(ctypes.byref(value), 1 if reset else 0))
    return value.value


def set_tuning(stages=0, force_generic=False):
    """Kernel selection for tests: force_generic 1 (or True) sends every launch to the
    stride-generic kernel, 2 keeps the fast per-partition kernel but turns the
    persistent ones off, 3 / 4 use the persistent CUDA-core / tensor-core kernel
    whenever the layout allows (also for batches with few split slots), 5 the
    tensor-core kernel's solo variant (4 never picks it); 0 restores the defaults."""
    check(library().qf_set_tuning(int(stages), int(force_generic)))
