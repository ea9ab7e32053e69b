"""GPU test of qf_grouped_splitk_decode_attention_static, the entry point for
callers that cannot allocate the split-K partial buffers (hosts without a caching
allocator, or whose device memory is already fully claimed): its partials live in
a static device array inside the library.

Collected last on purpose, so a run that stops at the first failure has already
run every other test.  Passes alone in a fresh process and after the other tests:
it relies on no state but the library's own array, whose old contents must not
matter, which is why each comparison is made on two calls in a row with different
inputs.  Each call is also checked against the CPU oracle, and against the claim in
its name: device memory in use is the same before and after the call."""

from __future__ import annotations

import ctypes

import pytest
import torch

from conftest import assert_attention_close, make_paged_inputs

pytestmark = pytest.mark.gpu


calls_so_far = {"count": 0}


def _run_both(package, oracle, device, lengths, split_k, seed):
    q, k, v, table, lens = make_paged_inputs(lengths, seed=seed, value_scale=0.5, poison=True)
    dq, dk, dv, dtable, dlens = (t.to(device) for t in (q, k, v, table, lens))
    reference = package.grouped_splitk_decode_attention(dq, dk, dv, dtable, dlens, split_k=split_k)

    # straight through the C ABI: the caller passes inputs and the output, no partials
    cabi = package.cabi
    splitk = package.kernel_module("paged_decode_grouped_splitk")
    out = torch.full_like(dq, float("nan"))
    args = splitk.fill_attention_args(cabi, dq, dk, dv, dtable, dlens, split_k=split_k,
                                      scale=128 ** -0.5, partials=None, out=out)
    assert not args.partial_out and not args.partial_max and not args.partial_sum
    stream = cabi.stream_pointer(device)
    torch.cuda.synchronize()
    # the claim in the name: with the output preallocated, the call takes nothing from any allocator
    allocated, reserved = torch.cuda.memory_allocated(device), torch.cuda.memory_reserved(device)
    free_before, _ = torch.cuda.mem_get_info(device)
    status = cabi.library().qf_grouped_splitk_decode_attention_static(ctypes.byref(args), stream)
    assert status == 0, cabi.library().qf_last_error()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(device) == allocated and torch.cuda.memory_reserved(device) == reserved
    if calls_so_far["count"] > 0:  # a first call may make the driver load the kernels' code
        assert torch.cuda.mem_get_info(device)[0] >= free_before, "the call took device memory"
    calls_so_far["count"] += 1
    expected = oracle.paged_attention(q, k, v, table, lens)
    assert_attention_close(out, expected)
    return out, reference, (dq, dk, dv, dtable, dlens)


def test_static_scratch_matches_the_allocating_entry_point_twice_in_a_row(package, oracle, cuda_device):
    first, ref_first, _ = _run_both(package, oracle, cuda_device, [0, 1, 17, 100, 700, 2048], split_k=6, seed=31)
    assert_attention_close(first, ref_first)
    # second call: other shapes and split count, so stale partials of the first call sit
    # in the array at different offsets than this call's rows
    second, ref_second, tensors = _run_both(package, oracle, cuda_device, [513, 64, 3, 1500], split_k=9, seed=32)
    assert_attention_close(second, ref_second)
    # same kernels, same data: the two entry points agree to the last bit
    assert torch.equal(first, ref_first) and torch.equal(second, ref_second)
    # the Python wrapper reaches the same entry point
    out = torch.empty_like(tensors[0])
    again = package.grouped_splitk_decode_attention_static(*tensors, out, split_k=9)
    assert again is out and torch.equal(out, ref_second)


def test_static_scratch_rejects_requests_beyond_its_size(package, cuda_device):
    cabi = package.cabi
    q, k, v, table, lens = (t.to(cuda_device) for t in make_paged_inputs([40] * 64, seed=3))
    out = torch.empty_like(q)
    too_many_splits = cabi.STATIC_SCRATCH_BYTES // (64 * 12 * 130 * 4) + 1
    with pytest.raises(RuntimeError, match="QF_STATIC_SCRATCH_BYTES"):
        package.grouped_splitk_decode_attention_static(q, k, v, table, lens, out, split_k=too_many_splits)
    # the largest request that fits is accepted
    package.grouped_splitk_decode_attention_static(q, k, v, table, lens, out, split_k=too_many_splits - 1)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
