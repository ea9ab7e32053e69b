"""GPU parity of GQA paged decode attention (split-K partial pass + combine) against
the CPU oracle and the committed reference outputs.  Every call goes through the
C ABI via the drop-in modules.

Bar: max-abs 2e-3 and rel 1e-2 against an fp32-accumulated reference for fp16
(the reference's own gate atol = rtol = 2e-3 is applied; 2e-2 for bf16)."""

from __future__ import annotations

import pytest
import torch

from conftest import (assert_attention_close, attention_case_tensors, make_paged_inputs, with_gaps)

pytestmark = pytest.mark.gpu


def _to(device, *tensors):
    return tuple(t.to(device) for t in tensors)


def _fast_path_inputs(device, lengths, **kwargs):
    """Contiguous Qwen-geometry inputs (the fast kernels' layout) on the device."""
    q, k, v, table, lens = make_paged_inputs(lengths, **kwargs)
    return (q, k, v, table, lens), _to(device, q, k, v, table, lens)


@pytest.mark.parametrize("split_k", [1, 2, 7, 22])
def test_golden_cases_every_split(package, attention_golden, cuda_device, split_k):
    """Reference outputs for ragged / strided / NaN-poisoned / boundary / adversarial
    inputs.  Strided cases are re-strided on the device (generic kernel); the
    contiguous ones take the fast kernels."""
    for name in attention_golden.names:
        fields = attention_golden.case(name)
        q, k, v, table, lens, scale, expected = attention_case_tensors(fields)
        dq, dk, dv, dtable, dlens = _to(cuda_device, q, k, v, table, lens)
        if tuple(fields["q_stride"]) != tuple(q.stride()):
            dq, dv, dtable, dlens = map(with_gaps, (dq, dv, dtable, dlens))
        out = package.grouped_splitk_decode_attention(dq, dk, dv, dtable, dlens, split_k=split_k, scale=scale)
        assert_attention_close(out, expected)
        assert torch.isfinite(out.float()).all(), name


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("split_k", [1, 3, 8])
def test_fast_kernel_ragged_poisoned(package, oracle, cuda_device, dtype, split_k):
    """Contiguous layout -> fast kernels.  Lengths straddle page boundaries, the tail
    of every last page is NaN, the table is padded with -1."""
    lengths = [0, 1, 15, 16, 17, 31, 32, 33, 81, 100, 129, 513, 1000]
    host, dev = _fast_path_inputs(cuda_device, lengths, dtype=dtype, seed=42, poison=True)
    expected = oracle.paged_attention(*host)
    out = package.grouped_splitk_decode_attention(*dev, split_k=split_k)
    assert_attention_close(out, expected)
    if split_k >= 2:
        native = package.native_grouped_splitk_decode_attention(*dev, split_k=split_k)
        assert torch.equal(native, out)


def test_fast_and_generic_kernels_agree(package, oracle, cuda_device):
    lengths = [5, 64, 257, 2048]
    host, dev = _fast_path_inputs(cuda_device, lengths, seed=3, value_scale=0.5)
    fast = package.grouped_splitk_decode_attention(*dev, split_k=4)
    package.cabi.set_tuning(force_generic=True)
    try:
        generic = package.grouped_splitk_decode_attention(*dev, split_k=4)
    finally:
        package.cabi.set_tuning()
    expected = oracle.paged_attention(*host)
    assert_attention_close(fast, expected)
    assert_attention_close(generic, expected)


@pytest.mark.parametrize("stages", [1, 3, 4, 12])
def test_pipeline_depths(package, oracle, cuda_device, stages):
    """Ring depths from the minimum (requests below three are raised to three) to the
    maximum give the same answer; partitions longer than 32 pages cross the page-id
    batch boundary."""
    lengths = [16 * 70 + 5, 16 * 33, 16 * 32, 40]
    host, dev = _fast_path_inputs(cuda_device, lengths, seed=8)
    expected = oracle.paged_attention(*host)
    package.cabi.set_tuning(stages=stages)
    try:
        for split_k in (1, 2):
            out = package.grouped_splitk_decode_attention(*dev, split_k=split_k)
            assert_attention_close(out, expected)
    finally:
        package.cabi.set_tuning()


def test_partials_match_oracle_partition_by_partition(package, oracle, cuda_device):
    """The fp32 partial buffers, partition by partition: out/sum rescaled to a
    common offset equal the oracle's; empty partitions are (0, -inf, 0)."""
    lengths = [0, 1, 17, 100, 700]
    split_k = 5
    host, dev = _fast_path_inputs(cuda_device, lengths, seed=11, value_scale=0.5)
    batch = len(lengths)
    partials = (torch.full((batch, split_k, 12, 128), float("nan"), device=cuda_device),
                torch.full((batch, split_k, 12), float("nan"), device=cuda_device),
                torch.full((batch, split_k, 12), float("nan"), device=cuda_device))
    package.grouped_gqa_splitk_partial_out(*dev, *partials, 128 ** -0.5)
    out = package.splitk_reduce(*partials, torch.empty_like(dev[0]))
    po, pm, ps = (t.cpu() for t in partials)
    ro, rm, rs = oracle.splitk_partial(*host, split_k=split_k)
    empty = rs == 0
    assert torch.equal(ps == 0, empty)
    assert torch.isinf(pm[empty]).all() and (pm[empty] < 0).all()
    assert (po[empty] == 0).all()
    # common offset: oracle's exact maximum
    factor = torch.where(empty, torch.zeros_like(pm), torch.exp(pm - rm))
    torch.testing.assert_close(ps * factor, rs, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(po * factor[..., None], ro, atol=2e-3, rtol=2e-3)
    assert_attention_close(out, oracle.splitk_reduce(ro, rm, rs))
    # the fused entry point (persistent kernel, pieces instead of partitions)
    fused = package.native_grouped_splitk_decode_attention(*dev, split_k=split_k)
    assert_attention_close(fused, out)


def test_known_answers(package, cuda_device):
    """experiments/tests/test_grouped_splitk_pipelined.py:40-66, :112-119."""
    dev = cuda_device
    q, k, v, table, lens = make_paged_inputs([0, 1, 17], poison=True)
    q.zero_()
    v[:, :, 0] = 3
    v[:, :, 1] = 9
    expected = torch.zeros_like(q)
    expected[1:, :6] = 3
    expected[1:, 6:] = 9
    for split_k in (1, 2, 7):
        out = package.grouped_splitk_decode_attention(*_to(dev, q, k, v, table, lens), split_k=split_k)
        assert torch.equal(out.cpu(), expected)

    q, k, v, table, lens = make_paged_inputs([1024])
    q.zero_(), k.zero_(), v.fill_(128)
    for split_k in (1, 2, 8):
        out = package.grouped_splitk_decode_attention(*_to(dev, q, k, v, table, lens), split_k=split_k)
        assert torch.equal(out.cpu(), torch.full_like(q, 128))  # fp32 partials: no fp16 overflow

    q, k, v, table, lens = make_paged_inputs([0, 0])
    for split_k in (1, 7):
        out = package.grouped_splitk_decode_attention(
            *_to(dev, q, k, v), table[:, :0].to(dev), lens.to(dev), split_k=split_k)
        assert torch.equal(out.cpu(), torch.zeros_like(q))


def test_large_scores_move_the_offset(package, oracle, cuda_device):
    """Scores that grow along the sequence force the running offset to move many
    times (the lazy-rescale branch), and scores far apart underflow cleanly."""
    lengths = [300, 45]
    q, k, v, table, lens = make_paged_inputs(lengths, seed=5)
    ramp = torch.linspace(0.0, 6.0, 16)[None, :, None, None]
    k.mul_(ramp.half())  # later rows of every page dominate
    host = (q, k, v, table, lens)
    expected = oracle.paged_attention(*host, scale=1.0)
    for split_k in (1, 3):
        out = package.grouped_splitk_decode_attention(*_to(cuda_device, *host), split_k=split_k, scale=1.0)
        assert_attention_close(out, expected)


@pytest.mark.parametrize("index_dtype", [torch.int32, torch.int64])
def test_index_dtypes_and_q_view(package, oracle, cuda_device, index_dtype):
    """int32/int64 metadata; q as the (B, 12, 1, 128)[:, :, 0, :] view the graph
    decoder passes (engine/graph/paged_graph_decoder.py:283-284)."""
    host, dev = _fast_path_inputs(cuda_device, [33, 130, 7], seed=2)
    dq, dk, dv, dtable, dlens = dev
    q4 = dq[:, :, None, :].contiguous()
    out = package.grouped_splitk_decode_attention(
        q4[:, :, 0, :], dk, dv, dtable.to(index_dtype), dlens.to(index_dtype), split_k=2)
    assert_attention_close(out, oracle.paged_attention(*host))


def test_other_geometries_use_generic_kernel(package, oracle, cuda_device):
    """Page 32, head_dim 64, group 4 / 3 KV heads: what the reference's Triton kernel
    accepts beyond the Qwen geometry."""
    host = make_paged_inputs([31, 32, 33, 129], page_size=32, kv_heads=3, group=4, head_dim=64, seed=6)
    expected = oracle.paged_attention(*host)
    for split_k in (1, 3):
        out = package.grouped_splitk_decode_attention(*_to(cuda_device, *host), split_k=split_k)
        assert_attention_close(out, expected)


def test_graph_replay_reads_updated_inputs(package, oracle, cuda_device):
    """Capture once, mutate q and seq_lens in place, replay
    (experiments/tests/test_grouped_splitk_pipelined.py:121-137)."""
    host, dev = _fast_path_inputs(cuda_device, [70, 70], seed=0)
    dq, dk, dv, dtable, dlens = dev
    for split_k in (1, 7):
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            package.grouped_splitk_decode_attention(dq, dk, dv, dtable, dlens, split_k=split_k)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            actual = package.grouped_splitk_decode_attention(dq, dk, dv, dtable, dlens, split_k=split_k)
        torch.cuda.current_stream().wait_stream(stream)
        dq.mul_(0.5)
        dlens.copy_(torch.tensor([0, 17], device=cuda_device, dtype=torch.int32))
        graph.replay()
        torch.cuda.synchronize()
        expected = oracle.paged_attention(dq.cpu(), host[1], host[2], host[3], dlens.cpu())
        assert_attention_close(actual, expected)
        dq.mul_(2.0)
        dlens.copy_(host[4].to(cuda_device))


def test_preallocated_partials_and_k1_contract(package, oracle, cuda_device):
    """K=1 returns partial_out.squeeze(1) in the q dtype; preallocated buffers are used."""
    host, dev = _fast_path_inputs(cuda_device, [1, 17, 81], seed=1)
    expected = oracle.paged_attention(*host)
    out = package.grouped_splitk_decode_attention(*dev, split_k=1)
    assert out.dtype == torch.float16 and out.shape == (3, 12, 128)
    assert_attention_close(out, expected)
    partials = (torch.empty(3, 4, 12, 128, device=cuda_device), torch.empty(3, 4, 12, device=cuda_device),
                torch.empty(3, 4, 12, device=cuda_device))
    out = package.grouped_splitk_decode_attention(*dev, split_k=4, partials=partials)
    assert_attention_close(out, expected)
    with pytest.raises(ValueError, match="do not match this launch shape"):
        package.grouped_splitk_decode_attention(*dev, split_k=5, partials=partials)


def test_validation_errors(package, cuda_device):
    (_, dev) = _fast_path_inputs(cuda_device, [17, 81])
    q, k, v, table, lens = dev
    for bad in (0, -1, 1.5):
        with pytest.raises(ValueError, match="positive integer"):
            package.grouped_splitk_decode_attention(q, k, v, table, lens, split_k=bad)
    with pytest.raises(ValueError, match="divisible"):
        package.grouped_splitk_decode_attention(q[:, :11], k, v, table, lens, split_k=2)
    with pytest.raises(ValueError, match="heads_per_program"):
        package.grouped_splitk_decode_attention(q, k, v, table, lens, split_k=2, heads_per_program=4)
    with pytest.raises(ValueError, match="split_k >= 2"):
        package.native_grouped_splitk_decode_attention(q, k, v, table, lens, split_k=1)
    with pytest.raises(ValueError, match="integer tensors"):
        package.grouped_splitk_decode_attention(q, k, v, table.float(), lens, split_k=2)


def test_diagnostics_and_stage_cycles(package, cuda_device):
    (_, dev) = _fast_path_inputs(cuda_device, [400, 90])
    q, k, v, table, lens = dev
    info = package.native_grouped_decode_diagnostics(q, table)
    assert info["threads_per_block"] == 256 and info["binary_version"] >= 100
    assert info["active_blocks_per_sm"] >= 1 and info["registers_per_thread"] <= 128
    cycles = package.native_grouped_stage_cycles(q, k, v, table, lens, split_k=2)
    assert cycles.shape == (2, 2, 2, 4) and cycles.dtype == torch.int64
    assert (cycles[..., 1] > 0).all()


def test_bad_page_id_is_reported_not_dereferenced(package, cuda_device):
    """A page id outside the pool reads as zeros and raises the status word; no fault."""
    (_, dev) = _fast_path_inputs(cuda_device, [40])
    q, k, v, table, lens = dev
    table = table.clone()
    table[0, 1] = 10_000
    out = package.grouped_splitk_decode_attention(q, k, v, table, lens, split_k=1)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert package.cabi.device_status() == 2
    assert package.cabi.device_status() == 0


# ---------------------------------------------------------------------------
# The persistent kernels behind the fused entry point (split_k >= 2): CTAs share
# the batch's pages equally, so a CTA's share crosses sequence boundaries.  Mode 3
# is the CUDA-core kernel, mode 4 the tensor-core kernel whose warps interleave over the
# pages (the instrumented variant), mode 5 its solo variant (what every call runs).
# ---------------------------------------------------------------------------
PERSISTENT = pytest.mark.parametrize("mode", [3, 4, 5], ids=["cuda_core", "tensor_core", "tensor_core_solo"])


def _persistent(package, mode, dev, split_k, **kwargs):
    package.cabi.set_tuning(force_generic=mode)  # whatever the batch size
    try:
        return package.grouped_splitk_decode_attention(*dev, split_k=split_k, **kwargs)
    finally:
        package.cabi.set_tuning()


def _partitioned(package, dev, split_k):
    package.cabi.set_tuning(force_generic=2)
    try:
        return package.grouped_splitk_decode_attention(*dev, split_k=split_k)
    finally:
        package.cabi.set_tuning()


@PERSISTENT
@pytest.mark.parametrize("split_k", [2, 3, 10, 64])
def test_persistent_kernel_mixed_lengths(package, oracle, cuda_device, split_k, mode):
    """Empty, one-token, page-straddling and long sequences in one batch; the table is
    padded with -1 and the tail of every last page is NaN."""
    generator = torch.Generator().manual_seed(split_k)
    lengths = [0, 1, 31, 32, 33, 0, 64, 65, 4000, 16, 17, 0] + \
        torch.randint(1, 1500, (40,), generator=generator).tolist()
    host, dev = _fast_path_inputs(cuda_device, lengths, seed=21, poison=True)
    expected = oracle.paged_attention(*host)
    out = _persistent(package, mode, dev, split_k)
    assert_attention_close(out, expected)
    assert_attention_close(_partitioned(package, dev, split_k), expected)
    assert torch.isfinite(out.float()).all()
    assert (out[[0, 5, 11]] == 0).all()


@PERSISTENT
def test_persistent_kernel_many_short_sequences(package, oracle, cuda_device, mode):
    """Hundreds of sequences of a few pages: every CTA's share holds many pieces, and
    most sequences fit in one."""
    generator = torch.Generator().manual_seed(5)
    lengths = torch.randint(0, 50, (700,), generator=generator).tolist()
    host, dev = _fast_path_inputs(cuda_device, lengths, seed=22)
    assert_attention_close(_persistent(package, mode, dev, 2), oracle.paged_attention(*host))


@PERSISTENT
def test_persistent_kernel_one_long_sequence_few_slots(package, oracle, cuda_device, mode):
    """split_k = 2 with one long sequence: the share is set by the slot limit (no
    sequence may be cut into more than split_k pieces), not by the CTA count."""
    host, dev = _fast_path_inputs(cuda_device, [9000, 40, 3], seed=23)
    expected = oracle.paged_attention(*host)
    for split_k in (2, 3):
        assert_attention_close(_persistent(package, mode, dev, split_k), expected)


@PERSISTENT
def test_persistent_kernel_reuses_partial_buffers(package, oracle, cuda_device, mode):
    """End-of-sequence marks left in the partial buffers by one call must not leak
    into the next call with other lengths (and NaN-filled buffers are harmless)."""
    split_k = 6
    first, dev_first = _fast_path_inputs(cuda_device, [3000, 10, 500, 0], seed=24)
    second, dev_second = _fast_path_inputs(cuda_device, [20, 2500, 0, 700], seed=25)
    partials = (torch.full((4, split_k, 12, 128), float("nan"), device=cuda_device),
                torch.full((4, split_k, 12), float("nan"), device=cuda_device),
                torch.full((4, split_k, 12), float("nan"), device=cuda_device))
    for host, dev in ((first, dev_first), (second, dev_second), (first, dev_first)):
        out = _persistent(package, mode, dev, split_k, partials=partials)
        assert_attention_close(out, oracle.paged_attention(*host))


@PERSISTENT
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_persistent_kernel_dtypes(package, oracle, cuda_device, dtype, mode):
    lengths = [700, 0, 33, 1200, 95]
    host, dev = _fast_path_inputs(cuda_device, lengths, dtype=dtype, seed=26)
    dq, dk, dv, dtable, dlens = dev
    out = _persistent(package, mode, (dq, dk, dv, dtable.long(), dlens.long()), 4)
    assert_attention_close(out, oracle.paged_attention(*host))


@PERSISTENT
def test_persistent_kernel_known_answers(package, cuda_device, mode):
    """Uniform scores: the output is the plain mean of V, exactly."""
    q, k, v, table, lens = make_paged_inputs([0, 1, 17, 1024], poison=True)
    q.zero_()
    v[:, :, 0] = 3
    v[:, :, 1] = 9
    expected = torch.zeros_like(q)
    expected[1:, :6] = 3
    expected[1:, 6:] = 9
    for split_k in (2, 7):
        out = _persistent(package, mode, _to(cuda_device, q, k, v, table, lens), split_k)
        assert torch.equal(out.cpu(), expected)


@PERSISTENT
def test_persistent_kernel_large_scores(package, oracle, cuda_device, mode):
    """Scores that grow along the sequence move the offset many times."""
    q, k, v, table, lens = make_paged_inputs([300, 45, 2000], seed=5)
    ramp = torch.linspace(0.0, 6.0, 16)[None, :, None, None]
    k.mul_(ramp.half())
    host = (q, k, v, table, lens)
    expected = oracle.paged_attention(*host, scale=1.0)
    out = _persistent(package, mode, _to(cuda_device, *host), 3, scale=1.0)
    assert_attention_close(out, expected)


def test_persistent_kernel_batch_above_prefix_capacity(package, oracle, cuda_device):
    """More than 1024 sequences do not fit the persistent kernels' shared-memory
    prefix; the per-partition kernel takes over."""
    generator = torch.Generator().manual_seed(9)
    lengths = torch.randint(0, 40, (1100,), generator=generator).tolist()
    host, dev = _fast_path_inputs(cuda_device, lengths, seed=27)
    out = package.grouped_splitk_decode_attention(*dev, split_k=2)
    assert_attention_close(out, oracle.paged_attention(*host))


@PERSISTENT
def test_persistent_kernel_bad_page_id(package, cuda_device, mode):
    (_, dev) = _fast_path_inputs(cuda_device, [200, 40])
    q, k, v, table, lens = dev
    table = table.clone()
    table[0, 3] = 10_000
    out = _persistent(package, mode, (q, k, v, table, lens), 2)
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    assert package.cabi.device_status() == 2
    assert package.cabi.device_status() == 0


def test_automatic_choice_runs_persistent_kernel_on_a_wide_batch(package, oracle, cuda_device):
    """64 sequences x split_k 10: the default path is the tensor-core kernel's solo variant; it
    must agree with the forced one bit for bit, and it and the interleaving variant with the oracle."""
    generator = torch.Generator().manual_seed(3)
    lengths = torch.randint(1, 900, (64,), generator=generator).tolist()
    host, dev = _fast_path_inputs(cuda_device, lengths, seed=28)
    automatic = package.grouped_splitk_decode_attention(*dev, split_k=10)
    assert torch.equal(automatic, _persistent(package, 5, dev, 10))
    assert_attention_close(automatic, oracle.paged_attention(*host))
    assert_attention_close(_persistent(package, 4, dev, 10), oracle.paged_attention(*host))


@pytest.mark.parametrize("mode", [0, 4], ids=["solo", "interleaving"])
def test_persistent_timeline(package, cuda_device, mode):
    """The instrumented tensor-core pass (the variant every call runs, and the one whose warps
    interleave over the pages): every CTA with work reports entry <= first tile <= exit and its
    share; the shares add up to the batch's pages (plus the interleaving variant's empty units)."""
    generator = torch.Generator().manual_seed(4)
    lengths = torch.randint(1, 900, (64,), generator=generator).tolist()
    (_, dev) = _fast_path_inputs(cuda_device, lengths, seed=29)
    package.cabi.set_tuning(force_generic=mode)
    try:
        timeline = package.native_grouped_persistent_timeline(*dev, split_k=10).cpu()
    finally:
        package.cabi.set_tuning()
    busy = timeline[timeline[:, 5] > 0]
    assert len(busy) >= 2
    for earlier, later in ((0, 1), (1, 2), (2, 3), (3, 4)):
        assert (busy[:, earlier] <= busy[:, later]).all()
    overhead = package.kv_layout.TENSOR_CORE_PIECE_OVERHEAD  # empty units per sequence, as in the kernel
    empty = package.kv_layout.sequence_overhead
    assert busy[:, 5].sum().item() == 2 * sum(-(-n // 16) + empty(-(-n // 16), overhead) for n in lengths)
    schedule = package.kv_layout.persistent_schedule if mode == 4 else package.kv_layout.solo_schedule
    extra = dict(overhead_units=overhead) if mode == 4 else {}
    _, pieces = schedule(lengths, split_k=10, ctas_per_head=len(timeline) // 2, **extra)
    per_cta = torch.bincount(torch.tensor([piece[0] for piece in pieces]), minlength=len(timeline) // 2)
    seen_by_warp0 = busy[:, 6].reshape(2, -1)  # pieces that held pages of warp 0
    # (in the solo variant warp 0's block of a small share may hold empty units only)
    assert (seen_by_warp0 >= (1 if mode == 4 else 0)).all()
    assert (seen_by_warp0 <= per_cta[:seen_by_warp0.shape[1]]).all()
    package.cabi.set_tuning(force_generic=2)  # the per-partition kernel has no timeline
    try:
        with pytest.raises(RuntimeError, match="tensor-core persistent kernel"):
            package.native_grouped_persistent_timeline(*dev, split_k=10)
    finally:
        package.cabi.set_tuning()


def test_stages_and_plan_entry_points(package, oracle, cuda_device):
    """The fused call's two launches run separately give the fused result bit for bit;
    the plan names the kernel the fused call uses."""
    import ctypes

    generator = torch.Generator().manual_seed(6)
    lengths = torch.randint(1, 700, (48,), generator=generator).tolist()
    host, dev = _fast_path_inputs(cuda_device, lengths, seed=31)
    cabi = package.cabi
    splitk = package.kernel_module("paged_decode_grouped_splitk")
    for split_k, mode, kernel in ((8, 0, "decode_mma_kernel (solo)"), (2, 0, "decode_mma_kernel (solo)"),
                                  (8, 4, "decode_mma_kernel"), (8, 5, "decode_mma_kernel (solo)"),
                                  (4, 2, "decode_partial_kernel"), (4, 3, "decode_stream_kernel")):
        cabi.set_tuning(force_generic=mode)
        try:
            fused = package.grouped_splitk_decode_attention(*dev, split_k=split_k)
            partials = (torch.empty(48, split_k, 12, 128, device=cuda_device),
                        torch.empty(48, split_k, 12, device=cuda_device),
                        torch.empty(48, split_k, 12, device=cuda_device))
            out = torch.full_like(dev[0], float("nan"))
            args = splitk.fill_attention_args(cabi, *dev, split_k=split_k, scale=128 ** -0.5,
                                              partials=partials, out=out)
            assert cabi.fused_kernel_plan(args)[0] == kernel
            stream = cabi.stream_pointer(cuda_device)
            lib = cabi.library()
            cabi.check(lib.qf_grouped_splitk_decode_attention_stages(ctypes.byref(args), cabi.STAGE_PARTIAL, stream))
            torch.cuda.synchronize()
            assert torch.isnan(out.float()).all()  # the partial pass alone writes no output
            cabi.check(lib.qf_grouped_splitk_decode_attention_stages(ctypes.byref(args), cabi.STAGE_COMBINE, stream))
        finally:
            cabi.set_tuning()
        assert torch.equal(out, fused)
        assert_attention_close(out, oracle.paged_attention(*host))
        assert lib.qf_grouped_splitk_decode_attention_stages(ctypes.byref(args), 0, stream) == -1


@pytest.mark.parametrize("mode", [0, 1, 2, 3], ids=["default", "generic", "partitioned", "cuda_core_persistent"])
def test_length_beyond_the_table_is_cut_not_followed(package, oracle, cuda_device, mode):
    """A sequence length larger than its block-table row can hold is cut to the row's
    capacity: the kernels never read table entries that do not exist."""
    lengths = [200, 64, 31]
    host, dev = _fast_path_inputs(cuda_device, lengths, seed=35)
    q, k, v, table, lens = dev
    capacity = table.shape[1] * 16
    too_long = lens.clone()
    too_long[1] = capacity + 1000  # row 1 only has 4 real pages; the rest of the row is -1 padding
    package.cabi.set_tuning(force_generic=mode)
    try:
        out = package.grouped_splitk_decode_attention(q, k, v, table, too_long, split_k=3)
    finally:
        package.cabi.set_tuning()
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
    # rows 0 and 2 are untouched by the bad length
    expected = oracle.paged_attention(*host)
    assert_attention_close(out[[0, 2]], expected[[0, 2]])
    # the padded entries of row 1 (-1) are reported as bad page ids, never dereferenced
    assert package.cabi.device_status() == 2


@pytest.mark.parametrize("mode", [2, 4], ids=["per_partition", "tensor_core"])
@pytest.mark.parametrize("split_k", [33, 64, 100, 256])
def test_many_split_slots_take_the_chained_combine(package, oracle, cuda_device, mode, split_k):
    """32 < split_k <= 256 (few long sequences cut into many pieces): the combine that keeps
    up to eight slots per lane, on partials of the per-partition kernel (every slot written,
    many of them empty) and of the persistent kernel (first few slots and an end mark),
    including NaN-filled partial buffers, an empty sequence and a one-token sequence."""
    lengths = [0, 1, 700, 5000, 40, 12000]
    q, k, v, table, lens = make_paged_inputs(lengths, seed=41, value_scale=0.5, poison=True)
    dev = cuda_device
    expected = oracle.paged_attention(q, k, v, table, lens)
    partials = (torch.full((len(lengths), split_k, 12, 128), float("nan"), device=dev),
                torch.full((len(lengths), split_k, 12), float("nan"), device=dev),
                torch.full((len(lengths), split_k, 12), float("nan"), device=dev))
    package.cabi.set_tuning(force_generic=mode)
    try:
        out = package.grouped_splitk_decode_attention(q.to(dev), k.to(dev), v.to(dev), table.to(dev), lens.to(dev),
                                                      split_k=split_k, partials=partials)
    finally:
        package.cabi.set_tuning()
    assert_attention_close(out, expected)
    assert (out[0] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("batch,split_k,longest", [(300, 3, 1024), (600, 2, 1024), (90, 8, 1024), (40, 6, 6000), (7, 2, 3000)])
def test_solo_variant_pieces_and_slots(package, oracle, cuda_device, dtype, batch, split_k, longest):
    """The tensor-core kernel of every call: each warp streams a block of consecutive pages on
    its own and what a CTA's warps hold of one sequence is merged at the CTA's end.  Many short
    sequences (several whole sequences per warp), long ones (a sequence over many warps and
    several CTAs), few slots (the share set by the slot bound, idle CTAs): lengths from 0 tokens
    up, page boundaries on both sides, NaN tails, NaN-filled partial buffers.  The filled slots
    are those of the host restatement of the schedule."""
    generator = torch.Generator().manual_seed(batch + split_k)
    lengths = torch.randint(0, longest + 1, (batch,), generator=generator).tolist()
    lengths[:7] = [0, 1, 15, 16, 17, longest - 1, longest]
    host, dev = _fast_path_inputs(cuda_device, lengths, dtype=dtype, seed=batch, value_scale=0.5, poison=True)
    cabi = package.cabi
    splitk = package.kernel_module("paged_decode_grouped_splitk")
    partials = (torch.full((batch, split_k, 12, 128), float("nan"), device=cuda_device),
                torch.full((batch, split_k, 12), float("nan"), device=cuda_device),
                torch.full((batch, split_k, 12), float("nan"), device=cuda_device))
    args = splitk.fill_attention_args(cabi, *dev, split_k=split_k, scale=128 ** -0.5, partials=partials,
                                      out=torch.empty_like(dev[0]))
    assert cabi.fused_kernel_plan(args)[0] == "decode_mma_kernel (solo)"
    out = package.grouped_splitk_decode_attention(*dev, split_k=split_k, partials=partials)
    assert cabi.device_status() == 0
    expected = oracle.paged_attention(*host)
    assert_attention_close(out, expected, dtype=dtype)
    assert (out[0] == 0).all()
    # slots: those of the host restatement of the schedule, filled from 0 without gaps, then
    # the end mark (sum -1) unless every slot is used
    ctas_per_head = cabi.fused_kernel_plan(args)[1]
    block, pieces = package.kv_layout.solo_schedule(lengths, split_k=split_k, ctas_per_head=ctas_per_head)
    slots = [0] * batch
    for _, sequence, _, _, slot in pieces:
        assert slot == slots[sequence] and slot < split_k
        slots[sequence] += 1
    sums = partials[2][:, :, 0].cpu()
    for row, length in enumerate(lengths):
        assert (sums[row, :slots[row]] > 0).all()
        if length and slots[row] < split_k:
            assert sums[row, slots[row]] == -1
    # the variant whose warps interleave over the pages gives the same attention (other rounding order)
    cabi.set_tuning(force_generic=4)
    try:
        shared = package.grouped_splitk_decode_attention(*dev, split_k=split_k)
    finally:
        cabi.set_tuning()
    assert_attention_close(shared, expected, dtype=dtype)


def test_row_per_warp_combine_equals_row_per_cta_combine(package, cuda_device):
    """Contiguous partials and output take the combine that gives a (sequence, head) row to a
    warp; an output whose rows are 130 elements apart (no 8-byte stores possible) keeps the
    one-CTA-per-row kernel.  Same operations in the same order, so the same bits, on the same
    partials through the combine entry point."""
    torch.manual_seed(9)
    batch, split_k = 171, 6
    po = torch.randn(batch, split_k, 12, 128, device=cuda_device)
    pm = torch.randn(batch, split_k, 12, device=cuda_device) * 3
    ps = torch.rand(batch, split_k, 12, device=cuda_device) + 0.1
    pm[3, 2:] = float("-inf")
    ps[3, 2:] = 0
    ps[5] = 0  # a row without any mass
    po[7, 4:] = float("nan")  # slots without mass may hold anything
    ps[7, 4:] = 0
    splitk = package.kernel_module("paged_decode_grouped_splitk")
    by_warp = splitk.splitk_reduce(po, pm, ps, torch.full((batch, 12, 128), float("nan"), dtype=torch.float16,
                                                          device=cuda_device))
    padded = torch.full((batch, 12, 130), float("nan"), dtype=torch.float16, device=cuda_device)
    by_cta = splitk.splitk_reduce(po, pm, ps, padded[:, :, :128])
    assert torch.isfinite(by_warp.float()).all()
    assert torch.equal(by_warp, by_cta)
    assert torch.isnan(padded[:, :, 128:].float()).all()


def test_misaligned_partial_buffer_keeps_off_the_vector_store_kernel(package, cuda_device):
    """The tensor-core kernel stores partial rows as 16-byte vectors.  A partial buffer that
    starts on a 4-byte boundary (a slice of a larger fp32 arena) must therefore be planned for
    the CUDA-core persistent kernel, whose stores are scalar.  Only the plan is asked: nothing
    is launched on the misaligned buffer."""
    q, k, v, table, lens = (t.to(cuda_device) for t in make_paged_inputs([300, 700], seed=5))
    cabi = package.cabi
    splitk = package.kernel_module("paged_decode_grouped_splitk")
    arena = torch.empty(2 * 8 * 12 * 128 + 4, dtype=torch.float32, device=cuda_device)
    stats = (torch.empty(2, 8, 12, device=cuda_device), torch.empty(2, 8, 12, device=cuda_device))
    out = torch.empty_like(q)
    for offset, kernel in ((0, "decode_mma_kernel (solo)"), (1, "decode_stream_kernel"), (4, "decode_mma_kernel (solo)")):
        partial_out = arena[offset:offset + 2 * 8 * 12 * 128].view(2, 8, 12, 128)
        assert partial_out.data_ptr() % 16 == (4 * offset) % 16
        args = splitk.fill_attention_args(cabi, q, k, v, table, lens, split_k=8, scale=128 ** -0.5,
                                          partials=(partial_out, *stats), out=out)
        assert cabi.fused_kernel_plan(args)[0] == kernel


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_pools_with_different_strides_take_the_cuda_core_persistent_kernel(package, oracle, cuda_device, dtype):
    """K in a contiguous pool, V as a view of a larger allocation (every page followed by an
    unused NaN page): the tensor-core kernel keeps one set of row offsets for both pools, so
    the fused call runs the CUDA-core persistent kernel, its default path; mixed lengths with
    NaN-poisoned tails against the oracle, through the plain public call (no forcing)."""
    generator = torch.Generator().manual_seed(12)
    lengths = [0, 1, 16, 17, 333, 4000] + torch.randint(1, 900, (40,), generator=generator).tolist()
    q, k, v, table, lens = make_paged_inputs(lengths, seed=52, value_scale=0.5, poison=True, dtype=dtype)
    dev = cuda_device
    v_storage = torch.full((v.shape[0], 2, 16, 2, 128), float("nan"), dtype=dtype, device=dev)
    v_storage[:, 0] = v.to(dev)
    v_view = v_storage[:, 0]
    assert v_view.stride(0) == 2 * k.stride(0)
    dq, dk, dtable, dlens = q.to(dev), k.to(dev), table.to(dev), lens.to(dev)
    cabi = package.cabi
    splitk = package.kernel_module("paged_decode_grouped_splitk")
    partials = (torch.empty(len(lengths), 6, 12, 128, device=dev), torch.empty(len(lengths), 6, 12, device=dev),
                torch.empty(len(lengths), 6, 12, device=dev))
    args = splitk.fill_attention_args(cabi, dq, dk, v_view, dtable, dlens, split_k=6, scale=128 ** -0.5,
                                      partials=partials, out=torch.empty_like(dq))
    assert cabi.fused_kernel_plan(args)[0] == "decode_stream_kernel"
    out = package.grouped_splitk_decode_attention(dq, dk, v_view, dtable, dlens, split_k=6)
    assert_attention_close(out, oracle.paged_attention(q, k, v, table, lens))
    assert torch.isnan(v_storage[:, 1].float()).all()
