"""GPU tests of the two-launch layer step (RoPE + KV write folded into the attention partial
pass): it must leave the pools and return the output exactly as the two operators it
replaces do -- packed_qkv_rope_cache, then grouped_splitk_decode_attention."""

from __future__ import annotations

import pytest
import torch

from conftest import assert_attention_close, make_paged_inputs

pytestmark = pytest.mark.gpu


def _inputs(device, lengths, dtype=torch.float16, seed=0, index_dtype=torch.int32):
    """Pools with every page of every sequence filled (the newest token's row poisoned with
    NaN: the step must overwrite it), a permuted block table, packed rows."""
    generator = torch.Generator().manual_seed(seed)
    batch = len(lengths)
    pages_of = [-(-n // 16) for n in lengths]
    total = sum(pages_of) + 3
    order = torch.randperm(total, generator=generator).tolist()
    width = max(pages_of) + 1
    table = torch.zeros((batch, width), dtype=torch.int64)
    cursor = 0
    for b, count in enumerate(pages_of):
        table[b, :count] = torch.tensor(order[cursor:cursor + count])
        cursor += count
    k_pool = (torch.randn((total, 16, 2, 128), generator=generator) * 0.5).to(dtype)
    v_pool = (torch.randn((total, 16, 2, 128), generator=generator) * 0.5).to(dtype)
    slots = torch.zeros(batch, dtype=torch.int64)
    for b, n in enumerate(lengths):
        position = n - 1
        slots[b] = table[b, position // 16] * 16 + position % 16
        k_pool.view(-1, 2, 128)[slots[b]] = float("nan")
        v_pool.view(-1, 2, 128)[slots[b]] = float("nan")
    packed = (torch.randn((batch, 2048), generator=generator) * 0.5).to(dtype)
    lens = torch.tensor(lengths, dtype=torch.int64)
    to = lambda t, kind=None: (t.to(kind) if kind is not None else t).to(device)
    return dict(packed=to(packed), positions=to(lens - 1, index_dtype), slots=to(slots), k_pool=to(k_pool),
                v_pool=to(v_pool), table=to(table, index_dtype), lens=to(lens, index_dtype))


def _pair(package, case, split_k):
    """The two operators.  The attention call and the fused step run the same variant of the
    tensor-core kernel, so their results can be compared bit for bit."""
    k_pool, v_pool = case["k_pool"].clone(), case["v_pool"].clone()
    q = package.packed_qkv_rope_cache(case["packed"], case["positions"], case["slots"], k_pool, v_pool)
    out = package.grouped_splitk_decode_attention(q, k_pool, v_pool, case["table"], case["lens"], split_k=split_k)
    return out, k_pool, v_pool


def _fused(package, case, split_k):
    k_pool, v_pool = case["k_pool"].clone(), case["v_pool"].clone()
    out = package.packed_qkv_rope_attention(case["packed"], case["positions"], case["slots"], k_pool, v_pool,
                                            case["table"], case["lens"], split_k=split_k,
                                            require_fused=split_k > 1)
    return out, k_pool, v_pool


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("lengths,split_k", [
    ([1, 16, 17, 32, 33, 100, 2049, 4000], 8),     # new token first / last in its page, one-token sequences
    ([513] * 8, 4),
    ([700, 9, 31, 1500, 64, 65, 3, 48, 1024, 1025, 250, 16], 6),
    ([9000], 3),                                    # one sequence cut into pieces by the slot limit
    (list(range(1, 130)), 10),                      # many short sequences: several whole sequences per warp
    (list(range(1, 130)), 4),
    ([3000, 100, 2000, 16, 4096] * 16, 32),         # sequences over many warps and several CTAs
])
def test_same_pools_and_output_as_the_two_operators(package, oracle, cuda_device, dtype, lengths, split_k):
    case = _inputs(cuda_device, lengths, dtype=dtype, seed=len(lengths))
    want_out, want_k, want_v = _pair(package, case, split_k)
    got_out, got_k, got_v = _fused(package, case, split_k)
    assert torch.equal(got_k.view(torch.int16), want_k.view(torch.int16))  # bit patterns: no NaN left, none added
    assert torch.equal(got_v.view(torch.int16), want_v.view(torch.int16))
    assert not bool(torch.isnan(got_k.float()).any()) and not bool(torch.isnan(got_v.float()).any())
    assert torch.equal(got_out, want_out)
    if dtype == torch.float16 and len(lengths) <= 12:
        # and both agree with the oracle's step
        k_cpu, v_cpu = case["k_pool"].cpu().clone(), case["v_pool"].cpu().clone()
        q_cpu = oracle.packed_qkv_rope_cache(case["packed"], case["positions"], case["slots"], k_cpu, v_cpu)
        assert_attention_close(got_out, oracle.paged_attention(q_cpu, k_cpu, v_cpu, case["table"], case["lens"]))
        assert torch.equal(got_v.cpu(), v_cpu)


def test_metadata_types_graph_replay_and_fallbacks(package, cuda_device):
    """int64 metadata; captured in a graph and replayed with new rows; split_k 1 and FP8 pools
    run the two operators instead (same call, same results)."""
    lengths = [40, 700, 16, 1, 333, 2048]
    case = _inputs(cuda_device, lengths, seed=5, index_dtype=torch.int64)
    want_out, want_k, want_v = _pair(package, case, 5)
    got_out, got_k, got_v = _fused(package, case, 5)
    assert torch.equal(got_out, want_out) and torch.equal(got_k, want_k) and torch.equal(got_v, want_v)

    k_pool, v_pool = case["k_pool"].clone(), case["v_pool"].clone()
    packed = case["packed"].clone()
    partials = (torch.empty((6, 5, 12, 128), dtype=torch.float32, device=cuda_device),
                torch.empty((6, 5, 12), dtype=torch.float32, device=cuda_device),
                torch.empty((6, 5, 12), dtype=torch.float32, device=cuda_device))
    run = lambda: package.packed_qkv_rope_attention(packed, case["positions"], case["slots"], k_pool, v_pool,
                                                    case["table"], case["lens"], split_k=5, partials=partials)
    stream = torch.cuda.Stream(cuda_device)
    stream.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(stream):
        run()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        out = run()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want_out) and torch.equal(k_pool, want_k)
    other = _inputs(cuda_device, lengths, seed=6, index_dtype=torch.int64)
    packed.copy_(other["packed"])  # new rows, same cache positions
    case2 = dict(case, packed=other["packed"])
    want_out2, want_k2, want_v2 = _pair(package, case2, 5)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, want_out2) and torch.equal(k_pool, want_k2) and torch.equal(v_pool, want_v2)

    # a position outside the table is clamped and recorded, never read out of bounds
    small = package.build_rope_table(64, device=cuda_device)
    package.packed_qkv_rope_attention(case["packed"], case["positions"], case["slots"], case["k_pool"].clone(),
                                      case["v_pool"].clone(), case["table"], case["lens"], split_k=5,
                                      rope_table=small, require_fused=True)
    assert package.cabi.device_status() == 4
    table = package.build_rope_table(4096, base=10_000.0, device=cuda_device)
    positions = torch.arange(4096, dtype=torch.float32)
    inv_freq = torch.tensor([float(f) for f in range(64)], dtype=torch.float32)
    assert table.shape == (4096, 64, 2) and float(table[0, :, 0].min()) == 1.0 and float(table[0, :, 1].abs().max()) == 0.0
    angle = positions[:, None].double() * torch.exp(inv_freq.double() * (-torch.log(torch.tensor(10_000.0)).double() / 64))
    torch.testing.assert_close(table[..., 0].cpu().double(), torch.cos(angle), atol=2e-3, rtol=0)
    del positions, inv_freq, angle
    # a sequence length beyond what its table row can hold: attended up to the table's end as
    # in the plain kernels, its new token (whose slot lies outside the table) is not written
    narrow = dict(case, table=case["table"][:, :3].contiguous())  # 48 tokens per row
    k_cut, v_cut = case["k_pool"].clone(), case["v_pool"].clone()
    package.packed_qkv_rope_attention(narrow["packed"], narrow["positions"], narrow["slots"], k_cut, v_cut,
                                      narrow["table"], narrow["lens"], split_k=5, require_fused=True)
    assert package.cabi.device_status() == 4
    fits = [b for b, n in enumerate(lengths) if n <= 48]
    cut = [b for b, n in enumerate(lengths) if n > 48]
    flat_k, want_flat_k = k_cut.view(-1, 2, 128), want_k.view(-1, 2, 128)
    assert torch.equal(flat_k[case["slots"][fits]], want_flat_k[case["slots"][fits]])
    untouched = torch.ones(flat_k.shape[0], dtype=torch.bool, device=cuda_device)
    untouched[case["slots"][fits]] = False
    assert torch.equal(flat_k[untouched].view(torch.int16), case["k_pool"].view(-1, 2, 128)[untouched].view(torch.int16))
    assert len(cut) == 3
    single_out, single_k, _ = _fused(package, case, 1)
    want_single, want_single_k, _ = _pair(package, case, 1)
    assert torch.equal(single_out, want_single) and torch.equal(single_k, want_single_k)
    with pytest.raises(RuntimeError, match="does not apply"):
        package.packed_qkv_rope_attention(case["packed"], case["positions"], case["slots"], k_pool, v_pool,
                                          case["table"], case["lens"], split_k=1, require_fused=True)
    with pytest.raises(ValueError, match="2048"):
        package.packed_qkv_rope_attention(case["packed"][:, :1024], case["positions"], case["slots"], k_pool, v_pool,
                                          case["table"], case["lens"], split_k=5)


def test_decode_step_with_the_fused_write(package, cuda_device):
    """DecodeStep over two layers, eager and captured: fused and unfused steps leave the same
    pools and return the same result; one launch fewer per layer."""
    workload = package.workloads.build_workload("decode_b64", batch=24, layers=2)
    plain = package.decode_step.DecodeStep(workload, cuda_device, split_k=6, package=package)
    fused = package.decode_step.DecodeStep(workload, cuda_device, split_k=6, package=package, fused_write=True)
    assert fused.kernel_launches_per_step == 4 and plain.kernel_launches_per_step == 6
    plain.load_packed_rows(), fused.load_packed_rows()
    want = plain.step().clone()
    got = fused.step().clone()
    assert torch.equal(got, want)
    for a, b in zip(fused.k_pools + fused.v_pools, plain.k_pools + plain.v_pools):
        live = workload.live_pages.to(cuda_device)
        assert torch.equal(a[live], b[live])
    fused.capture()
    assert torch.equal(fused.replay(), want)


def test_slot_check_refuses_rows_the_fused_kernel_would_place_elsewhere(package, cuda_device):
    """The fused kernel never reads the slot mapping (it writes at the block table's slot), so
    a batch with a skipped row (slot -1) belongs to the operator pair; `check_slots=True`
    says so before anything is launched, and passes the engine's own mapping."""
    lengths = [40, 17, 300]
    q, k, v, table, lens = (t.to(cuda_device) for t in make_paged_inputs(lengths, seed=9, value_scale=0.5))
    packed = torch.randn(3, 2048, device=cuda_device).mul_(0.5).half()
    positions = (lens - 1).to(torch.int32)
    rows = torch.arange(3, device=cuda_device)
    slots = table[rows, ((lens - 1) // 16).long()].long() * 16 + ((lens - 1) % 16).long()
    out = package.packed_qkv_rope_attention(packed, positions, slots, k.clone(), v.clone(), table, lens,
                                            split_k=4, require_fused=True, check_slots=True)
    assert out.shape == (3, 12, 128)
    skipped = slots.clone()
    skipped[1] = -1
    k_before = k.clone()
    with pytest.raises(ValueError, match="slot_mapping differs"):
        package.packed_qkv_rope_attention(packed, positions, skipped, k, v, table, lens,
                                          split_k=4, require_fused=True, check_slots=True)
    assert torch.equal(k, k_before)  # refused before any launch


def test_fused_step_on_the_interleaving_variant(package, oracle, cuda_device):
    """qf_set_tuning mode 4 keeps the variant of the tensor-core kernel whose warps interleave
    over the pages (the instrumented one): fused step and operator pair agree bit for bit there
    too, and with the default variant within the attention tolerance."""
    lengths = [700, 9, 31, 1500, 64, 65, 3, 48, 1024, 1025, 250, 16] * 3
    case = _inputs(cuda_device, lengths, dtype=torch.float16, seed=11)
    default_out, default_k, default_v = _fused(package, case, 6)
    package.cabi.set_tuning(force_generic=4)
    try:
        want_out, want_k, want_v = _pair(package, case, 6)
        got_out, got_k, got_v = _fused(package, case, 6)
    finally:
        package.cabi.set_tuning()
    assert torch.equal(got_out, want_out)
    assert torch.equal(got_k.view(torch.int16), want_k.view(torch.int16))
    assert torch.equal(got_v.view(torch.int16), want_v.view(torch.int16))
    assert torch.equal(got_k.view(torch.int16), default_k.view(torch.int16))
    assert_attention_close(got_out, default_out)
