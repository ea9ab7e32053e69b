"""GPU tests of the QKV projection with the RoPE + paged-cache epilogue (tcgen05 / TMA
kernel) against the unfused path it must equal -- packed_qkv_rope_cache applied to the
model-dtype output of the projection -- and against the CPU oracle."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(device, rows, width=1536, dtype=torch.float16, exact=False, seed=0, pages=24):
    """Inputs of one projection: exact=True draws values whose products and sums are exact
    in fp32 in any order, so every correct kernel returns the same bits."""
    generator = torch.Generator().manual_seed(seed)
    if exact:
        x = torch.randint(-2, 3, (rows, width), generator=generator).float() * 0.5
        weight = torch.randint(-4, 5, (2048, width), generator=generator).float() * 0.25
        bias = torch.randint(-8, 9, (2048,), generator=generator).float() * 0.125
    else:
        x = torch.randn(rows, width, generator=generator) * 0.5
        weight = torch.randn(2048, width, generator=generator) * 0.05
        bias = torch.randn(2048, generator=generator) * 0.1
    positions = torch.randint(0, 32768, (rows,), generator=generator)
    slots = torch.randperm(pages * 16, generator=generator)[:rows]
    to = lambda t: t.to(dtype).to(device)
    return to(x), to(weight), to(bias), positions.to(device), slots.to(device)


def _pools(device, dtype, pages=24):
    make = lambda value: torch.full((pages, 16, 2, 128), value, dtype=dtype, device=device)
    return make(-1.0), make(-2.0)


def _unfused(package, x, weight, bias, positions, slots, k_pool, v_pool, **kwargs):
    packed = torch.nn.functional.linear(x, weight, bias)
    return package.packed_qkv_rope_cache(packed, positions, slots, k_pool, v_pool, **kwargs)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 7, 64, 128, 130, 300])
def test_exact_inputs_equal_the_unfused_path_bit_for_bit(package, oracle, cuda_device, dtype, rows):
    """With sums that are exact in fp32 the accumulation order cannot matter: Q, the K rows
    and the V rows must be identical to projection + packed epilogue, and to the oracle; the
    rest of the (poisoned) pools stays untouched."""
    pages = 24
    x, weight, bias, positions, slots = _case(cuda_device, rows, dtype=dtype, exact=True, seed=rows, pages=pages)
    k_fused, v_fused = _pools(cuda_device, dtype, pages)
    k_plain, v_plain = _pools(cuda_device, dtype, pages)
    q = package.qkv_rope_cache(x, weight, bias, None, positions=positions, slots=slots,
                               k_pool=k_fused, v_pool=v_fused)
    q_plain = _unfused(package, x, weight, bias, positions, slots, k_plain, v_plain)
    assert q.shape == (rows, 12, 128) and torch.equal(q, q_plain)
    assert torch.equal(k_fused, k_plain) and torch.equal(v_fused, v_plain)
    k_cpu, v_cpu = (pool.cpu() for pool in _pools(cuda_device, dtype, pages))
    q_cpu = oracle.qkv_rope_cache(x, weight, bias, positions, slots, k_cpu, v_cpu)
    assert torch.equal(v_fused.cpu(), v_cpu)
    if dtype == torch.float16:
        # same rounded projection; the rotation is within one fp16 unit (taken at the
        # magnitude of its operands) of the oracle's single-rounding fp32 rotation
        packed = oracle.qkv_projection(x, weight, bias).view(rows, 16, 128)
        pairs = lambda heads: torch.maximum(heads[..., :64].abs(), heads[..., 64:].abs()).repeat(1, 1, 2)
        written = slots.cpu()
        assert oracle.ulp_distance_fp16(q.cpu(), q_cpu, pairs(packed[:, :12])).max().item() <= 1.0
        assert oracle.ulp_distance_fp16(k_fused.cpu().view(-1, 2, 128)[written], k_cpu.view(-1, 2, 128)[written],
                                        pairs(packed[:, 12:14])).max().item() <= 1.0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_random_inputs_against_the_oracle(package, oracle, cuda_device, dtype):
    """Random activations and weights: the fp32 accumulation order may flip a rounding tie
    of the projection, which the rotation carries along; V is the projection itself."""
    rows = 96
    x, weight, bias, positions, slots = _case(cuda_device, rows, dtype=dtype, seed=3)
    k_pool, v_pool = _pools(cuda_device, dtype)
    q = package.qkv_rope_cache(x, weight, bias, None, positions=positions, slots=slots,
                               k_pool=k_pool, v_pool=v_pool)
    k_cpu, v_cpu = (pool.cpu() for pool in _pools(cuda_device, dtype))
    q_cpu = oracle.qkv_rope_cache(x, weight, bias, positions, slots, k_cpu, v_cpu)
    packed = oracle.qkv_projection(x, weight, bias).view(rows, 16, 128)
    written = slots.cpu()
    v_rows, k_rows = v_pool.cpu().view(-1, 2, 128)[written], k_pool.cpu().view(-1, 2, 128)[written]
    # The fp32 sum of 1536 products carries an absolute error of a few 1e-6 whatever the
    # size of the result, so units in the last place are taken at a magnitude of at least
    # 1/4 (one fp16 unit there is 2.4e-4): projection within one unit, rotation within three.
    bits = 10 if dtype == torch.float16 else 7
    spacing = lambda reference: torch.exp2(torch.floor(torch.log2(reference.clamp_min(0.25))) - bits)
    error = (v_rows.float() - packed[:, 14:].float()).abs() / spacing(packed[:, 14:].float().abs())
    assert error.max().item() <= 1.0 and (error > 0).float().mean().item() < 2e-2
    magnitude = lambda heads: torch.maximum(heads[..., :64].float().abs(), heads[..., 64:].float().abs()).repeat(1, 1, 2)
    for actual, expected, heads in ((q.cpu(), q_cpu, packed[:, :12]),
                                    (k_rows, k_cpu.view(-1, 2, 128)[written], packed[:, 12:14])):
        error = (actual.float() - expected.float()).abs() / spacing(torch.maximum(magnitude(heads), expected.float().abs()))
        assert error.max().item() <= 3.0
        assert (error > 1.0).float().mean().item() < 5e-3
    # everything that was not written keeps its poison
    untouched = torch.ones(k_pool.shape[0] * 16, dtype=torch.bool)
    untouched[written] = False
    assert bool((k_pool.cpu().view(-1, 2, 128)[untouched] == -1).all())
    assert bool((v_pool.cpu().view(-1, 2, 128)[untouched] == -2).all())
    # no bias, and the unfused GPU path as a second witness (its own accumulation order)
    k2, v2 = _pools(cuda_device, dtype)
    k3, v3 = _pools(cuda_device, dtype)
    q2 = package.qkv_rope_cache(x, weight, None, None, positions=positions, slots=slots, k_pool=k2, v_pool=v2)
    q3 = _unfused(package, x, weight, None, positions, slots, k3, v3)
    tolerance = dict(atol=2e-2, rtol=2e-2)  # the reference's bound for its fused RoPE paths
    torch.testing.assert_close(q2.float(), q3.float(), **tolerance)
    torch.testing.assert_close(k2.float(), k3.float(), **tolerance)
    torch.testing.assert_close(v2.float(), v3.float(), **tolerance)


def test_other_widths_strides_and_metadata_types(package, cuda_device):
    """Input widths of one, four and many 64-wide blocks (fewer blocks than ring stages, and
    several trips round the ring), activations that are a strided view, int32 metadata."""
    for width in (64, 256, 1536, 3072):
        x, weight, bias, positions, slots = _case(cuda_device, 40, width=width, exact=True, seed=width)
        wide = torch.zeros((40, width + 128), dtype=x.dtype, device=cuda_device)
        wide[:, 64:64 + width] = x
        view = wide[:, 64:64 + width]
        k_fused, v_fused = _pools(cuda_device, x.dtype)
        k_plain, v_plain = _pools(cuda_device, x.dtype)
        q = package.qkv_rope_cache(view, weight, bias, None, positions=positions.int(), slots=slots.int(),
                                   k_pool=k_fused, v_pool=v_fused, theta=10_000.0)
        q_plain = _unfused(package, x, weight, bias, positions, slots, k_plain, v_plain, base=10_000.0)
        assert torch.equal(q, q_plain) and torch.equal(k_fused, k_plain) and torch.equal(v_fused, v_plain), width


def test_padded_rows_and_bad_slots(package, cuda_device):
    """Rows at or beyond valid_tokens: zero queries, no cache write (token-bucket graphs).
    A slot outside the pool is skipped and recorded, never written."""
    rows = 70
    x, weight, bias, positions, slots = _case(cuda_device, rows, exact=True, seed=11)
    valid = torch.tensor(45, dtype=torch.int32, device=cuda_device)
    k_fused, v_fused = _pools(cuda_device, x.dtype)
    k_plain, v_plain = _pools(cuda_device, x.dtype)
    q = package.qkv_rope_cache(x, weight, bias, None, positions=positions, slots=slots,
                               k_pool=k_fused, v_pool=v_fused, valid_tokens=valid)
    q_plain = _unfused(package, x, weight, bias, positions, slots, k_plain, v_plain, valid_tokens=valid)
    assert torch.equal(q, q_plain) and bool((q[45:] == 0).all()) and bool((q[:45] != 0).any())
    assert torch.equal(k_fused, k_plain) and torch.equal(v_fused, v_plain)
    dead = slots[45:].cpu()
    assert bool((k_fused.cpu().view(-1, 2, 128)[dead] == -1).all())

    bad = slots.clone()
    bad[3], bad[9] = -1, k_fused.shape[0] * 16
    k_bad, v_bad = _pools(cuda_device, x.dtype)
    q_bad = package.qkv_rope_cache(x, weight, bias, None, positions=positions, slots=bad, k_pool=k_bad, v_pool=v_bad)
    assert package.cabi.device_status() == 2
    k_ref, v_ref = _pools(cuda_device, x.dtype)
    q_ref = package.qkv_rope_cache(x, weight, bias, None, positions=positions, slots=slots, k_pool=k_ref, v_pool=v_ref)
    assert torch.equal(q_bad, q_ref)
    skipped = slots[[3, 9]].cpu()
    assert bool((k_bad.cpu().view(-1, 2, 128)[skipped] == -1).all())
    keep = torch.ones(rows, dtype=torch.bool)
    keep[[3, 9]] = False
    kept = slots.cpu()[keep]
    assert torch.equal(k_bad.cpu().view(-1, 2, 128)[kept], k_ref.cpu().view(-1, 2, 128)[kept])
    assert package.qkv_rope_cache(x[:0], weight, bias, None, positions=positions[:0], slots=slots[:0],
                                  k_pool=k_bad, v_pool=v_bad).shape == (0, 12, 128)


def test_layer_front_in_a_graph(package, oracle, cuda_device):
    """Projection + epilogue feeding the attention of the same layer, captured with chained
    launches and replayed: equal to the eager run with every launch fully ordered."""
    workload = package.workloads.build_workload("decode_b64", batch=24, layers=1)
    step = package.decode_step.DecodeStep(workload, cuda_device, split_k=4, package=package)
    x, weight, bias, _, _ = _case(cuda_device, 24, seed=5)

    def front():
        q = package.qkv_rope_cache(x, weight, bias, None, positions=step.positions, slots=step.slot_mapping,
                                   k_pool=step.k_pools[0], v_pool=step.v_pools[0])
        return package.grouped_splitk_decode_attention(q, step.k_pools[0], step.v_pools[0], step.block_table,
                                                       step.seq_lens, split_k=4, partials=step.partials)

    package.cabi.set_dependent_launch(False)
    try:
        expected = front().clone()
    finally:
        package.cabi.set_dependent_launch(True)
    stream = torch.cuda.Stream(cuda_device)
    stream.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(stream):
        front()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        out = front()
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, expected)


def test_timeline_is_ordered_and_leaves_results_alone(package, cuda_device):
    """The profiling entry returns the same outputs plus per-CTA timestamps in program
    order: entry <= ready <= ... <= TMEM released, for every CTA that exists."""
    for rows, ctas in ((64, 128), (200, 128), (300, 96)):
        x, weight, bias, positions, slots = _case(cuda_device, rows, exact=True, seed=rows)
        k_a, v_a = _pools(cuda_device, x.dtype)
        k_b, v_b = _pools(cuda_device, x.dtype)
        q_a = package.qkv_rope_cache(x, weight, bias, None, positions=positions, slots=slots, k_pool=k_a, v_pool=v_a)
        q_b, timeline = package.qkv_rope_cache_timeline(x, weight, bias, None, positions=positions, slots=slots,
                                                        k_pool=k_b, v_pool=v_b)
        assert torch.equal(q_a, q_b) and torch.equal(k_a, k_b) and torch.equal(v_a, v_b)
        stamps = timeline.cpu()
        live = stamps[stamps[:, 0] > 0]
        assert live.shape[0] == ctas
        order = [0, 1, 3, 4, 5, 7, 8, 9]  # columns every CTA writes, in program order
        for earlier, later in zip(order, order[1:]):
            assert bool((live[:, earlier] <= live[:, later]).all()), (rows, earlier, later)
        assert int((live[:, 9] - live[:, 0]).max()) < 1_000_000  # a kernel of microseconds
