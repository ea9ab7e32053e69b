"""GPU tests of the device-side metadata advance (positions, lengths, slot mapping of a
stable decode cohort) and of consecutive decode steps recorded as one graph with no
host-to-device copy between them."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtypes", [
    (torch.int64, torch.int32, torch.int64, torch.int32),   # the reference engine's buffers
    (torch.int32, torch.int32, torch.int64, torch.int32),   # the graph decoder's
    (torch.int32, torch.int64, torch.int32, torch.int64),
])
def test_advance_follows_the_reference_steps(package, oracle, cuda_device, dtypes):
    """Forty consecutive steps of the reference's build_decode_step_inputs (golden), each
    reproduced from the one before by the kernel, bit for bit; the oracle walks along."""
    data = np.load(GOLDEN_DIR / "metadata_steps.npz")
    positions = torch.from_numpy(data["positions"][0]).to(cuda_device, dtypes[0])
    seq_lens = torch.from_numpy(data["seq_lens"][0]).to(cuda_device, dtypes[1])
    slots = torch.from_numpy(data["slot_mapping"][0]).to(cuda_device, dtypes[2])
    table = torch.from_numpy(data["block_table"]).to(cuda_device, dtypes[3])
    wide = torch.full((table.shape[0], 2 * table.shape[1] + 3), -7, dtype=dtypes[3], device=cuda_device)
    wide[:, 3::2] = table
    strided = wide[:, 3::2]  # a non-contiguous view of the table
    reference = (data["positions"][0], data["seq_lens"][0])
    for step in range(1, data["positions"].shape[0]):
        package.advance_decode_state(positions, seq_lens, slots, strided if step % 2 else table)
        reference = oracle.advance_decode_state(reference[0], reference[1], data["block_table"])
        for actual, key, walked in ((positions, "positions", reference[0]), (seq_lens, "seq_lens", reference[1]),
                                    (slots, "slot_mapping", reference[2])):
            assert np.array_equal(actual.cpu().numpy().astype(np.int64), data[key][step].astype(np.int64)), (key, step)
            assert np.array_equal(walked, data[key][step].astype(np.int64))
    assert positions.dtype == dtypes[0] and slots.dtype == dtypes[2]


def test_advance_other_block_size_and_large_cohort(package, oracle, cuda_device):
    """Block size 4 as in the reference's own test (engine/cpp/tests/test_iteration_loop.py:
    545-551: slots == blocks.gather(positions // 4) * 4 + positions % 4), and a cohort of
    1000 sequences (several CTAs, a ragged last one)."""
    generator = torch.Generator().manual_seed(3)
    for batch, block_size, width in ((3, 4, 5), (1000, 16, 40), (1000, 1, 64)):
        table = torch.randperm(batch * width, generator=generator).reshape(batch, width).to(torch.int32)
        positions = torch.randint(0, width * block_size - 1, (batch,), generator=generator)
        seq_lens = (positions + 1).to(torch.int32)
        dev = [t.to(cuda_device) for t in (positions, seq_lens, torch.zeros(batch, dtype=torch.int64), table)]
        package.advance_decode_state(*dev, block_size=block_size, num_pages=batch * width)
        want = oracle.advance_decode_state(positions.numpy(), seq_lens.numpy(), table.numpy(), block_size)
        for actual, expected in zip(dev[:3], want):
            assert np.array_equal(actual.cpu().numpy().astype(np.int64), expected)
        gathered = dev[3].long().gather(1, (dev[0] // block_size).reshape(-1, 1)).reshape(-1)
        assert torch.equal(dev[2], gathered * block_size + dev[0] % block_size)
    empty = [torch.zeros(0, dtype=dtype, device=cuda_device) for dtype in (torch.int64, torch.int32, torch.int64)]
    package.advance_decode_state(*empty, torch.zeros((0, 4), dtype=torch.int32, device=cuda_device))
    with pytest.raises(ValueError, match="int32 or int64"):
        package.advance_decode_state(dev[0].float(), dev[1], dev[2], dev[3])


def test_advance_beyond_the_table_is_flagged_and_harmless(package, cuda_device):
    """Where the reference's gather would raise, the slot becomes -1 (a row the KV write
    skips) and the status word says why; the other sequences advance normally."""
    positions = torch.tensor([14, 15, 31, 3], dtype=torch.int64, device=cuda_device)
    seq_lens = (positions + 1).to(torch.int32)
    slots = torch.zeros(4, dtype=torch.int64, device=cuda_device)
    table = torch.tensor([[5, 6], [7, 8], [9, 10], [99, 11]], dtype=torch.int32, device=cuda_device)
    package.advance_decode_state(positions, seq_lens, slots, table, num_pages=50)
    assert positions.tolist() == [15, 16, 32, 4] and seq_lens.tolist() == [16, 17, 33, 5]
    assert slots.tolist() == [5 * 16 + 15, 8 * 16, -1, -1]
    assert package.cabi.device_status() in (2, 4)  # both were recorded; the last write stays
    package.advance_decode_state(positions[2:3].clone(), seq_lens[2:3].clone(), slots[2:3].clone(), table[2:3])
    assert package.cabi.device_status() == 4       # position 33 of a two-page table
    package.advance_decode_state(torch.full_like(positions[3:], 15), seq_lens[3:].clone(), slots[3:].clone(),
                                 torch.tensor([[0, -1]], dtype=torch.int32, device=cuda_device), num_pages=50)
    assert package.cabi.device_status() == 2
    # a row with slot -1 leaves the pools untouched
    pool_k = torch.full((4, 16, 2, 128), -1.0, dtype=torch.float16, device=cuda_device)
    pool_v = torch.full((4, 16, 2, 128), -2.0, dtype=torch.float16, device=cuda_device)
    packed = torch.ones((1, 2048), dtype=torch.float16, device=cuda_device)
    package.packed_qkv_rope_cache(packed, positions[2:3], slots[2:3], pool_k, pool_v)
    assert bool((pool_k == -1).all()) and bool((pool_v == -2).all())
    package.cabi.device_status()  # the skipped row is recorded too; leave the word clean


@pytest.mark.parametrize("fp8,fused", [(False, False), (True, False), (False, True)])
def test_unrolled_steps_equal_host_driven_steps(package, cuda_device, fp8, fused):
    """Twenty decode steps (every sequence crosses a page boundary) as ONE graph with the
    metadata advanced on the device, against twenty eager steps whose metadata the host
    builds and copies in, fully ordered launches: same pools, same outputs, same final
    metadata, bit for bit; a replay from restored state repeats it.  Also with the two-launch
    layer step, whose partial pass reads the advanced positions."""
    steps = 20
    name = "fp8_b128" if fp8 else "decode_b64"
    workload = package.workloads.build_workload(name, batch=12, layers=2, reserve_tokens=steps)
    layout = package.kv_layout
    make = lambda fused_write=False: package.decode_step.DecodeStep(
        workload, cuda_device, split_k=4, package=package, fused_write=fused_write)

    host_driven = make()
    host_driven.load_packed_rows()
    package.cabi.set_dependent_launch(False)
    try:
        tables = [row[:-(-(context + 1 + steps) // 16)].tolist()
                  for row, context in zip(workload.block_table, workload.contexts)]
        outputs = []
        for step in range(steps):
            positions, seq_lens, _, slots = layout.decode_step_inputs(
                [context + 1 + step for context in workload.contexts], tables, workload.block_table.shape[1])
            host_driven.positions.copy_(torch.from_numpy(positions))
            host_driven.seq_lens.copy_(torch.from_numpy(seq_lens))
            host_driven.slot_mapping.copy_(torch.from_numpy(slots))
            outputs.append(host_driven.step().clone())
    finally:
        package.cabi.set_dependent_launch(True)

    unrolled = make(fused)  # fused: the RoPE + KV write inside the partial pass, positions advanced on the device
    unrolled.load_packed_rows()
    pristine = [pool.clone() for pool in unrolled.k_pools + unrolled.v_pools]
    unrolled.capture_steps(steps)
    for pool, saved in zip(unrolled.k_pools + unrolled.v_pools, pristine):
        pool.copy_(saved)  # undo the warm-up run's writes
    for replay in range(2):
        unrolled.steps_graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(unrolled.result, outputs[-1]), replay
        live = workload.live_pages.to(cuda_device)
        for a, b in zip(unrolled.k_pools + unrolled.v_pools, host_driven.k_pools + host_driven.v_pools):
            assert torch.equal(a[live], b[live])
        if fp8:
            for a, b in zip(unrolled.k_scales + unrolled.v_scales, host_driven.k_scales + host_driven.v_scales):
                assert torch.equal(a[live], b[live])
        assert unrolled.positions.tolist() == [context + steps for context in workload.contexts]
        assert unrolled.seq_lens.tolist() == [context + 1 + steps for context in workload.contexts]
        unrolled.reset_metadata()
        for pool, saved in zip(unrolled.k_pools + unrolled.v_pools, pristine):
            pool.copy_(saved)
