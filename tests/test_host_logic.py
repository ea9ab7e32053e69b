"""CPU tests of everything around the kernels: the C ABI loads and exports what the
header declares, the ctypes structs match the C layout, wrapper validation fires
before any device work, and the host-side integer logic (allocator, metadata,
split policy, sharding, workloads) reproduces the reference's."""

from __future__ import annotations

import ctypes
import re
import shutil
import subprocess
from unittest import mock

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR, REPO_ROOT


# ------------------------------------------------------------------- C ABI

def test_library_exports_every_declared_symbol(package):
    header = (REPO_ROOT / "include" / "qf_hotpath.h").read_text()
    declared = set(re.findall(r"^(?:int|const char\*)\s+(qf_\w+)\s*\(", header, flags=re.M))
    assert declared == set(package.cabi.EXPORTED_SYMBOLS)
    lib = package.cabi.library()
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.qf_abi_version() == package.cabi.ABI_VERSION == 1


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_ctypes_structs_match_c_layout(package, tmp_path):
    fields = {"qf_rope_kv_write_args": package.cabi.RopeKvWriteArgs,
              "qf_decode_attention_args": package.cabi.DecodeAttentionArgs,
              "qf_qkv_rope_cache_args": package.cabi.QkvRopeCacheArgs}
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "qf_hotpath.h"', "int main(void) {"]
    for struct, cls in fields.items():
        lines.append(f'printf("{struct} %zu\\n", sizeof({struct}));')
        for name, _ in cls._fields_:
            lines.append(f'printf("{struct}.{name} %zu\\n", offsetof({struct}, {name}));')
    lines.append("return 0; }")
    source = tmp_path / "layout.c"
    source.write_text("\n".join(lines))
    binary = tmp_path / "layout"
    subprocess.run(["gcc", "-I", str(REPO_ROOT / "include"), str(source), "-o", str(binary)], check=True)
    reported = dict(line.split() for line in subprocess.run(
        [str(binary)], check=True, capture_output=True, text=True).stdout.splitlines())
    for struct, cls in fields.items():
        assert int(reported[struct]) == ctypes.sizeof(cls)
        for name, _ in cls._fields_:
            assert int(reported[f"{struct}.{name}"]) == getattr(cls, name).offset, (struct, name)


def test_c_side_validation_without_a_gpu(package):
    """Argument errors come back as a negative status and a message; nothing is launched."""
    cabi = package.cabi
    lib = cabi.library()
    args = cabi.DecodeAttentionArgs()
    args.batch, args.q_heads, args.kv_heads, args.head_dim, args.page_size = 2, 12, 5, 128, 16
    args.split_k = 1
    assert lib.qf_grouped_splitk_decode_attention(ctypes.byref(args), None) == -1
    assert b"divisible" in lib.qf_last_error()
    args.kv_heads, args.split_k = 2, 0
    assert lib.qf_grouped_gqa_splitk_partial_out(ctypes.byref(args), None) == -1
    assert b"split_k" in lib.qf_last_error()
    rope = cabi.RopeKvWriteArgs()
    rope.rows, rope.q_heads, rope.kv_heads, rope.head_dim, rope.dtype = 1, 12, 2, 100, 0
    assert lib.qf_rope_kv_write(ctypes.byref(rope), None) == -1
    assert b"head dimension" in lib.qf_last_error()
    with pytest.raises(RuntimeError, match="libqf_hotpath"):
        cabi.check(-1)
    assert lib.qf_set_tuning(99, 0) == -1
    assert lib.qf_set_tuning(0, 0) == 0
    advance = lambda *dtypes, batch=1, page=16: lib.qf_advance_decode_metadata(
        None, dtypes[0], None, dtypes[1], None, dtypes[2], None, dtypes[3], 1, 1, 1, 1, batch, page, None)
    assert advance(1, 0, 1, 0, batch=0) == 0            # an empty cohort is a no-op, nothing launched
    assert advance(2, 0, 1, 0) == -1 and b"integer dtype" in lib.qf_last_error()
    assert advance(1, 0, 1, 0, page=0) == -1 and b"page size" in lib.qf_last_error()
    assert advance(1, 0, 1, 0) == -1 and b"must not be null" in lib.qf_last_error()
    assert lib.qf_rms_norm(None, 8, None, None, 8, 0, 8, 0, 1e-6, None) == 0   # no rows: nothing launched
    assert lib.qf_rms_norm(None, 8, None, None, 8, 4, 8, 7, 1e-6, None) == -1 and b"fp16 or bf16" in lib.qf_last_error()
    assert lib.qf_rms_norm(None, 8, None, None, 8, 4, 0, 0, 1e-6, None) == -1 and b"hidden" in lib.qf_last_error()
    assert lib.qf_residual_add_rms_norm(None, 8, None, 8, None, None, 8, None, 8, 4, 8, 1, 1e-6, None) == -1
    assert b"must not be null" in lib.qf_last_error()
    assert lib.qf_build_rope_table(None, 0, 1e6, None) == 0          # no positions: nothing launched
    assert lib.qf_build_rope_table(None, 8, 1e6, None) == -1 and b"aligned" in lib.qf_last_error()
    step_args = cabi.DecodeAttentionArgs()
    step_args.batch, step_args.q_heads, step_args.kv_heads, step_args.head_dim, step_args.page_size = 2, 12, 2, 128, 16
    step_args.split_k = 4
    assert lib.qf_packed_rope_decode_attention(ctypes.byref(step_args), None, 0, 1, None, 0, 3, None) == -1
    assert lib.qf_packed_rope_decode_attention(ctypes.byref(step_args), None, 0, 1, None, 0, 9, None) == -1
    assert b"stages" in lib.qf_last_error()
    gemm = cabi.QkvRopeCacheArgs()
    gemm.rows, gemm.in_features, gemm.dtype = 4, 1500, 0
    assert lib.qf_qkv_rope_cache(ctypes.byref(gemm), None) == -1 and b"multiple of 64" in lib.qf_last_error()
    gemm.in_features, gemm.rows = 1536, 0
    assert lib.qf_qkv_rope_cache(ctypes.byref(gemm), None) == 0   # no rows: nothing launched
    gemm.rows = 4
    assert lib.qf_qkv_rope_cache(ctypes.byref(gemm), None) == -1 and b"must not be null" in lib.qf_last_error()


def test_missing_library_fails_loudly_with_one_build_command(package):
    cabi = package.cabi
    native = package.kernel_module("paged_decode_native_grouped")
    with mock.patch.object(cabi, "_library", None), \
            mock.patch.object(cabi, "LIBRARY_PATH", REPO_ROOT / "does-not-exist.so"):
        with pytest.raises(RuntimeError, match=r"python qwen-frence_b200/build\.py"):
            cabi.library()
        with pytest.raises(RuntimeError, match=r"not built; run: python qwen-frence_b200/build\.py"):
            native._extension()


def test_product_never_touches_the_oracle():
    """No file of the package imports, opens or names the oracle."""
    for path in (REPO_ROOT / "qwen-frence_b200").rglob("*"):
        if path.suffix in (".py", ".cu", ".cuh", ".h") and "build" not in path.parts[-2:-1]:
            assert "oracle" not in path.read_text().lower(), path


# ------------------------------------------------- wrapper contracts (fakes)

class FakeTensor:
    """Shape/ndim/dtype only, like the reference's CPU contract tests
    (experiments/tests/test_native_grouped_decode.py:18-24)."""

    def __init__(self, shape, *, dtype="fp16", device="cuda"):
        self.shape = tuple(shape)
        self.ndim = len(shape)
        self.dtype = dtype
        self.device = device


def _fake_inputs(group=6, head_dim=128, page_size=16):
    return (FakeTensor((8, 2 * group, head_dim)), FakeTensor((2048, page_size, 2, head_dim)),
            FakeTensor((2048, page_size, 2, head_dim)), FakeTensor((8, 256), dtype="int32"),
            FakeTensor((8,), dtype="int32"))


def test_native_wrapper_rejects_unsupported_layouts(package):
    """experiments/tests/test_native_grouped_decode.py:43-60."""
    fn = package.native_grouped_splitk_decode_attention
    with pytest.raises(ValueError, match="six query heads"):
        fn(*_fake_inputs(group=4), split_k=8)
    with pytest.raises(ValueError, match="head_dim=128"):
        fn(*_fake_inputs(head_dim=64), split_k=8)
    with pytest.raises(ValueError, match="head_dim=128"):
        fn(*_fake_inputs(page_size=32), split_k=8)
    with pytest.raises(ValueError, match="split_k >= 2"):
        fn(*_fake_inputs(), split_k=1)
    with pytest.raises(ValueError, match="split_k >= 2"):
        fn(*_fake_inputs(), split_k=2.0)


def test_cpu_tensors_are_rejected_not_computed(package):
    """There is no CPU path: CPU tensors are a ValueError, never a fallback."""
    q = torch.zeros(2, 12, 128, dtype=torch.float16)
    pool = torch.zeros(4, 16, 2, 128, dtype=torch.float16)
    table = torch.zeros(2, 2, dtype=torch.int32)
    lens = torch.ones(2, dtype=torch.int32)
    with pytest.raises(ValueError, match="CUDA device"):
        package.grouped_splitk_decode_attention(q, pool, pool, table, lens, split_k=1)
    with pytest.raises(ValueError, match="share a device"):
        package.native_grouped_splitk_decode_attention(q, pool, pool, table, lens, split_k=2)
    with pytest.raises(ValueError, match="CUDA"):
        package.packed_qkv_rope_cache(torch.zeros(2, 2048, dtype=torch.float16), lens, lens, pool, pool)
    with pytest.raises(ValueError, match="CUDA"):
        package.advance_decode_state(lens.long(), lens, lens.long(), table)
    hidden = torch.zeros(2, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="CUDA"):
        package.rms_norm(hidden, hidden[0])
    with pytest.raises(ValueError, match="CUDA"):
        package.residual_add_rms_norm(hidden, hidden, hidden[0])
    with pytest.raises(ValueError, match="CUDA"):
        package.qkv_rope_cache(torch.zeros(2, 1536, dtype=torch.float16), torch.zeros(2048, 1536, dtype=torch.float16),
                               None, None, positions=lens.long(), slots=lens.long(), k_pool=pool, v_pool=pool)
    with pytest.raises(ValueError, match="norm folding"):
        package.qkv_rope_cache(torch.zeros(2, 1536, dtype=torch.float16), torch.zeros(2048, 1536, dtype=torch.float16),
                               None, torch.zeros(2), positions=lens.long(), slots=lens.long(), k_pool=pool, v_pool=pool)
    with pytest.raises(ValueError, match="one entry per sequence"):
        package.advance_decode_state(lens.long(), lens[:1], lens.long(), table)
    with pytest.raises(ValueError, match="CUDA"):
        package.rope_kv_write(q[None].transpose(1, 2)[:, :, :, :], pool[:1, :2].transpose(1, 2)[:, :, :2],
                              pool[:1, :2].transpose(1, 2)[:, :, :2], lens, lens, pool, pool)


# ------------------------------------------------------ allocator + metadata

def test_page_pool_replays_reference_allocator(package):
    """Golden: the reference PagedKVCache driven through allocate / free / truncate."""
    data = np.load(GOLDEN_DIR / "metadata_case.npz")
    pool = package.kv_layout.PagePool(4, 64)
    pool.allocate([5, 16, 17, 1])
    pool.allocate([1, 1, 0, 40])
    pool.free(1)
    pool.allocate([0, 33, 1, 0])
    pool.truncate(3, 20)
    pool.allocate([1, 1, 1, 1])
    assert pool.cur_lens == data["cur_lens"].tolist()
    assert pool.free_pages == data["free_blocks"].tolist()
    tables = [[int(p) for p in row if p >= 0] for row in data["tables"]]
    assert pool.block_tables == tables
    positions, seq_lens, table, slots = package.kv_layout.decode_step_inputs(
        pool.cur_lens, pool.block_tables, int(data["max_blocks"]))
    for actual, key in ((positions, "positions"), (seq_lens, "seq_lens"), (table, "block_table"),
                        (slots, "slot_mapping")):
        assert actual.dtype == data[key].dtype and np.array_equal(actual, data[key]), key


def test_page_pool_is_atomic_on_exhaustion(package):
    layout = package.kv_layout
    pool = layout.PagePool(2, 3)
    pool.allocate([16, 16])
    before = (list(pool.free_pages), [list(t) for t in pool.block_tables], list(pool.cur_lens))
    with pytest.raises(layout.CacheFullError):
        pool.allocate([1, 17])  # needs 1 + 2 pages, 1 free
    assert (pool.free_pages, pool.block_tables, pool.cur_lens) == before
    with pytest.raises(ValueError, match="max_seq_len"):
        layout.PagePool(1, 4, max_seq_len=32).allocate([33])
    with pytest.raises(ValueError, match="cannot truncate"):
        pool.truncate(0, 17)
    pool.reset()
    assert pool.free_pages == [0, 1, 2] and pool.cur_lens == [0, 0]


def test_split_policy_matches_reference_table(package):
    data = np.load(GOLDEN_DIR / "splitk_policy.npz")
    for context, split_k, stages in zip(data["contexts"], data["split_k"], data["num_stages"]):
        config = package.kv_layout.select_splitk_config(int(context))
        assert (config["split_k"], config["num_stages"]) == (int(split_k), int(stages))
        assert config["heads_per_program"] == 1 and config["num_warps"] == 4
    with pytest.raises(ValueError):
        package.kv_layout.select_splitk_config(0)


def test_plan_split_k_uses_host_bounds_only(package):
    plan = package.kv_layout.plan_split_k
    assert plan(256, 8193) == 3          # enough (sequence, head) pairs already
    assert plan(64, 4097) == 10
    assert plan(4, 32769) == 148         # long, tiny batch: fill the machine
    assert plan(1, 64) == 1              # never shorter than 8 pages per split
    assert plan(8, 513) == 4
    # many short sequences stay on the persistent kernel (which needs split_k >= 2) ...
    assert plan(512, 101) == 3 and plan(256, 1024) == 3 and plan(1024, 61) == 3
    # ... smaller batches and wider tables keep the old plan
    assert plan(255, 101) == 1 and plan(64, 201) == 1 and plan(256, 1025) == 3
    for batch, context in ((1, 1), (3, 100000), (1024, 16)):
        assert 1 <= plan(batch, context) <= 65535


def test_algorithmic_bytes(package):
    layout = package.kv_layout
    assert layout.kv_bytes_per_layer([4096] * 64) == 64 * 2 * 4096 * 128 * 2 * 2  # reference's unique_bytes
    one = layout.algorithmic_bytes_per_layer([17], split_k=1)
    assert one == 17 * 1024 + 2 * 4 + 2 * 3072 + (4096 + 3072 + 1024 + 12)
    assert layout.algorithmic_bytes_per_layer([17], split_k=2) - one == 2 * 2 * 12 * 130 * 4
    assert layout.algorithmic_bytes_per_layer([32], split_k=1, fp8=True) == \
        32 * 512 + 2 * 4 + 2 * 16 + 2 * 3072 + (4096 + 3072 + 512 + 12)


# ----------------------------------------------------------------- workloads

def test_workloads_have_the_configured_shapes(package):
    build = package.workloads.build_workload
    w = build("cpu_single_layer_b8")
    assert (w.layers, w.batch, w.num_pages, w.block_table.shape) == (1, 8, 512, (8, 33))
    assert w.seq_lens.tolist() == [513] * 8 and w.positions.tolist() == [512] * 8
    pages = w.block_table.flatten().tolist()
    assert len(set(pages)) == len(pages) and pages != sorted(pages)  # permuted, disjoint
    rows = torch.arange(8)
    expected_slots = w.block_table[rows, 32].long() * 16 + 0
    assert torch.equal(w.slot_mapping, expected_slots)

    w = build("decode_b64")
    assert w.layers == 28 and w.batch == 64
    assert 128 <= min(w.contexts) and max(w.contexts) <= 4096
    w2 = build("decode_b64")
    assert w2.contexts == w.contexts and torch.equal(w2.block_table, w.block_table)  # seeded
    other = build("decode_b64", rank=1, world_size=2)  # weak: the same lengths (equal cost), its own pages and values
    assert other.contexts == w.contexts and not torch.equal(other.block_table, w.block_table)
    assert other.value_seed != w.value_seed

    # pages reserved at admission for the tokens of coming steps: same first step,
    # wider tables that the device-side advance can walk
    plain, reserved = build("decode_b64", batch=8, layers=1), build("decode_b64", batch=8, layers=1, reserve_tokens=40)
    assert torch.equal(reserved.positions, plain.positions) and torch.equal(reserved.seq_lens, plain.seq_lens)
    for b, context in enumerate(reserved.contexts):
        pages = reserved.block_table[b, :-(-(context + 1 + 40) // 16)].tolist()
        assert len(set(pages)) == len(pages) and all(0 <= page < reserved.num_pages for page in pages)
    assert reserved.live_pages.numel() > plain.live_pages.numel()

    w = build("long_skew_b4")
    assert sorted(w.contexts) == [512, 4096, 16384, 32768] and w.block_table.shape[1] == 2049
    w = build("fp8_b128", layers=2)
    assert w.fp8 and w.batch == 128 and set(w.contexts) == {2048}


def test_strong_scaling_shards_cover_the_batch_once(package):
    build = package.workloads.build_workload
    everyone = package.workloads.context_lengths("sweep_b256")
    assert len(everyone) == 256 and 64 <= min(everyone) and max(everyone) <= 8192
    seen = []
    loads = []
    for rank in range(8):
        w = build("sweep_b256", rank=rank, world_size=8, scaling="strong", layers=1)
        assert w.num_pages == 131072 // 8
        assert [everyone[i] for i in w.global_indices] == w.contexts
        used = int((w.block_table > 0).sum()) + 1
        assert used <= w.num_pages and w.meta["filler_pages"] > 0
        seen += w.global_indices
        loads.append(sum(w.contexts))
    assert sorted(seen) == list(range(256))
    assert max(loads) / (sum(loads) / 8) < 1.02  # snake dealing balances the ranks


def test_partition_policies(package):
    sharding = package.sharding
    lengths = [100, 5, 80, 7, 60, 9, 40, 11]
    snake = sharding.partition_sequences(lengths, 2)
    assert sorted(snake[0] + snake[1]) == list(range(8))
    assert snake[0] == [0, 1, 6, 7] and snake[1] == [2, 3, 4, 5]  # dealt by length, kept in batch order
    assert sharding.imbalance(lengths, snake) < sharding.imbalance(
        lengths, sharding.partition_sequences(lengths, 2, "block")) + 1e-9
    block = sharding.partition_sequences(lengths, 3, "block")
    assert block == [[0, 1, 2], [3, 4, 5], [6, 7]]
    assert sharding.partition_sequences([], 4) == [[], [], [], []]
    assert sharding.shard_pages([17, 16, 1], [[0, 1], [2]]) == [3, 1]
    with pytest.raises(ValueError):
        sharding.partition_sequences(lengths, 0)


def test_persistent_schedule_respects_split_slots(package):
    """The share rule of the persistent kernels: pieces tile every sequence exactly,
    CTAs get at most `share` units, and no sequence needs more than split_k slots."""
    import random

    schedule = package.kv_layout.persistent_schedule
    rng = random.Random(7)
    for trial in range(200):
        batch = rng.choice([1, 2, 5, 64, 300])
        lengths = [rng.choice([0, 1, 15, 16, 17, 500, rng.randint(0, 9000)]) for _ in range(batch)]
        split_k = rng.choice([2, 3, 10, 64])
        ctas = rng.choice([1, 7, 74, 148])
        unit = rng.choice([16, 32])
        overhead = rng.choice([0, 0, 6])
        share, pieces = schedule(lengths, split_k=split_k, ctas_per_head=ctas, unit_tokens=unit,
                                 overhead_units=overhead)
        units = [-(-t // unit) for t in lengths]
        covered = [0] * batch
        load = {}
        for cta, sequence, first, count, slot in pieces:
            assert count >= 1 and first == covered[sequence] and 0 <= slot < split_k
            assert 0 <= cta < ctas
            covered[sequence] += count
            load[cta] = load.get(cta, 0) + count
        assert covered == units
        assert all(v <= share for v in load.values())
        slots = {}
        for cta, sequence, first, count, slot in pieces:
            slots.setdefault(sequence, []).append(slot)
        assert all(s == list(range(len(s))) for s in slots.values())
    with pytest.raises(ValueError):
        schedule([5], split_k=1, ctas_per_head=4)


def test_solo_schedule_covers_every_page_once_within_the_slots(package):
    """Host restatement of the solo variant's cut: every page of every sequence in exactly one
    piece, in order, slots counted from 0 per sequence without gaps and below split_k -- also
    when the slot limit, not the unit count, sets the share."""
    import random

    kv_layout = package.kv_layout
    random.seed(3)
    for split_k, ctas, lengths in (
            (3, 74, [random.randint(0, 1024) for _ in range(300)]),
            (2, 74, [100] * 600),
            (2, 74, [2000] + [40] * 30 + [0, 700]),
            (8, 148, [1] * 90),
            (4, 74, [0, 0, 0])):
        share, pieces = kv_layout.solo_schedule(lengths, split_k=split_k, ctas_per_head=ctas)
        pages = [-(-n // 16) for n in lengths]
        if sum(pages) == 0:
            assert pieces == []
            continue
        units = [n + kv_layout.sequence_overhead(n, kv_layout.TENSOR_CORE_PIECE_OVERHEAD) for n in pages]
        assert share * ctas >= sum(units) and share * (split_k - 1) >= max(units)
        seen = [0] * len(lengths)
        next_slot = [0] * len(lengths)
        last_cta = -1
        for cta, sequence, first, count, slot in pieces:
            assert count >= 1 and first == seen[sequence] and cta >= last_cta
            last_cta = cta
            seen[sequence] += count
            assert slot == next_slot[sequence] < split_k
            next_slot[sequence] += 1
        assert seen == pages
