"""Pins the CPU oracle (oracle/) against outputs of the reference's own Python
functions (tests/golden/*.npz) and against the reference's known-answer tests.
CPU only."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import (GOLDEN_DIR, assert_attention_close, attention_case_tensors, make_paged_inputs,
                      tensor_from_bits)


# ---------------------------------------------------------------- attention

def test_oracle_attention_matches_reference_outputs(oracle, attention_golden):
    """Golden: attention_reference (experiments/decode/grouped_splitk_validation.py:43-60)
    on ragged, strided, NaN-poisoned, boundary and adversarial cases."""
    assert len(attention_golden.names) >= 17
    for name in attention_golden.names:
        q, k, v, table, lens, scale, expected = attention_case_tensors(attention_golden.case(name))
        actual = oracle.paged_attention(q, k, v, table, lens, scale=scale)
        assert_attention_close(actual, expected)
        assert torch.isfinite(actual.float()).all(), name


def test_oracle_attention_matches_engine_oracles(oracle, attention_golden):
    """Golden: decode_attention_reference / decode_attention_sdpa
    (engine/kvcache/paged_decode_attention.py:268-314)."""
    checked = 0
    for name in attention_golden.names:
        fields = attention_golden.case(name)
        if "expected_engine_sdpa" not in fields:
            continue
        q, k, v, table, lens, scale, _ = attention_case_tensors(fields)
        actual = oracle.paged_attention(q, k, v, table.clamp_min(0), lens, scale=scale)
        for key in ("expected_engine_reference", "expected_engine_sdpa"):
            assert_attention_close(actual, tensor_from_bits(fields[key], str(fields["dtype"])))
        checked += 1
    assert checked >= 6


@pytest.mark.parametrize("split_k", [1, 2, 7, 22])
def test_oracle_splitk_equals_dense(oracle, attention_golden, split_k):
    """Partial + combine restatement agrees with the dense oracle, including
    split_k > pages (empty partitions) and NaN-poisoned tails."""
    for name in ("ragged_strided_matrix_float16", "negative_scores_empty_splits_float16",
                 "unnormalized_overflow_float16", "boundary_page32_31_32_33_129"):
        q, k, v, table, lens, scale, expected = attention_case_tensors(attention_golden.case(name))
        actual = oracle.splitk_attention(q, k, v, table, lens, split_k=split_k, scale=scale)
        assert_attention_close(actual, expected)


def test_reference_known_answers(oracle):
    """experiments/tests/test_grouped_splitk_pipelined.py:40-66 restated."""
    q, k, v, table, lens = make_paged_inputs([0, 1, 17], poison=True)
    q.zero_()
    v[:, :, 0] = 3
    v[:, :, 1] = 9
    expected = torch.zeros_like(q)
    expected[1:, :6] = 3
    expected[1:, 6:] = 9
    assert torch.equal(oracle.paged_attention(q, k, v, table, lens), expected)

    q, k, v, table, lens = make_paged_inputs([0, 1, 17])
    q.fill_(1), k.fill_(-1), v.fill_(1)
    out = oracle.splitk_attention(q, k, v, table, lens, split_k=7, scale=1.0)
    assert torch.equal(out[0], torch.zeros_like(out[0])) and torch.equal(out[1:], torch.ones_like(out[1:]))

    q, k, v, table, lens = make_paged_inputs([1024])
    q.zero_(), k.zero_(), v.fill_(128)
    po, pm, ps = oracle.splitk_partial(q, k, v, table, lens, split_k=2)
    assert po.max().item() > 65504  # un-normalised partials exceed the fp16 range
    assert torch.equal(oracle.splitk_reduce(po, pm, ps), torch.full_like(q, 128))


def test_all_empty_batch_and_zero_width_table(oracle):
    q, k, v, table, lens = make_paged_inputs([0, 0])
    out = oracle.paged_attention(q, k, v, table[:, :0], lens)
    assert torch.equal(out, torch.zeros_like(q))


# --------------------------------------------------------------------- rope

def test_oracle_rope_matches_reference_fp32_path(oracle, rope_golden):
    """Golden: rope_reference (custom_kernels/rope.py:104-129), fp32 single rounding.
    Its inv_freq is theta**(-i/half) instead of the kernels' exp(i * -ln(theta)/half);
    one fp32 ulp of inv_freq times the position moves the angle, so the bound widens
    with position: exact-to-1-ulp at small positions, a few ulp by 32k."""
    for name, bound in (("pos0", 0.0), ("small", 1.0), ("check_custom_kernels", 2.0), ("large", 8.0)):
        fields = rope_golden.case(name)
        x = tensor_from_bits(fields["x"])
        expected = tensor_from_bits(fields["expected_fp32_path"])
        actual = oracle.rope(x, torch.from_numpy(fields["positions"]))
        partner = torch.cat((x[..., 64:], x[..., :64]), dim=-1)
        magnitude = torch.maximum(x.float().abs(), partner.float().abs())
        ulp = oracle.ulp_distance_fp16(actual, expected, magnitude)
        assert ulp.max().item() <= bound, (name, ulp.max().item())
        if name == "pos0":
            assert torch.equal(actual, x)


def test_oracle_rope_vs_engine_fp16_table_path(oracle, rope_golden):
    """Golden: apply_rotary_pos_emb with fp16 cos/sin tables
    (baseline/naive_forward.py:38-48, engine/kvcache/paged_forward.py:32-44).  The
    reference itself only holds the fused kernels to atol = rtol = 2e-2 against this
    path (experiments/memory/benchmark_native_decode_rope_kv.py:103-104)."""
    for name in rope_golden.names:
        fields = rope_golden.case(name)
        x = tensor_from_bits(fields["x"])
        expected = tensor_from_bits(fields["expected_fp16_table_path"])
        actual = oracle.rope(x, torch.from_numpy(fields["positions"]))
        torch.testing.assert_close(actual, expected, atol=2e-2, rtol=2e-2)


def test_inv_freq_formula(oracle):
    table = oracle.inv_freq(1_000_000.0, 64)
    assert table[0].item() == 1.0
    expected = np.exp(np.arange(64, dtype=np.float32) * np.float32(-np.float32(np.log(1e6)) / 64))
    np.testing.assert_allclose(table.numpy(), expected, rtol=2e-7)


# ------------------------------------------------- fused epilogue + metadata

def test_packed_epilogue_known_answers(oracle):
    """experiments/tests/test_packed_qkv_epilogue.py:21-66 restated on the oracle."""
    packed = torch.arange(2048, dtype=torch.float32).to(torch.float16).view(1, 2048)
    k_pool = torch.full((1, 16, 2, 128), -1, dtype=torch.float16)
    v_pool = torch.full_like(k_pool, -2)
    q = oracle.packed_qkv_rope_cache(packed, torch.zeros(1, dtype=torch.int32),
                                     torch.tensor([3]), k_pool, v_pool)
    segments = packed.view(16, 128)
    assert torch.equal(q[0], segments[:12])
    assert torch.equal(k_pool.view(-1, 2, 128)[3], segments[12:14])
    assert torch.equal(v_pool.view(-1, 2, 128)[3], segments[14:16])

    generator = torch.Generator().manual_seed(3)
    packed = torch.randn(3, 2048, generator=generator).half()
    k_pool = torch.full((1, 16, 2, 128), -1, dtype=torch.float16)
    v_pool = torch.full_like(k_pool, -2)
    q = oracle.packed_qkv_rope_cache(packed, torch.zeros(3, dtype=torch.int32),
                                     torch.tensor([3, 4, 0]), k_pool, v_pool, valid_tokens=2)
    segments = packed.view(3, 16, 128)
    assert torch.equal(q[:2], segments[:2, :12]) and torch.equal(q[2], torch.zeros_like(q[2]))
    assert torch.equal(k_pool.view(-1, 2, 128)[3:5], segments[:2, 12:14])
    assert torch.equal(v_pool.view(-1, 2, 128)[3:5], segments[:2, 14:16])
    assert (k_pool.view(-1, 2, 128)[0] == -1).all() and (v_pool.view(-1, 2, 128)[0] == -2).all()


def test_decode_step_against_reference_routes(oracle):
    """Golden: one decode step (B=2, context 512, page 16, permuted pool) through
    the reference's CPU code, both routes."""
    data = np.load(GOLDEN_DIR / "decode_step_b2_ctx512.npz")
    k_pool, v_pool = tensor_from_bits(data["k_pool"]).clone(), tensor_from_bits(data["v_pool"]).clone()
    packed = tensor_from_bits(data["packed"])
    table, lens = torch.from_numpy(data["table"]), torch.from_numpy(data["seq_lens"])
    slots, positions = torch.from_numpy(data["slots"]), torch.from_numpy(data["positions"])
    q = oracle.packed_qkv_rope_cache(packed, positions, slots, k_pool, v_pool)
    k_rows, v_rows = k_pool.view(-1, 2, 128)[slots], v_pool.view(-1, 2, 128)[slots]
    out = oracle.paged_attention(q, k_pool, v_pool, table, lens)

    # fused-arithmetic route: rope_reference + index_copy_ + attention_reference
    assert torch.equal(v_rows, tensor_from_bits(data["fused_fp32/v_rows"]))  # V bit-exact
    source_k = packed[:, 1536:1792].view(2, 2, 128)
    source_q = packed[:, :1536].view(2, 12, 128)
    for actual, key, source in ((k_rows, "fused_fp32/k_rows", source_k), (q, "fused_fp32/q_rot", source_q)):
        expected = tensor_from_bits(data[key])
        partner = torch.cat((source[..., 64:], source[..., :64]), dim=-1)
        ulp = oracle.ulp_distance_fp16(actual, expected, torch.maximum(source.abs(), partner.abs()))
        assert ulp.max().item() <= 1.0
    assert_attention_close(out, tensor_from_bits(data["fused_fp32/attention"]))

    # engine-default route (fp16 cos/sin tables): V still bit-exact, Q/K within the
    # reference's own 2e-2 bound, attention within 2e-3
    assert torch.equal(v_rows, tensor_from_bits(data["engine_fp16_tables/v_rows"]))
    torch.testing.assert_close(k_rows, tensor_from_bits(data["engine_fp16_tables/k_rows"]), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(q, tensor_from_bits(data["engine_fp16_tables/q_rot"]), atol=2e-2, rtol=2e-2)
    assert_attention_close(out, tensor_from_bits(data["engine_fp16_tables/attention"]))


def test_metadata_against_reference(oracle):
    """Golden: PagedKVCache + build_decode_step_inputs
    (engine/kvcache/paged_kv_cache.py, engine/graph/paged_graph_decoder.py:392-417)."""
    data = np.load(GOLDEN_DIR / "metadata_case.npz")
    tables = [[int(p) for p in row if p >= 0] for row in data["tables"]]
    positions, seq_lens, table, slots = oracle.decode_step_inputs(
        data["cur_lens"].tolist(), tables, int(data["max_blocks"]))
    for actual, key in ((positions, "positions"), (seq_lens, "seq_lens"), (table, "block_table"),
                        (slots, "slot_mapping")):
        assert actual.dtype == data[key].dtype and np.array_equal(actual, data[key]), key


def test_advance_decode_state_against_reference_steps(oracle):
    """Golden: build_decode_step_inputs evaluated at 40 consecutive steps of a cohort
    whose pages were reserved up front; the advance of step s must be step s + 1
    (engine/cpp/src/iteration_loop.cpp:500-528; the relation asserted by
    engine/cpp/tests/test_iteration_loop.py:545-551)."""
    data = np.load(GOLDEN_DIR / "metadata_steps.npz")
    table = data["block_table"]
    positions, seq_lens = data["positions"][0], data["seq_lens"][0]
    for step in range(1, data["positions"].shape[0]):
        positions, seq_lens, slots = oracle.advance_decode_state(positions, seq_lens, table)
        assert np.array_equal(positions, data["positions"][step])
        assert np.array_equal(seq_lens, data["seq_lens"][step])
        assert np.array_equal(slots, data["slot_mapping"][step])
    # page size 4, the block size of the reference's own test
    positions, seq_lens, slots = oracle.advance_decode_state([2, 3, 10], [3, 4, 11], [[5, 9, 1], [7, 2, 8], [6, 0, 3]], 4)
    assert slots.tolist() == [5 * 4 + 3, 2 * 4 + 0, 3 * 4 + 3]
    with pytest.raises(IndexError):
        oracle.advance_decode_state([15], [16], [[3]])


# ------------------------------------------------------------------ RMSNorm

def _norm_cases():
    data = np.load(GOLDEN_DIR / "rms_norm_cases.npz")
    for name in sorted({key.split("/")[0] for key in data.files}):
        dtype_name = str(data[f"{name}/dtype"])
        yield name, {key.split("/")[1]: (tensor_from_bits(data[key], dtype_name) if data[key].dtype == np.int16
                                         else data[key])
                     for key in data.files if key.startswith(name + "/")}


def test_rms_norm_against_reference(oracle):
    """Golden: rms_norm_reference on the model-dtype residual sum
    (custom_kernels/fused_rms.py:137-140; the sum is exact, the norm within one unit in
    the last place of the 16-bit output -- the reference's own bounds are 0 and 2e-3,
    experiments/decode/benchmark_fa3_fusion_kernels.py:77-78) and nn.RMSNorm, the model's
    path without custom kernels (baseline/naive_forward.py:59-64)."""
    seen = 0
    for name, case in _norm_cases():
        epsilon = float(case["epsilon"])
        summed, normalized = oracle.residual_add_rms_norm(case["residual"], case["branch"], case["weight"], epsilon)
        assert torch.equal(summed, case["summed"]), name
        for actual, key in ((normalized, "normalized"), (oracle.rms_norm(case["residual"], case["weight"], epsilon), "plain")):
            distance = oracle.ulp_distance(actual, case[key])
            assert distance.max().item() <= 1.0, (name, key)
            assert (distance > 0).float().mean().item() < 1e-3, (name, key)  # rounding ties only
        torch.testing.assert_close(normalized.float(), case["torch_rmsnorm"].float(), atol=2e-3, rtol=1e-2)
        seen += 1
    assert seen == 5
    zero_row = oracle.rms_norm(torch.zeros(1, 8, dtype=torch.float16), torch.ones(8, dtype=torch.float16))
    assert torch.equal(zero_row, torch.zeros(1, 8, dtype=torch.float16))


# ---------------------------------------------------------------------- fp8

def test_e4m3_decode_table_matches_reference_and_torch(oracle):
    """Golden: dequantize on all 256 bytes (experiments/quant/tests/test_attention.py:18-22)."""
    data = np.load(GOLDEN_DIR / "fp8_codec.npz")
    table = oracle.e4m3_decode_table()
    expected = tensor_from_bits(data["decode_table"]).float()
    torch.testing.assert_close(table, expected, atol=0, rtol=0, equal_nan=True)
    native = torch.arange(256, dtype=torch.int32).to(torch.uint8).view(torch.float8_e4m3fn).float()
    torch.testing.assert_close(table, native, atol=0, rtol=0, equal_nan=True)


def test_e4m3_encode_matches_reference_quantize(oracle):
    """Golden: quantize() bytes with token and head scaling
    (experiments/quant/attention.py:27-41), byte for byte."""
    data = np.load(GOLDEN_DIR / "fp8_codec.npz")
    values = tensor_from_bits(data["values"]).float()
    for mode in ("token", "head"):
        scales = torch.from_numpy(data[f"{mode}_scales"])
        scaled = (values / scales[..., None]).clamp(-448.0, 448.0)
        assert torch.equal(oracle.e4m3_encode(scaled), torch.from_numpy(data[f"{mode}_bits"])), mode
    # every representable value encodes to itself; ties go to even
    table = oracle.e4m3_decode_table()
    finite = torch.isfinite(table)
    codes = torch.arange(256, dtype=torch.uint8)
    round_trip = oracle.e4m3_encode(table[finite])
    assert torch.equal(round_trip & 0x7F, codes[finite] & 0x7F)
    assert torch.equal(oracle.e4m3_encode(torch.tensor([17.0, 19.0, 500.0, -1e9, 2.0 ** -10])),
                       torch.tensor([0x58, 0x5A, 0x7E, 0xFE, 0x00], dtype=torch.uint8))


def test_page_quantizer_round_trip(oracle):
    generator = torch.Generator().manual_seed(5)
    pool = (torch.randn(6, 16, 2, 128, generator=generator) * 0.5).half()
    pool[2] = 0
    pool8, scales = oracle.quantize_pages(pool)
    amax = pool.float().abs().amax(dim=(1, 3))
    torch.testing.assert_close(scales, (amax / 448.0).clamp_min(1e-12), atol=0, rtol=0)
    expected = (pool.float() / scales[:, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    assert torch.equal(pool8, expected.view(torch.uint8))
    restored = oracle.dequantize_pages(pool8, scales)
    assert torch.isfinite(restored.float()).all()
    # e4m3 keeps 3 mantissa bits: relative error <= 2^-4 of the page maximum
    assert ((restored.float() - pool.float()).abs() <= amax[:, None, :, None] / 16 + 1e-6).all()
