"""GPU parity of the FP8-e4m3 KV-cache variant (per-page scales, in-kernel
dequantisation).  No reference kernel exists for this layout, so parity is pinned
as: codec bytes equal the reference codec's (through the oracle, which is pinned to
it), and attention over the FP8 cache equals the fp16 path run on the dequantised
cache, within the attention tolerance."""

from __future__ import annotations

import pytest
import torch

from conftest import assert_attention_close, make_paged_inputs

pytestmark = pytest.mark.gpu


def test_page_quantizer_is_byte_exact(package, oracle, cuda_device):
    generator = torch.Generator().manual_seed(5)
    pool = (torch.randn(40, 16, 2, 128, generator=generator) * 0.5).half()
    pool[3] = 0
    pool[4, :, 1] = 1000.0
    pool8, scales = package.quantize_kv_pool_e4m3(pool.to(cuda_device))
    ref8, ref_scales = oracle.quantize_pages(pool)
    assert torch.equal(scales.cpu(), ref_scales)
    assert torch.equal(pool8.cpu(), ref8)
    restored = package.dequantize_kv_pool_e4m3(pool8, scales)
    assert torch.equal(restored.cpu(), oracle.dequantize_pages(ref8, ref_scales))


@pytest.mark.parametrize("split_k", [1, 2, 8])
def test_fp8_attention_equals_fp16_on_dequantised_cache(package, oracle, cuda_device, split_k):
    lengths = [0, 1, 16, 17, 100, 513, 2048]
    q, k, v, table, lens = make_paged_inputs(lengths, seed=21, value_scale=0.5)
    dev = cuda_device
    k8, ks = package.quantize_kv_pool_e4m3(k.to(dev))
    v8, vs = package.quantize_kv_pool_e4m3(v.to(dev))
    out8 = package.grouped_splitk_decode_attention_fp8(
        q.to(dev), k8, v8, ks, vs, table.to(dev), lens.to(dev), split_k=split_k)
    # (a) the fp16 kernels on the dequantised cache
    k_hat = package.dequantize_kv_pool_e4m3(k8, ks)
    v_hat = package.dequantize_kv_pool_e4m3(v8, vs)
    out16 = package.grouped_splitk_decode_attention(q.to(dev), k_hat, v_hat, table.to(dev), lens.to(dev),
                                                    split_k=split_k)
    assert_attention_close(out8, out16)
    # (b) the CPU oracle on the dequantised cache
    expected = oracle.paged_attention(q, oracle.dequantize_pages(k8.cpu(), ks.cpu()),
                                      oracle.dequantize_pages(v8.cpu(), vs.cpu()), table, lens)
    assert_attention_close(out8, expected)
    # (c) quantisation error itself stays small against the unquantised cache: e4m3
    # keeps three mantissa bits, so a single value is off by at most 1/16 of itself
    # (a one-token sequence returns V itself); values here stay below 2.5
    exact = oracle.paged_attention(q, k, v, table, lens)
    assert (out8.cpu().float() - exact.float()).abs().max().item() <= 2.5 / 16


def test_fp8_generic_path_and_view_as_float8(package, oracle, cuda_device):
    """float8_e4m3fn-typed pools are accepted; the stride-generic kernel gives the same answer."""
    q, k, v, table, lens = make_paged_inputs([33, 200], seed=2, value_scale=0.5)
    dev = cuda_device
    k8, ks = package.quantize_kv_pool_e4m3(k.to(dev))
    v8, vs = package.quantize_kv_pool_e4m3(v.to(dev))
    args = (q.to(dev), k8.view(torch.float8_e4m3fn), v8.view(torch.float8_e4m3fn), ks, vs,
            table.to(dev), lens.to(dev))
    fast = package.grouped_splitk_decode_attention_fp8(*args, split_k=2)
    package.cabi.set_tuning(force_generic=True)
    try:
        generic = package.grouped_splitk_decode_attention_fp8(*args, split_k=2)
    finally:
        package.cabi.set_tuning()
    assert_attention_close(fast, generic)


def test_fp8_fixed_scale_write(package, oracle, cuda_device):
    """New token rows are quantised with the page's existing scale: V bytes equal the
    oracle's byte for byte (no rotation involved); K bytes may differ by one code
    where the fp32 rotation lands on a rounding boundary."""
    generator = torch.Generator().manual_seed(13)
    batch, pages = 24, 6
    packed = (torch.randn(batch, 2048, generator=generator) * 0.5).half()
    positions = torch.arange(batch, dtype=torch.int32) * 97 + 5
    slots = torch.randperm(pages * 16, generator=generator)[:batch]
    k_scale = torch.rand(pages, 2, generator=generator) * 0.004 + 0.002
    v_scale = torch.rand(pages, 2, generator=generator) * 0.004 + 0.002
    k8 = torch.full((pages, 16, 2, 128), 0x11, dtype=torch.uint8)
    v8 = torch.full((pages, 16, 2, 128), 0x22, dtype=torch.uint8)
    dev = cuda_device
    k8_dev, v8_dev = k8.to(dev), v8.to(dev)
    q = package.packed_qkv_rope_cache_fp8(packed.to(dev), positions.to(dev), slots.to(dev), k8_dev, v8_dev,
                                          k_scale.to(dev), v_scale.to(dev))
    k_rows = oracle.rope_f32(packed[:, 1536:1792].view(batch, 2, 128), positions)
    v_rows = packed[:, 1792:].view(batch, 2, 128).float()
    oracle.write_fixed_scale(k_rows, slots, k8, k_scale)
    oracle.write_fixed_scale(v_rows, slots, v8, v_scale)
    assert torch.equal(v8_dev.cpu(), v8)
    table = oracle.e4m3_decode_table()
    got, want = table[k8_dev.cpu().long()], table[k8.long()]
    mismatched = (k8_dev.cpu() != k8)
    assert mismatched.float().mean().item() < 1e-3
    # a differing byte is an adjacent code: at most one e4m3 step (<= 2^-3 relative)
    assert ((got - want).abs() <= want.abs() / 8 + 2.0 ** -9)[mismatched].all()
    q_ref = oracle.rope(packed[:, :1536].view(batch, 12, 128), positions)
    assert oracle.ulp_distance_fp16(q.cpu(), q_ref, packed[:, :1536].view(batch, 12, 128)).max().item() <= 1.0

    # decode layout entry point writes the same bytes
    k8_b, v8_b = torch.full_like(k8_dev, 0x11), torch.full_like(v8_dev, 0x22)
    p = packed.to(dev)[:, None, :]
    package.native_decode_rope_kv_write_fp8(
        p[..., :1536].view(batch, 1, 12, 128).transpose(1, 2),
        p[..., 1536:1792].view(batch, 1, 2, 128).transpose(1, 2),
        p[..., 1792:].view(batch, 1, 2, 128).transpose(1, 2),
        positions.to(dev), slots.to(dev), k8_b, v8_b, k_scale.to(dev), v_scale.to(dev))
    assert torch.equal(k8_b, k8_dev) and torch.equal(v8_b, v8_dev)


@pytest.mark.parametrize("mode", [3, 4, 5], ids=["cuda_core", "tensor_core", "tensor_core_solo"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fp8_persistent_kernels(package, oracle, cuda_device, mode, dtype):
    """The persistent kernels on FP8 pools (forced, whatever the batch size): mixed
    lengths with empty and one-token sequences, NaN bytes in the unused tail of every
    last page, per-page scales that differ by orders of magnitude, a bad page id."""
    generator = torch.Generator().manual_seed(17)
    lengths = [0, 1, 15, 16, 17, 33, 700, 0, 2500] + torch.randint(1, 600, (30,), generator=generator).tolist()
    q, k, v, table, lens = make_paged_inputs(lengths, seed=33, value_scale=0.5, dtype=dtype)
    # pages whose magnitudes differ: the scales span 1e-3 .. 1e1
    page_gain = torch.logspace(-1, 1.3, k.shape[0])[torch.randperm(k.shape[0], generator=generator)]
    k = (k.float() * page_gain[:, None, None, None].clamp(max=4.0)).to(dtype)
    v = (v.float() * page_gain[:, None, None, None]).to(dtype)
    dev = cuda_device
    k8, ks = package.quantize_kv_pool_e4m3(k.to(dev))
    v8, vs = package.quantize_kv_pool_e4m3(v.to(dev))
    # poison the unused rows of every last page with the e4m3 NaN byte
    for row, length in enumerate(lengths):
        if length % 16:
            page = table[row, (length - 1) // 16].item()
            k8[page, length % 16:] = 0x7F
            v8[page, length % 16:] = 0x7F
    expected = oracle.paged_attention(q, oracle.dequantize_pages(k8.cpu(), ks.cpu(), dtype=dtype),
                                      oracle.dequantize_pages(v8.cpu(), vs.cpu(), dtype=dtype), table, lens)
    for split_k in (2, 5, 22):
        package.cabi.set_tuning(force_generic=mode)
        try:
            out = package.grouped_splitk_decode_attention_fp8(
                q.to(dev), k8, v8, ks, vs, table.to(dev), lens.to(dev), split_k=split_k)
        finally:
            package.cabi.set_tuning()
        assert torch.isfinite(out.float()).all()
        # relative to the magnitude of the values (up to ~20 here)
        scale = expected.float().abs().amax(dim=-1, keepdim=True).clamp(min=1.0)
        error = ((out.cpu().float() - expected.float()).abs() / scale).max().item()
        assert error <= (2e-2 if dtype == torch.bfloat16 else 4e-3), error
    assert package.cabi.device_status() == 0


def test_fp8_tensor_core_long_share(package, oracle, cuda_device):
    """One long sequence and two split slots: a CTA's share is hundreds of pages, so every
    warp walks several 32-page descriptor chunks and the ring wraps many times."""
    q, k, v, table, lens = make_paged_inputs([20000, 300], seed=37, value_scale=0.5)
    dev = cuda_device
    k8, ks = package.quantize_kv_pool_e4m3(k.to(dev))
    v8, vs = package.quantize_kv_pool_e4m3(v.to(dev))
    expected = oracle.paged_attention(q, oracle.dequantize_pages(k8.cpu(), ks.cpu()),
                                      oracle.dequantize_pages(v8.cpu(), vs.cpu()), table, lens)
    for split_k in (2, 9):
        out = package.grouped_splitk_decode_attention_fp8(
            q.to(dev), k8, v8, ks, vs, table.to(dev), lens.to(dev), split_k=split_k)
        assert_attention_close(out, expected)
    assert package.cabi.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fp8_fused_step_equals_the_two_operators(package, oracle, cuda_device, dtype):
    """The decode step on FP8 pools in two launches (RoPE + KV write inside the partial pass):
    the pools' bytes -- new rows quantised at their page's scales, everything else untouched --
    and the attention output are those of packed_qkv_rope_cache_fp8 followed by
    grouped_splitk_decode_attention_fp8, bit for bit; new token first / last in its page,
    one-token sequences, sequences over several CTAs, many short ones."""
    generator = torch.Generator().manual_seed(5)
    for lengths, split_k in (([1, 16, 17, 32, 33, 100, 2049, 4000], 8),
                             (torch.randint(1, 300, (200,), generator=generator).tolist(), 3),
                             ([700, 9, 31, 1500, 64, 65, 3, 48, 1024, 1025, 250, 16] * 4, 6)):
        q, k, v, table, lens = make_paged_inputs(lengths, seed=len(lengths), value_scale=0.5, dtype=dtype)
        dev = cuda_device
        k8, ks = package.quantize_kv_pool_e4m3(k.to(dev))
        v8, vs = package.quantize_kv_pool_e4m3(v.to(dev))
        batch = len(lengths)
        packed = (torch.randn((batch, 2048), generator=generator) * 0.5).to(dtype).to(dev)
        positions = (lens - 1).to(dev)
        rows = torch.arange(batch)
        slots = (table[rows, ((lens - 1) // 16).long()].long() * 16 + ((lens - 1) % 16).long()).to(dev)
        table_dev, lens_dev = table.to(dev), lens.to(dev)
        # poison the new rows: both paths must overwrite them
        for pool in (k8, v8):
            pool.view(-1, 2, 128)[slots] = 0x7F
        k_pair, v_pair = k8.clone(), v8.clone()
        q_pair = package.packed_qkv_rope_cache_fp8(packed, positions, slots, k_pair, v_pair, ks, vs)
        want = package.grouped_splitk_decode_attention_fp8(q_pair, k_pair, v_pair, ks, vs, table_dev, lens_dev,
                                                           split_k=split_k)
        k_fused, v_fused = k8.clone(), v8.clone()
        got = package.packed_qkv_rope_attention_fp8(packed, positions, slots, k_fused, v_fused, ks, vs, table_dev,
                                                    lens_dev, split_k=split_k, require_fused=True)
        assert package.cabi.device_status() == 0
        assert torch.equal(k_fused, k_pair) and torch.equal(v_fused, v_pair)
        assert not bool((k_fused.view(-1, 2, 128)[slots] == 0x7F).all())
        assert torch.equal(got, want)
        assert torch.isfinite(got.float()).all()
