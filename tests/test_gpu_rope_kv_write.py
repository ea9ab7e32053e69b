"""GPU parity of the fused RoPE + paged KV write kernels against the CPU oracle and
the committed reference outputs.  Every call goes through the C ABI
(libqf_hotpath.so) via the drop-in modules.

Bars: slot placement and V rows bit-exact; untouched pool rows untouched;
rotated Q/K within 1 fp16 ulp of the fp32 single-rounding oracle (ulp measured at
the magnitude of the rotation's operands)."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR, tensor_from_bits

pytestmark = pytest.mark.gpu


def _operand_magnitude(x):
    half = x.shape[-1] // 2
    partner = torch.cat((x[..., half:], x[..., :half]), dim=-1)
    return torch.maximum(x.float().abs(), partner.float().abs())


def _assert_rotation_close(oracle, actual, expected, source, max_ulp=1.0):
    """<= max_ulp fp16 units in the last place, the unit taken at the magnitude of the
    rotation's operands (x1*c - x2*s cancels: a result can be far smaller than the values it
    was computed from).  The plain largest difference is printed and reported beside it, and
    bounded by that many units at the largest operand."""
    magnitude = _operand_magnitude(source.cpu())
    ulp = oracle.ulp_distance_fp16(actual, expected, magnitude)
    plain = (actual.float() - expected.float()).abs().max().item()
    print(f"rotation: {ulp.max().item():.2f} ulp at the operands' magnitude, plain max-abs {plain:.3e}")
    assert ulp.max().item() <= max_ulp, f"{ulp.max().item()} ulp (plain max-abs {plain})"
    largest = float(magnitude.max())
    assert plain <= max_ulp * 2.0 ** -10 * max(largest, 2.0 ** -14) , f"plain max-abs {plain}"
    assert torch.isfinite(actual.float()).all()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("position_dtype", [torch.int32, torch.int64, torch.float32])
def test_native_decode_layout(package, oracle, cuda_device, dtype, position_dtype):
    """(B, H, 1, D) strided views of a packed projection, NaN-filled pools, random
    slot permutation (correctness/checks/check_custom_kernels.py:109-148 adapted to
    the decode layout)."""
    generator = torch.Generator().manual_seed(4)
    batch, pages = 37, 5
    packed = (torch.randn(batch, 1, 2048, generator=generator) * 0.5).to(dtype)
    q = packed[..., :1536].view(batch, 1, 12, 128).transpose(1, 2)
    k = packed[..., 1536:1792].view(batch, 1, 2, 128).transpose(1, 2)
    v = packed[..., 1792:].view(batch, 1, 2, 128).transpose(1, 2)
    positions = (torch.arange(batch) * 331 + 4090).to(position_dtype)
    slots = torch.randperm(pages * 16, generator=generator)[:batch]
    k_pool = torch.full((pages, 16, 2, 128), float("nan"), dtype=dtype)
    v_pool = torch.full_like(k_pool, float("nan"))

    dev = cuda_device
    packed_dev = packed.to(dev)
    q_dev = packed_dev[..., :1536].view(batch, 1, 12, 128).transpose(1, 2)
    k_dev = packed_dev[..., 1536:1792].view(batch, 1, 2, 128).transpose(1, 2)
    v_dev = packed_dev[..., 1792:].view(batch, 1, 2, 128).transpose(1, 2)
    kp, vp = k_pool.to(dev), v_pool.to(dev)
    out = package.native_decode_rope_kv_write(
        q_dev, k_dev, v_dev, positions.to(dev), slots.to(dev), kp, vp, rotate_q=True)
    assert out.shape == q.shape and out.dtype == dtype

    q_ref = oracle.rope(q[:, :, 0, :], positions)
    k_ref = oracle.rope(k[:, :, 0, :], positions)
    if dtype == torch.float16:
        _assert_rotation_close(oracle, out.cpu()[:, :, 0, :], q_ref, q[:, :, 0, :])
        _assert_rotation_close(oracle, kp.cpu().view(-1, 2, 128)[slots], k_ref, k[:, :, 0, :])
    else:
        # one bf16 ulp is eight fp16 ulps
        _assert_rotation_close(oracle, out.cpu()[:, :, 0, :], q_ref, q[:, :, 0, :], max_ulp=8.0)
        _assert_rotation_close(oracle, kp.cpu().view(-1, 2, 128)[slots], k_ref, k[:, :, 0, :], max_ulp=8.0)
    # V: bit-exact; every slot not in the mapping still NaN
    assert torch.equal(vp.cpu().view(-1, 2, 128)[slots].view(torch.int16),
                       v[:, :, 0, :].contiguous().view(torch.int16))
    untouched = torch.ones(pages * 16, dtype=torch.bool)
    untouched[slots] = False
    assert torch.isnan(kp.cpu().view(-1, 2, 128)[untouched].float()).all()
    assert torch.isnan(vp.cpu().view(-1, 2, 128)[untouched].float()).all()

    # rotate_q=False: q returned untouched (same object), only K/V written
    kp2, vp2 = k_pool.to(dev), v_pool.to(dev)
    same = package.native_decode_rope_kv_write(
        q_dev, k_dev, v_dev, positions.to(dev), slots.to(dev), kp2, vp2, rotate_q=False)
    assert same is q_dev
    assert torch.equal(kp2.view(torch.int16), kp.view(torch.int16))
    assert torch.equal(vp2.view(torch.int16), vp.view(torch.int16))


def test_packed_layout_129_tokens(package, oracle, cuda_device):
    """rope_kv_write on (1, H, T, D): 129 tokens at positions 4096.., NaN pools,
    random slots; V error exactly 0 (correctness/checks/check_custom_kernels.py:109-148)."""
    torch.manual_seed(4)
    tokens, page = 129, 16
    q = torch.randn(1, tokens, 12, 128).half().transpose(1, 2)
    k = torch.randn(1, tokens, 2, 128).half().transpose(1, 2)
    v = torch.randn(1, tokens, 2, 128).half().transpose(1, 2)
    positions = torch.arange(4096, 4096 + tokens, dtype=torch.int32)[None]
    num_slots = ((tokens + page - 1) // page + 2) * page
    slots = torch.randperm(num_slots)[:tokens]
    dev = cuda_device
    kp = torch.full((num_slots // page, page, 2, 128), float("nan"), dtype=torch.float16, device=dev)
    vp = torch.full_like(kp, float("nan"))
    q_out = package.rope_kv_write(q.to(dev), k.to(dev), v.to(dev), positions.to(dev), slots.to(dev),
                                  kp, vp, base=1_000_000.0, num_warps=2, num_stages=2)
    assert q_out.shape == q.shape
    q_rows = q[0].transpose(0, 1)
    k_rows = k[0].transpose(0, 1)
    _assert_rotation_close(oracle, q_out.cpu()[0].transpose(0, 1), oracle.rope(q_rows, positions[0]), q_rows)
    _assert_rotation_close(oracle, kp.cpu().view(-1, 2, 128)[slots], oracle.rope(k_rows, positions[0]), k_rows)
    assert torch.equal(vp.cpu().view(-1, 2, 128)[slots], v[0].transpose(0, 1).contiguous())


def test_packed_qkv_epilogue_known_answers(package, cuda_device):
    """experiments/tests/test_packed_qkv_epilogue.py:21-66: position 0 is the
    identity, K and V restart their head index, padded rows write zero Q and no KV."""
    dev = cuda_device
    packed = torch.arange(2048, device=dev, dtype=torch.float32).to(torch.float16).view(1, 2048)
    k_pool = torch.full((1, 16, 2, 128), -1, device=dev, dtype=torch.float16)
    v_pool = torch.full_like(k_pool, -2)
    q = package.packed_qkv_rope_cache(packed, torch.zeros(1, device=dev, dtype=torch.int32),
                                      torch.tensor([3], device=dev), k_pool, v_pool)
    segments = packed.view(16, 128)
    assert torch.equal(q[0], segments[:12])
    assert torch.equal(k_pool.view(-1, 2, 128)[3], segments[12:14])
    assert torch.equal(v_pool.view(-1, 2, 128)[3], segments[14:16])

    packed = torch.randn(3, 2048, device=dev, dtype=torch.float16)
    k_pool = torch.full((1, 16, 2, 128), -1, device=dev, dtype=torch.float16)
    v_pool = torch.full_like(k_pool, -2)
    q = package.packed_qkv_rope_cache(
        packed, torch.zeros(3, device=dev, dtype=torch.int32), torch.tensor([3, 4, 0], device=dev),
        k_pool, v_pool, valid_tokens=torch.tensor(2, device=dev, dtype=torch.int32))
    segments = packed.view(3, 16, 128)
    assert torch.equal(q[:2], segments[:2, :12])
    assert torch.equal(q[2], torch.zeros_like(q[2]))
    assert torch.equal(k_pool.view(-1, 2, 128)[3:5], segments[:2, 12:14])
    assert torch.equal(v_pool.view(-1, 2, 128)[3:5], segments[:2, 14:16])
    assert (k_pool.view(-1, 2, 128)[0] == -1).all() and (v_pool.view(-1, 2, 128)[0] == -2).all()


def test_packed_epilogue_matches_reference_outputs(package, oracle, cuda_device):
    """Golden: the decode step the reference's CPU code produced (both routes)."""
    data = np.load(GOLDEN_DIR / "decode_step_b2_ctx512.npz")
    dev = cuda_device
    kp = tensor_from_bits(data["k_pool"]).to(dev)
    vp = tensor_from_bits(data["v_pool"]).to(dev)
    packed = tensor_from_bits(data["packed"])
    slots = torch.from_numpy(data["slots"])
    q = package.packed_qkv_rope_cache(packed.to(dev)[:, None, :], torch.from_numpy(data["positions"]).to(dev),
                                      slots.to(dev), kp, vp)
    k_rows, v_rows = kp.cpu().view(-1, 2, 128)[slots], vp.cpu().view(-1, 2, 128)[slots]
    assert torch.equal(v_rows, tensor_from_bits(data["fused_fp32/v_rows"]))
    _assert_rotation_close(oracle, k_rows, tensor_from_bits(data["fused_fp32/k_rows"]),
                           packed[:, 1536:1792].view(2, 2, 128))
    _assert_rotation_close(oracle, q.cpu(), tensor_from_bits(data["fused_fp32/q_rot"]),
                           packed[:, :1536].view(2, 12, 128))
    torch.testing.assert_close(q.cpu(), tensor_from_bits(data["engine_fp16_tables/q_rot"]), atol=2e-2, rtol=2e-2)
    # pool rows outside the two written slots are bit-identical to the input pool
    mask = torch.ones(kp.shape[0] * 16, dtype=torch.bool)
    mask[slots] = False
    assert torch.equal(kp.cpu().view(-1, 2, 128)[mask], tensor_from_bits(data["k_pool"]).view(-1, 2, 128)[mask])


def test_strided_elements_and_odd_geometry(package, oracle, cuda_device):
    """Element-strided sources (no 16-byte vectors possible), head_dim 64, 4 KV
    heads: exercises the scalar path of the kernel."""
    generator = torch.Generator().manual_seed(9)
    tokens, hq, hkv, dim = 19, 8, 4, 64
    wide_q = (torch.randn(1, hq, tokens, dim * 2, generator=generator) * 0.5).half()
    wide_k = (torch.randn(1, hkv, tokens, dim * 2, generator=generator) * 0.5).half()
    wide_v = (torch.randn(1, hkv, tokens, dim * 2, generator=generator) * 0.5).half()
    positions = torch.arange(100, 100 + tokens, dtype=torch.int64)
    slots = torch.randperm(32, generator=generator)[:tokens].int()
    dev = cuda_device
    kp = torch.zeros(2, 16, hkv, dim, dtype=torch.float16, device=dev)
    vp = torch.zeros_like(kp)
    q_out = package.rope_kv_write(wide_q.to(dev)[..., ::2], wide_k.to(dev)[..., ::2], wide_v.to(dev)[..., ::2],
                                  positions.to(dev), slots.to(dev), kp, vp)
    q_rows = wide_q[0, :, :, ::2].transpose(0, 1)
    k_rows = wide_k[0, :, :, ::2].transpose(0, 1)
    _assert_rotation_close(oracle, q_out.cpu()[0].transpose(0, 1), oracle.rope(q_rows, positions), q_rows)
    _assert_rotation_close(oracle, kp.cpu().view(-1, hkv, dim)[slots.long()], oracle.rope(k_rows, positions), k_rows)
    assert torch.equal(vp.cpu().view(-1, hkv, dim)[slots.long()], wide_v[0, :, :, ::2].transpose(0, 1).contiguous())


def test_validation_errors(package, cuda_device):
    dev = cuda_device
    q = torch.zeros(2, 12, 1, 128, device=dev, dtype=torch.float16)
    k = torch.zeros(2, 2, 1, 128, device=dev, dtype=torch.float16)
    pool = torch.zeros(1, 16, 2, 128, device=dev, dtype=torch.float16)
    pos = torch.zeros(2, device=dev, dtype=torch.int32)
    with pytest.raises(ValueError, match="one entry per batch row"):
        package.native_decode_rope_kv_write(q, k, k, pos[:1], pos, pool, pool)
    with pytest.raises(ValueError, match="share FP16 or BF16"):
        package.native_decode_rope_kv_write(q, k, k, pos, pos, pool.float(), pool.float())
    with pytest.raises(ValueError, match="contiguous"):
        strided_pool = torch.zeros(1, 2, 16, 128, device=dev, dtype=torch.float16).transpose(1, 2)
        package.native_decode_rope_kv_write(q, k, k, pos, pos, strided_pool, strided_pool)
    with pytest.raises(ValueError, match=r"\(batch, 2048\)"):
        package.packed_qkv_rope_cache(torch.zeros(2, 1024, device=dev, dtype=torch.float16), pos, pos, pool, pool)
    with pytest.raises(ValueError, match="CUDA int32 scalar"):
        package.packed_qkv_rope_cache(torch.zeros(2, 2048, device=dev, dtype=torch.float16), pos, pos, pool, pool,
                                      valid_tokens=torch.tensor(1))
    with pytest.raises(ValueError, match="batch dimension one"):
        package.rope_kv_write(q, k, k, pos, pos, pool, pool)
