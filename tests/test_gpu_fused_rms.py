"""GPU tests of RMSNorm and residual-add + RMSNorm (the steps either side of attention in
a decode layer) against the oracle, the golden outputs of the reference's CPU statement,
and the reference's own bounds."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from conftest import GOLDEN_DIR, tensor_from_bits

pytestmark = pytest.mark.gpu


def _golden_cases():
    data = np.load(GOLDEN_DIR / "rms_norm_cases.npz")
    for name in sorted({key.split("/")[0] for key in data.files}):
        dtype_name = str(data[f"{name}/dtype"])
        yield name, {key.split("/")[1]: (tensor_from_bits(data[key], dtype_name) if data[key].dtype == np.int16
                                         else data[key])
                     for key in data.files if key.startswith(name + "/")}


def _assert_one_ulp(oracle, actual, expected, context):
    distance = oracle.ulp_distance(actual, expected)
    assert distance.max().item() <= 1.0, context
    assert (distance > 0).float().mean().item() < 2e-3, context  # rounding ties only


def test_golden_cases(package, oracle, cuda_device):
    """The residual sum is bit-exact; the normalised rows are within one unit in the last
    place of the reference's CPU statement and of the oracle (fp32 sums taken in a
    different order can flip a rounding tie, nothing more)."""
    for name, case in _golden_cases():
        epsilon = float(case["epsilon"])
        residual, branch, weight = (case[key].to(cuda_device) for key in ("residual", "branch", "weight"))
        summed, normalized = package.residual_add_rms_norm(residual, branch, weight, epsilon)
        assert torch.equal(summed.cpu(), case["summed"]), name
        _assert_one_ulp(oracle, normalized, case["normalized"], name)
        _assert_one_ulp(oracle, normalized, oracle.residual_add_rms_norm(residual, branch, weight, epsilon)[1], name)
        torch.testing.assert_close(normalized.cpu().float(), case["normalized"].float(), atol=2e-3, rtol=2e-3)
        plain = package.rms_norm(residual, weight, epsilon)
        _assert_one_ulp(oracle, plain, case["plain"], name)
        assert torch.equal(residual.cpu(), case["residual"]) and torch.equal(branch.cpu(), case["branch"])


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_reference_check_shapes(package, oracle, cuda_device, dtype):
    """The shapes of the reference's own check (custom_kernels/fused_rms.py:166-180; bound
    max_err < 2e-2 there) plus a decode batch shaped (B, 1, 1536) as the layer passes it
    (experiments/decode/benchmark_fa3_fusion_kernels.py:64-78)."""
    generator = torch.Generator(device=cuda_device).manual_seed(7)
    for rows, hidden in ((128, 512), (256, 1000), (17, 4096), (512, 8192), (3, 20000)):
        x = torch.randn((rows, hidden), device=cuda_device, dtype=dtype, generator=generator)
        weight = torch.randn((hidden,), device=cuda_device, dtype=dtype, generator=generator)
        out = package.rms_norm(x, weight, 1e-6)
        expected = oracle.rms_norm(x, weight, 1e-6)
        if dtype == torch.float16:  # the reference's bound, stated for fp16
            assert (out.cpu().float() - expected.float()).abs().max().item() < 2e-2
        _assert_one_ulp(oracle, out, expected, (rows, hidden))
    residual = torch.randn((64, 1, 1536), device=cuda_device, dtype=dtype, generator=generator)
    branch = torch.randn(residual.shape, device=cuda_device, dtype=dtype, generator=generator)
    weight = torch.randn((1536,), device=cuda_device, dtype=dtype, generator=generator)
    summed, normalized = package.residual_add_rms_norm(residual, branch, weight)
    assert summed.shape == residual.shape and normalized.shape == residual.shape
    assert torch.equal(summed, residual + branch)
    _assert_one_ulp(oracle, normalized, oracle.residual_add_rms_norm(residual, branch, weight)[1], "decode")


def test_scalar_path_and_c_abi_strides(package, oracle, cuda_device):
    """Odd widths and unaligned rows take the element-wise path; row strides wider than a
    row, and outputs aliased onto inputs, go through the C ABI directly."""
    cabi = package.cabi
    generator = torch.Generator(device=cuda_device).manual_seed(9)
    for hidden in (1001, 7, 1):
        residual = torch.randn((6, hidden), device=cuda_device, dtype=torch.float16, generator=generator)
        branch = torch.randn((6, hidden), device=cuda_device, dtype=torch.float16, generator=generator)
        weight = torch.randn((hidden,), device=cuda_device, dtype=torch.float16, generator=generator)
        summed, normalized = package.residual_add_rms_norm(residual, branch, weight, 1e-5)
        want_sum, want_norm = oracle.residual_add_rms_norm(residual, branch, weight, 1e-5)
        assert torch.equal(summed.cpu(), want_sum)
        _assert_one_ulp(oracle, normalized, want_norm, hidden)
    # strided rows, in place: summed overwrites residual, normalized overwrites branch
    hidden, pitch = 1536, 2048
    storage = torch.randn((2, 9, pitch), device=cuda_device, dtype=torch.float16, generator=generator)
    before = storage.clone()
    weight = torch.randn((hidden,), device=cuda_device, dtype=torch.float16, generator=generator)
    residual, branch = storage[0, :, 8:8 + hidden], storage[1, :, 16:16 + hidden]
    want_sum, want_norm = oracle.residual_add_rms_norm(residual.contiguous(), branch.contiguous(), weight)
    cabi.check(cabi.library().qf_residual_add_rms_norm(
        residual.data_ptr(), pitch, branch.data_ptr(), pitch, weight.data_ptr(),
        residual.data_ptr(), pitch, branch.data_ptr(), pitch, 9, hidden, cabi.DTYPE_F16, 1e-6,
        cabi.stream_pointer(cuda_device)))
    assert torch.equal(storage[0, :, 8:8 + hidden].cpu(), want_sum)
    _assert_one_ulp(oracle, storage[1, :, 16:16 + hidden], want_norm, "in place")
    outside = torch.ones_like(storage, dtype=torch.bool)
    outside[0, :, 8:8 + hidden] = False
    outside[1, :, 16:16 + hidden] = False
    assert torch.equal(storage[outside], before[outside])  # nothing beyond the rows was touched


def test_error_behaviour_and_empty_inputs(package, cuda_device):
    x = torch.zeros((4, 64), dtype=torch.float16, device=cuda_device)
    weight = torch.ones(64, dtype=torch.float16, device=cuda_device)
    with pytest.raises(AssertionError, match="rows, N"):
        package.rms_norm(x[None], weight)
    with pytest.raises(AssertionError, match="contiguous"):
        package.rms_norm(x.t(), weight)
    with pytest.raises(AssertionError, match="weight must be"):
        package.rms_norm(x, weight[:32])
    with pytest.raises(ValueError, match="matching shapes and dtypes"):
        package.residual_add_rms_norm(x, x[:2], weight)
    with pytest.raises(ValueError, match="rank >= 2 FP16 or BF16"):
        package.residual_add_rms_norm(x.float(), x.float(), weight)
    with pytest.raises(ValueError, match="contiguous"):
        package.residual_add_rms_norm(x.t(), x.t(), weight)
    with pytest.raises(ValueError, match="hidden dimension"):
        package.residual_add_rms_norm(x, x, weight[:32])
    with pytest.raises(ValueError, match="device and dtype"):
        package.residual_add_rms_norm(x, x, weight.bfloat16())
    empty = torch.zeros((0, 64), dtype=torch.float16, device=cuda_device)
    assert package.rms_norm(empty, weight).shape == (0, 64)
    summed, normalized = package.residual_add_rms_norm(empty, empty, weight)
    assert summed.shape == (0, 64) and normalized.shape == (0, 64)
    zeros = package.rms_norm(x, weight)  # a zero row: epsilon alone under the root
    assert torch.equal(zeros, torch.zeros_like(x))


def test_chained_behind_attention_in_a_graph(package, oracle, cuda_device):
    """The layer's tail as the engine records it: KV write, attention, then the residual
    norm on a tensor derived from the attention output, captured in one graph with chained
    launches; replays equal the eager run with every launch fully ordered."""
    workload = package.workloads.build_workload("decode_b64", batch=16, layers=1)
    step = package.decode_step.DecodeStep(workload, cuda_device, split_k=4, package=package)
    step.load_packed_rows()
    generator = torch.Generator(device=cuda_device).manual_seed(13)
    residual = torch.randn((16, 1, 1536), device=cuda_device, dtype=torch.float16, generator=generator)
    weight = torch.randn((1536,), device=cuda_device, dtype=torch.float16, generator=generator)

    def tail():
        attention = step.layer(0)                      # (16, 12, 128)
        branch = attention.reshape(16, 1, 1536)        # stands in for o_proj(attention)
        return package.residual_add_rms_norm(residual, branch, weight)

    package.cabi.set_dependent_launch(False)
    try:
        want_sum, want_norm = (t.clone() for t in tail())
    finally:
        package.cabi.set_dependent_launch(True)
    stream = torch.cuda.Stream(cuda_device)
    stream.wait_stream(torch.cuda.current_stream(cuda_device))
    with torch.cuda.stream(stream):
        tail()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=stream):
        got_sum, got_norm = tail()
    for _ in range(3):
        got_sum.zero_(), got_norm.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(got_sum, want_sum) and torch.equal(got_norm, want_norm)
    _assert_one_ulp(oracle, got_norm, oracle.rms_norm(got_sum, weight), "graph")
