"""Shared fixtures.  GPU tests carry @pytest.mark.gpu and call through the C ABI;
everything else runs on CPU: the oracle against the committed golden vectors,
the host logic, and the load/export check of libqf_hotpath.so."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import pytest
import torch

REPO_ROOT = Path(__file__).resolve().parents[1]
GOLDEN_DIR = Path(__file__).resolve().parent / "golden"
if str(REPO_ROOT) not in sys.path:
    sys.path.insert(0, str(REPO_ROOT))

import __graft_entry__ as entry  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def package():
    """The product package; builds libqf_hotpath.so first when nvcc is available."""
    pkg = entry.load_package()
    if not pkg.cabi.LIBRARY_PATH.is_file():
        pkg.build.build_library()
    return pkg


@pytest.fixture(scope="session")
def oracle():
    return entry.load_oracle()


@pytest.fixture(scope="session")
def cuda_device():
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    return torch.device("cuda:0")


@pytest.fixture(autouse=True)
def _clean_device_status(request):
    """Every GPU test must leave the kernels' status word at zero."""
    yield
    if request.node.get_closest_marker("gpu") and torch.cuda.is_available():
        status = entry.load_package().cabi.device_status()
        assert status == 0, f"a kernel recorded status {status}"


def tensor_from_bits(array, dtype_name="float16"):
    """Inverse of make_golden.bits(): int16 bit patterns -> fp16 / bf16 tensor."""
    tensor = torch.from_numpy(np.ascontiguousarray(array))
    if tensor.dtype == torch.int16:
        return tensor.view(torch.float16 if dtype_name == "float16" else torch.bfloat16)
    return tensor


class GoldenCases:
    """Access to an .npz whose keys are 'case/field'."""

    def __init__(self, name):
        self.data = np.load(GOLDEN_DIR / name)
        self.names = sorted({key.split("/")[0] for key in self.data.files if "/" in key})

    def case(self, name):
        prefix = name + "/"
        return {key[len(prefix):]: self.data[key] for key in self.data.files if key.startswith(prefix)}


@pytest.fixture(scope="session")
def attention_golden():
    return GoldenCases("attention_cases.npz")


@pytest.fixture(scope="session")
def rope_golden():
    return GoldenCases("rope_cases.npz")


def attention_case_tensors(fields):
    """(q, k, v, table, lens, scale, expected) of one golden attention case."""
    dtype_name = str(fields["dtype"])
    q = tensor_from_bits(fields["q"], dtype_name)
    k = tensor_from_bits(fields["k"], dtype_name)
    v = tensor_from_bits(fields["v"], dtype_name)
    table = torch.from_numpy(fields["table"].copy())
    lens = torch.from_numpy(fields["lens"].copy())
    expected = tensor_from_bits(fields["expected"], dtype_name)
    return q, k, v, table, lens, float(fields["scale"]), expected


def with_gaps(tensor):
    """Strided, NaN/-1 padded view with the same values: every other element of a
    doubled last dimension (the layout stress of the reference's make_inputs,
    experiments/decode/grouped_splitk_validation.py:31-39)."""
    shape = list(tensor.shape)
    shape[-1] *= 2
    storage = torch.empty(shape, dtype=tensor.dtype, device=tensor.device)
    storage.fill_(float("nan") if tensor.is_floating_point() else -1)
    view = storage[..., ::2]
    view.copy_(tensor)
    return view


def make_paged_inputs(lengths, *, dtype=torch.float16, seed=0, page_size=16, kv_heads=2,
                      group=6, head_dim=128, poison=False, value_scale=1.0, extra_pages=0):
    """Seeded CPU inputs: random Q/K/V, randomly permuted pages, -1 table padding,
    optional NaN in the unused tail of each last page."""
    generator = torch.Generator().manual_seed(seed)
    counts = [(n + page_size - 1) // page_size for n in lengths]
    pages = max(1, sum(counts)) + extra_pages
    width = max(1, max(counts))
    q = (torch.randn(len(lengths), kv_heads * group, head_dim, generator=generator) * value_scale).to(dtype)
    k = (torch.randn(pages, page_size, kv_heads, head_dim, generator=generator) * value_scale).to(dtype)
    v = (torch.randn(pages, page_size, kv_heads, head_dim, generator=generator) * value_scale).to(dtype)
    order = torch.randperm(pages, generator=generator)
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    cursor = 0
    for row, (length, count) in enumerate(zip(lengths, counts)):
        table[row, :count] = order[cursor:cursor + count].int()
        if poison and length % page_size:
            last = order[cursor + count - 1]
            k[last, length % page_size:] = float("nan")
            v[last, length % page_size:] = float("nan")
        cursor += count
    return q, k, v, table, torch.tensor(lengths, dtype=torch.int32)


def assert_attention_close(actual, expected, dtype=None):
    """The reference's own gate (experiments/decode/grouped_splitk_validation.py:81-89):
    same dtype and shape, atol = rtol = 2e-3 for fp16 and 2e-2 for bf16; also the
    north-star bound max-abs 2e-3 / rel 1e-2 for fp16."""
    assert actual.dtype == expected.dtype and actual.shape == expected.shape
    tolerance = 2e-2 if actual.dtype == torch.bfloat16 else 2e-3
    torch.testing.assert_close(actual.cpu(), expected.cpu(), atol=tolerance, rtol=tolerance)
