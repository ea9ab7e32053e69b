"""CPU checks of bench.py's contract: the reference arm prints one JSON line with the keys the
driver reads, measured on whole steps, and names its workload with exactly the dictionary the
GPU arm prints; the staged reference path agrees with the oracle."""

from __future__ import annotations

import importlib.util
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

REPO_ROOT = Path(__file__).resolve().parents[1]


def _load(name, path):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


@pytest.fixture(scope="module")
def bench():
    return _load("qf_bench", REPO_ROOT / "bench.py")


def test_reference_arm_line(package, bench):
    result = subprocess.run(
        [sys.executable, str(REPO_ROOT / "bench.py"), "--impl", "reference", "--workload", "cpu_single_layer_b8",
         "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=600, cwd=REPO_ROOT)
    assert result.returncode == 0, result.stderr[-2000:]
    line = json.loads(result.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == bench.METRIC and line["unit"] == bench.UNIT
    assert line["higher_is_better"] is True and line["steps"] == 2 and line["n_gpus"] == 1
    assert line["value"] > 0 and line["ms_per_step"] > 0
    assert line["e2e"] == {"value": line["value"], "unit": bench.UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    baseline = line["cpu_baseline"]
    assert baseline["kind"] in ("reference", "port") and baseline["cores"] >= 1 and baseline["value"] == line["value"]
    # tokens/s = sequences of the step / measured step time: a measured step, not an extrapolation
    assert line["value"] == pytest.approx(8 / (line["ms_per_step"] * 1e-3), rel=1e-6)
    # the workload is named exactly as the GPU arm names it
    workload = package.workloads.build_workload("cpu_single_layer_b8")
    assert line["config"] == bench.workload_config(package, "cpu_single_layer_b8", workload, 1, "weak")


def test_workload_config_names_no_implementation(package, bench):
    workload = package.workloads.build_workload("decode_b64", rank=1, world_size=4)
    config = bench.workload_config(package, "decode_b64", workload, 4, "weak")
    assert config["workload"] == "decode_b64" and config["global_batch"] == 256 and config["batch_per_gpu"] == 64
    assert "equal cost" in config["rank_batches"]
    assert not {"split_k", "kernel", "fused_write", "model"} & set(config)
    strong = package.workloads.build_workload("sweep_b256", rank=0, world_size=8, scaling="strong")
    config = bench.workload_config(package, "sweep_b256", strong, 8, "strong")
    assert config["global_batch"] == 256 and config["batch_per_gpu"] == 32


def test_sample_spreads_over_the_length_range(bench):
    lengths = list(range(100, 164))
    picks = bench.sample_indices(lengths, 8)
    assert len(picks) == len(set(picks)) == 8 and picks == sorted(picks)
    mean = sum(lengths[i] for i in picks) / 8
    assert abs(mean - sum(lengths) / 64) <= 1.0
    assert bench.sample_indices(lengths, 100) == list(range(64))


def test_staged_reference_path_agrees_with_the_oracle(package, oracle):
    """The reference's own torch path (when staged) against the oracle on one small layer: V rows
    bit for bit, K rows and attention within the bounds the reference holds its fused kernels to
    against this very path (experiments/memory/benchmark_native_decode_rope_kv.py:103-105)."""
    build_ref = _load("qf_build_ref", REPO_ROOT / "oracle" / "build_ref.py")
    if not build_ref.available():
        build_ref.build_ref()
    if not build_ref.available():
        pytest.skip("oracle/_ref/ is not staged and the reference tree is not on this machine")
    reference = build_ref.ReferencePath()
    workload = package.workloads.build_workload("cpu_single_layer_b8")
    generator = torch.Generator().manual_seed(3)
    k_pool = (torch.randn(workload.num_pages, 16, 2, 128, generator=generator) * 0.5).half()
    v_pool = (torch.randn(workload.num_pages, 16, 2, 128, generator=generator) * 0.5).half()
    packed = (torch.randn(workload.batch, 2048, generator=generator) * 0.5).half()
    k_ref, v_ref = k_pool.clone(), v_pool.clone()
    out_ref = reference.layer(packed, workload.positions, workload.slot_mapping, k_ref, v_ref,
                              workload.block_table, workload.seq_lens)
    k_or, v_or = k_pool.clone(), v_pool.clone()
    q = oracle.packed_qkv_rope_cache(packed, workload.positions, workload.slot_mapping, k_or, v_or)
    out_or = oracle.paged_attention(q, k_or, v_or, workload.block_table, workload.seq_lens)
    assert torch.equal(v_ref, v_or)
    torch.testing.assert_close(k_ref.float(), k_or.float(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(out_ref.float(), out_or.float(), atol=2e-3, rtol=2e-3)
