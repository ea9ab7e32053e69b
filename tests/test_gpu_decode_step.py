"""GPU tests of the whole decode step (RoPE + KV write, then attention, per layer)
on the benchmark configurations, through the public operators, eagerly, under CUDA
graph capture and through the host-buffer entry; plus the plugin boundary: the
drop-in files loaded the way the reference's kernel_dispatch loads them."""

from __future__ import annotations

import importlib.util

import pytest
import torch

from conftest import assert_attention_close

pytestmark = pytest.mark.gpu


def _oracle_step(oracle, workload, packed, k_pool, v_pool):
    """One layer on the CPU oracle; mutates the CPU pools, returns (q, out)."""
    q = oracle.packed_qkv_rope_cache(packed, workload.positions, workload.slot_mapping, k_pool, v_pool)
    out = oracle.paged_attention(q, k_pool, v_pool, workload.block_table, workload.seq_lens)
    return q, out


def _check_layer(oracle, step, layer, out_dev):
    w = step.workload
    k_cpu, v_cpu = step.k_pools[layer].cpu(), step.v_pools[layer].cpu()
    slots = w.slot_mapping
    # rebuild the pre-step pool: the written rows are the only difference
    packed = step.packed[layer].cpu()
    k_ref, v_ref = k_cpu.clone(), v_cpu.clone()
    _, out_ref = _oracle_step(oracle, w, packed, k_ref, v_ref)
    assert torch.equal(v_cpu.view(-1, 2, 128)[slots], packed[:, 1792:].view(-1, 2, 128))
    written, wanted = k_cpu.view(-1, 2, 128)[slots], k_ref.view(-1, 2, 128)[slots]
    ulp = oracle.ulp_distance_fp16(written, wanted, packed[:, 1536:1792].view(-1, 2, 128))
    k_plain = (written.float() - wanted.float()).abs().max().item()
    print(f"{w.name}: new K rows {ulp.max().item():.2f} ulp at the operands' magnitude, plain max-abs "
          f"{k_plain:.3e}; attention plain max-abs {(out_dev.cpu().float() - out_ref.float()).abs().max().item():.3e}")
    assert ulp.max().item() <= 1.0, f"{ulp.max().item()} ulp (plain max-abs {k_plain})"
    assert_attention_close(out_dev, out_ref)


def test_cpu_runnable_configuration(package, oracle, cuda_device):
    """Batch 8, context 512, one layer, 512-page permuted pool: eager, captured and
    host-buffer runs agree with the oracle and with each other."""
    workload = package.workloads.build_workload("cpu_single_layer_b8")
    for split_k in (1, 4):
        step = package.decode_step.DecodeStep(workload, cuda_device, split_k=split_k, package=package)
        step.load_packed_rows()
        eager = step.step().clone()
        _check_layer(oracle, step, 0, eager)
        step.capture()
        replayed = step.replay().clone()
        assert torch.equal(replayed, eager)
        host_out = step.run_from_host()
        torch.cuda.synchronize()
        assert torch.equal(host_out.to(cuda_device), eager)
        # the same call as one graph with the copies pipelined against the layers;
        # new host contents are picked up at replay
        step.capture_from_host()
        host = step.host_buffers()
        host["out"].zero_()
        assert torch.equal(step.run_from_host().to(cuda_device), eager)
        torch.cuda.synchronize()
        host["packed"].mul_(0.5)
        step.run_from_host()
        torch.cuda.synchronize()  # the call is asynchronous; the result is in pinned host memory now
        halved = host["out"].clone()
        host["packed"].mul_(2.0)
        assert not torch.equal(halved.to(cuda_device), eager)
        assert torch.equal(step.run_from_host().to(cuda_device), eager)
        assert step.h2d_bytes() == 8 * 2048 * 2 + 8 * (4 + 4 + 8) + 8 * 33 * 4
        assert step.d2h_bytes() == 8 * 12 * 128 * 2


def _plain_error(out_dev, out_ref):
    return (out_dev.cpu().float() - out_ref.float()).abs().max().item()


@pytest.mark.parametrize("fused_write", [False, True], ids=["three_launches", "two_launches"])
@pytest.mark.parametrize("name", ["decode_b64", "long_skew_b4", "sweep_b256"])
def test_full_size_single_layer(package, oracle, cuda_device, name, fused_write):
    """Full batch, context lengths and POOL of the large configurations, one layer, through
    the launches the benchmark times (split count as DecodeStep plans it -- 10 for decode_b64,
    3 for sweep_b256, 148 for long_skew_b4 -- with the RoPE / KV write as its own kernel and
    folded into the partial pass): checked against the oracle row by row, and split-count
    invariance.  sweep_b256
    runs in its real pool of 131 072 pages (1 GiB per tensor): page ids above 65 535 and
    byte offsets above 2^30 are indexed."""
    workload = package.workloads.build_workload(name, layers=1)
    if name == "sweep_b256":
        assert workload.num_pages == 131072 and int(workload.block_table.max()) > 65535
    step = package.decode_step.DecodeStep(workload, cuda_device, package=package,
                                          fused_write="always" if fused_write else False)
    assert step.fused_write == fused_write
    assert step.split_k == {"decode_b64": 10, "sweep_b256": 3, "long_skew_b4": 148}[name]
    step.load_packed_rows()
    out = step.step().clone()
    _check_layer(oracle, step, 0, out)
    other = package.decode_step.DecodeStep(workload, cuda_device, split_k=max(2, step.split_k // 2),
                                           fill_pools=False, package=package,
                                           fused_write="always" if fused_write else False)
    other.k_pools, other.v_pools, other.packed = step.k_pools, step.v_pools, step.packed
    assert_attention_close(other.step(), out)
    # the captured graph the benchmark replays gives the same bits as the eager launches
    step.capture()
    assert torch.equal(step.replay(), out)


def test_full_size_fp8_single_layer(package, oracle, cuda_device):
    """fp8_b128 at its full batch of 128 sequences x 2048 tokens, one layer: the new rows'
    V bytes equal the oracle's fixed-scale quantiser, attention equals the oracle on the
    dequantised cache, and the captured graph replays the same bits."""
    workload = package.workloads.build_workload("fp8_b128", layers=1)
    assert workload.batch == 128
    step = package.decode_step.DecodeStep(workload, cuda_device, package=package)
    step.load_packed_rows()
    v_before = step.v_pools[0].cpu()
    out = step.step().clone()
    packed = step.packed[0].cpu()
    oracle.write_fixed_scale(packed[:, 1792:].view(-1, 2, 128).float(), workload.slot_mapping, v_before,
                             step.v_scales[0].cpu())
    assert torch.equal(step.v_pools[0].cpu(), v_before)
    q = oracle.rope(packed[:, :1536].view(-1, 12, 128), workload.positions)
    expected = oracle.paged_attention(
        q, oracle.dequantize_pages(step.k_pools[0].cpu(), step.k_scales[0].cpu()),
        oracle.dequantize_pages(step.v_pools[0].cpu(), step.v_scales[0].cpu()),
        workload.block_table, workload.seq_lens)
    assert_attention_close(out, expected)
    step.capture()
    assert torch.equal(step.replay(), out)


def test_page_placement_invariance(package, cuda_device):
    """Moving every page somewhere else (pool and table permuted together) leaves the
    result bit-identical: only slot arithmetic changed."""
    workload = package.workloads.build_workload("decode_b64", layers=1, batch=16)
    step = package.decode_step.DecodeStep(workload, cuda_device, split_k=3, package=package)
    step.load_packed_rows()
    before = step.step().clone()
    generator = torch.Generator().manual_seed(77)
    perm = torch.randperm(workload.num_pages, generator=generator).to(cuda_device)  # new id of old page
    inverse = torch.empty_like(perm)
    inverse[perm] = torch.arange(workload.num_pages, device=cuda_device)
    step.k_pools[0] = step.k_pools[0][inverse].contiguous()
    step.v_pools[0] = step.v_pools[0][inverse].contiguous()
    step.block_table = perm[step.block_table.long()].int()
    step.slot_mapping = perm[(step.slot_mapping // 16)] * 16 + step.slot_mapping % 16
    assert torch.equal(step.step(), before)


def test_multi_layer_fp8_configuration(package, oracle, cuda_device):
    """Two layers of the FP8 configuration (batch 128, context 2048) against the
    fp16 kernels and the oracle on the dequantised cache."""
    workload = package.workloads.build_workload("fp8_b128", layers=2, batch=32)
    step = package.decode_step.DecodeStep(workload, cuda_device, package=package)
    step.load_packed_rows()
    out = step.step()
    layer = 1
    k_hat = package.dequantize_kv_pool_e4m3(step.k_pools[layer], step.k_scales[layer])
    v_hat = package.dequantize_kv_pool_e4m3(step.v_pools[layer], step.v_scales[layer])
    q = oracle.rope(step.packed[layer].cpu()[:, :1536].view(-1, 12, 128), workload.positions)
    expected = oracle.paged_attention(q, k_hat.cpu(), v_hat.cpu(), workload.block_table, workload.seq_lens)
    assert_attention_close(out, expected)
    step.capture()
    assert torch.equal(step.replay(), out)


def test_files_load_the_way_kernel_dispatch_loads_them(package, oracle, cuda_device):
    """baseline/kernel_dispatch.py:13-23 imports custom_kernels/<name>.py by file path
    under a private module name; the drop-in directory must work the same way."""
    def load(name):
        path = package.KERNEL_DIR / f"{name}.py"
        spec = importlib.util.spec_from_file_location(f"_inference_engine_{name}", path)
        module = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(module)
        return module

    names = {
        "rope_kv_write": ("rope_kv_write", "native_decode_rope_kv_write"),
        "packed_qkv_rope_cache": ("packed_qkv_rope_cache",),
        "paged_decode_grouped_splitk": ("grouped_splitk_decode_attention",),
        "paged_decode_native_grouped": ("native_grouped_splitk_decode_attention",
                                        "native_grouped_decode_diagnostics", "native_grouped_stage_cycles"),
    }
    modules = {name: load(name) for name in names}
    for name, functions in names.items():
        for function in functions:
            assert callable(getattr(modules[name], function))

    workload = package.workloads.build_workload("cpu_single_layer_b8")
    step = package.decode_step.DecodeStep(workload, cuda_device, split_k=8, package=package)
    step.load_packed_rows()
    # the accepted decode variant: (B, H, 1, D) views + native_decode_rope_kv_write,
    # then the dispatch call with the engine's frozen config
    packed = step.packed[0]
    batch = packed.shape[0]
    q = packed[:, :1536].view(batch, 1, 12, 128).transpose(1, 2)
    k = packed[:, 1536:1792].view(batch, 1, 2, 128).transpose(1, 2)
    v = packed[:, 1792:].view(batch, 1, 2, 128).transpose(1, 2)
    q_rot = modules["rope_kv_write"].native_decode_rope_kv_write(
        q, k, v, step.positions, step.slot_mapping, step.k_pools[0], step.v_pools[0],
        base=1_000_000.0, rotate_q=True)
    config = package.kv_layout.select_splitk_config(workload.max_context)
    out = modules["paged_decode_grouped_splitk"].grouped_splitk_decode_attention(
        q_rot[:, :, 0, :], step.k_pools[0], step.v_pools[0], step.block_table, step.seq_lens,
        scale=None, partials=None, **config)
    native = modules["paged_decode_native_grouped"].native_grouped_splitk_decode_attention(
        q_rot[:, :, 0, :], step.k_pools[0], step.v_pools[0], step.block_table, step.seq_lens,
        scale=None, partials=None, split_k=config["split_k"])
    _check_layer(oracle, step, 0, out)
    assert torch.equal(native, out)


def test_dependent_launch_on_and_off_agree(package, cuda_device):
    """The chained (programmatic dependent) launches and ordinary launches of the layer's
    three kernels give bit-identical pools and outputs, eagerly and in a replayed graph."""
    workload = package.workloads.build_workload("decode_b64", layers=3, batch=48)
    results = []
    for enabled in (True, False, True):
        package.cabi.set_dependent_launch(enabled)
        try:
            step = package.decode_step.DecodeStep(workload, cuda_device, package=package)
            eager = step.step().clone()
            step.capture()
            for _ in range(3):
                replayed = step.replay()
            torch.cuda.synchronize()
            replayed = replayed.clone()
            live = workload.live_pages.to(cuda_device)  # the rest of a pool is never written or read
            pools = [pool[live] for pool in step.k_pools] + [pool[live] for pool in step.v_pools]
        finally:
            package.cabi.set_dependent_launch(True)
        assert torch.equal(eager, replayed)
        assert torch.isfinite(eager.float()).all()
        results.append((eager, pools))
    for eager, pools in results[1:]:
        assert torch.equal(eager, results[0][0])
        for a, b in zip(pools, results[0][1]):
            assert torch.equal(a, b)
    assert package.cabi.device_status() == 0
