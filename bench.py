"""Benchmark of the decode-step attention hot path (fused RoPE + paged KV write, then
GQA paged decode attention with split-K combine, over all 28 layers).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--split-k S]
    python bench.py --impl reference ...        # the reference's CPU implementation, same metric
    python bench.py --op layer_glue             # the small kernels either side of the path

A step is one pass of the hot path over one batch of synthetic input: for every
layer, the packed-QKV RoPE + KV write and the attention over the block tables.
Rank 0 prints ONE JSON line.

  parity     before anything is timed, one layer of every workload goes through exactly
             the call the timed graph records and is compared with the CPU oracle (pool
             rows bit for bit / within one fp16 ulp, attention within 2e-3); a failure
             ends the run without a number (the rule of the reference's own benchmarks,
             experiments/decode/benchmark_native_grouped_decode.py:123-135).
  value      decode tokens/s of the whole job with inputs resident in HBM: the step
             is replayed from one CUDA graph, `--steps` replays per timed region between
             barriers, CUDA events on the launching stream, max over ranks; the median
             of `--repeats` such regions (min and max beside it).
  e2e        the same metric through DecodeStep.run_from_host: per step the packed
             QKV rows and the metadata are copied from pinned host memory, the step
             runs and the result is copied back, all inside the timed region (one
             graph in which the copy of layer l + 1's rows overlaps layer l).
  roofline   achieved HBM bandwidth of the dominant kernel (the attention partial
             pass): its algorithmic bytes per launch divided by its average launch
             time, measured here with CUDA events over a graph of one launch per
             layer (28 different pools, 3.9 GB: nothing is served from L2).
  workloads  the other four benchmark configurations, each with its own parity check,
             step time and partial-pass roofline (one GPU); and `short_b512`, which is
             not one of the five: 512 sequences of 100 tokens, the regime in which the
             attention call picks the tensor-core kernel's solo variant.
  strong_sweep_b256  the batch of 256 sequences partitioned by sequence over the N
             ranks (snake dealing by length), tokens/s = 256 / slowest rank's step.
  cpu_baseline  the reference's own PyTorch path (staged under oracle/_ref/) on the
             host cores, on a bounded sample; its C port beside it; reported, not a target.

With N > 1 (torchrun) every rank owns a full batch of its own sequences and their
KV pages (weak scaling: the same multiset of context lengths on every rank, so the
ranks' costs are equal; pages and values differ); no collective runs inside a
timed region.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

REPO_ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO_ROOT))

import __graft_entry__ as entry  # noqa: E402

METRIC = "decode_attention_hot_path_tokens_per_s"
UNIT = "tokens/s"
LAYERS = 28
NOMINAL_HBM_GBS = 8000.0
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126e6
# the other four benchmark configurations, and one extra: the many-short-sequences regime
OTHER_WORKLOADS = ("cpu_single_layer_b8", "sweep_b256", "long_skew_b4", "fp8_b128", "short_b512")
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel, from the
# ncu captures summarised beside this file (same per-launch workload as a full-size launch:
# one layer of the named workload at seed 0).  Workloads without a capture report null.
NCU_TRAFFIC_BYTES_PER_LAUNCH = {  # (workload, seed, kernel): (bytes, split_k of the captured launches)
    ("decode_b64", 0, "decode_mma_kernel (solo)+rope"): (137.52e6 + 3.76e6, 10),  # the default: write folded in
    ("decode_b64", 0, "decode_mma_kernel"): (137.52e6 + 4.00e6, 10),      # interleaving variant, write as its own kernel
    ("decode_b64", 0, "decode_mma_kernel+rope"): (137.57e6 + 4.19e6, 10),  # interleaving variant, write folded in
    ("decode_b64", 0, "decode_partial_kernel"): (137.92e6 + 5.0e6, 10),
    ("sweep_b256", 0, "decode_mma_kernel (solo)+rope"): (410.24e6 + 2.58e6, 3),  # the default: write folded in
    ("sweep_b256", 0, "decode_mma_kernel (solo)"): (409.85e6 + 1.99e6, 3),
    ("sweep_b256", 0, "decode_mma_kernel"): (409.63e6 + 3.54e6, 3),
    ("long_skew_b4", 0, "decode_mma_kernel (solo)+rope"): (55.17e6 + 0.01e6, 148),  # the partials stay in L2
    ("long_skew_b4", 0, "decode_mma_kernel+rope"): (55.17e6 + 0.01e6, 148),
    ("fp8_b128", 0, "decode_mma_kernel (solo)+rope"): (135.23e6 + 1.92e6, 5),  # the default: write folded in
    ("fp8_b128", 0, "decode_mma_kernel (solo)"): (135.09e6 + 1.80e6, 5),
    ("fp8_b128", 0, "decode_mma_kernel"): (135.19e6 + 1.92e6, 5),
    ("short_b512", 0, "decode_mma_kernel (solo)+rope"): (54.63e6 + 0.05e6, 3),  # the default; the partials stay in L2
    ("short_b512", 0, "decode_mma_kernel (solo)"): (54.61e6 + 0.05e6, 3),
}


# --kernel -> qf_set_tuning mode: profiling and A/B runs of the other partial-pass kernels
KERNEL_MODES = {"auto": 0, "partitioned": 2, "persistent_cuda_core": 3, "persistent_mma": 4,
                "persistent_mma_solo": 5}


def parse_args():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--repeats", type=int, default=20,
                        help="timed regions of --steps replays each; the median region is reported with min and max\n"
                             "(the reference takes the median of at least 20 graph-amortised samples,\n"
                             "experiments/decode/benchmark_native_grouped_decode.py:44-68); the other\n"
                             "configurations take min(repeats, 5) regions")
    parser.add_argument("--impl", choices=("b200", "reference"), default="b200")
    parser.add_argument("--workload", default="decode_b64")
    parser.add_argument("--op", choices=("decode_step", "layer_glue", "cta_timeline"), default="decode_step",
                        help="layer_glue: residual-add + RMSNorm and the device-side metadata advance\n"
                             "cta_timeline: per-CTA time stamps of chained partial-pass launches\n"
                             "(one GPU; each prints its own JSON line)")
    parser.add_argument("--uniform-context", type=int, default=0,
                        help="cta_timeline: give every sequence this context length (equal work per CTA)")
    parser.add_argument("--shard-of", type=int, default=1,
                        help="cta_timeline: look at rank 0's shard of the workload split by sequence over this many ranks")
    parser.add_argument("--scaling", choices=("weak", "strong"), default="weak")
    parser.add_argument("--split-k", type=int, default=0, help="0: plan from host bounds")
    parser.add_argument("--layers", type=int, default=0, help="0: the workload's own (28)")
    parser.add_argument("--cpu-seconds", type=float, default=20.0, help="budget of the CPU baseline leg")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-workloads", action="store_true",
                        help="skip the other four configurations and the strong-scaling sweep")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--unfused-write", action="store_true",
                        help="RoPE + KV write as its own kernel: three launches per layer instead of two")
    parser.add_argument("--kernel", choices=tuple(KERNEL_MODES), default="auto",
                        help="partial-pass kernel of the fused attention call (auto: the library's choice)")
    return parser.parse_args()


def measured_peak_gbs():
    path = REPO_ROOT / "MEASURED_PEAKS.json"
    try:
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    except (OSError, KeyError, ValueError):
        return FALLBACK_HBM_GBS, "fallback"


def load_reference_path():
    """oracle/build_ref.py's view of the staged reference files, or None when they are absent."""
    spec = importlib.util.spec_from_file_location("qf_build_ref", REPO_ROOT / "oracle" / "build_ref.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    if not module.available():
        module.build_ref()  # only does something where the reference tree is on disk
    return module.ReferencePath() if module.available() else None


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index):
        self.device_index = device_index
        self.process = None
        self.file = None

    def __enter__(self):
        try:
            self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device_index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.process = None
        return self

    def __exit__(self, *exc):
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        return False

    def summary(self):
        result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.file is None:
            return result
        try:
            self.file.flush()
            rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.strip()]
            os.unlink(self.file.name)
        except OSError:
            return result
        clocks, reasons = [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for row in rows:
            if len(row) < 9:
                continue
            try:
                clocks.append(float(row[1]))
                result["sm_max_mhz"] = float(row[2])
            except ValueError:
                continue
            for name, cell in zip(names, row[5:9]):
                if cell.strip().lower() == "active":
                    reasons.add(name)
        if clocks:
            result["sm_mhz"] = statistics.median(clocks)
        result["reasons"] = sorted(reasons)
        result["samples"] = len(clocks)
        return result


def spread(samples):
    """median / min / max of a list of per-step milliseconds."""
    return {"median": statistics.median(samples), "min": min(samples), "max": max(samples), "regions": len(samples)}


def workload_config(package, name, workload, world, scaling):
    """What the timed workload is; the same dictionary in both arms (it names no implementation)."""
    fp8 = workload.fp8
    lengths = workload.seq_lens.tolist()
    kv_step = workload.layers * package.kv_layout.kv_bytes_per_layer(lengths, elem_bytes=1 if fp8 else 2)
    global_batch = workload.batch * world if scaling == "weak" else package.workloads.WORKLOADS[name]["batch"]
    config = {
        "workload": name, "doc": workload.meta["doc"], "global_batch": global_batch,
        "batch_per_gpu": workload.batch, "layers": workload.layers, "page_size": 16,
        "heads": "12q/2kv x 128", "parallelism": f"by-sequence x{world}",
        "l2": ("inputs exceed L2: each step reads %.2f GB of K/V from %d per-layer pools (L2 is 126 MB)"
               % (kv_step / 1e9, 2 * workload.layers)) if kv_step > L2_BYTES else
              "L2-resident: %.1f MB of K/V per step; timed L2-warm (back-to-back replays) and L2-evicted "
              "(a 256 MB buffer rewritten before every replay)" % (kv_step / 1e6),
    }
    if world > 1 and scaling == "weak":
        config["rank_batches"] = ("every rank runs the same multiset of context lengths (equal cost per rank); "
                                  "its pages, block tables and values are its own")
    return config


def partial_kernel_bytes(package, workload, split_k, fp8, kernel, ctas_per_head):
    """Algorithmic bytes of ONE launch of the attention partial pass (one layer):
    K+V of every attended token, the block table (and FP8 scales), the sequence
    lengths, Q, and what the kernel writes: fp32 partials + statistics of every
    split slot it fills (all of them for the per-partition kernel, one per piece for
    the persistent kernels), or the fp16 result when split_k is 1."""
    elem = 1 if fp8 else 2
    lengths = [int(t) for t in workload.seq_lens.tolist()]
    pages = sum(-(-t // 16) for t in lengths)
    total = sum(lengths) * 2 * 2 * 128 * elem + pages * 4
    if fp8:
        total += pages * 2 * 2 * 4
    batch = len(lengths)
    total += batch * 12 * 128 * 2 + batch * 4
    if split_k == 1:
        return total + batch * 12 * 128 * 2
    if kernel == "decode_partial_kernel":
        return total + batch * split_k * 12 * 130 * 4
    if kernel == "decode_mma_kernel (solo)":
        _, pieces = package.kv_layout.solo_schedule(lengths, split_k=split_k, ctas_per_head=ctas_per_head)
        return total + 2 * len(pieces) * 6 * 130 * 4
    tensor_core = kernel == "decode_mma_kernel"
    _, pieces = package.kv_layout.persistent_schedule(
        lengths, split_k=split_k, ctas_per_head=ctas_per_head, unit_tokens=16 if tensor_core else 32,
        overhead_units=package.kv_layout.TENSOR_CORE_PIECE_OVERHEAD if tensor_core else 0)
    return total + 2 * len(pieces) * 6 * 130 * 4


# --------------------------------------------------------------------------- parity gate
class ParityError(RuntimeError):
    pass


def preflight(package, oracle, step, layer=0):
    """One layer of `step`'s workload through exactly the call the timed graph records
    (`step.layer`), against the CPU oracle on the same inputs.  16-bit pools: V rows and
    every untouched pool row bit for bit, the new K rows within one fp16 ulp (unit taken
    at the magnitude of the rotation's operands; the plain difference is reported too),
    attention within max-abs 2e-3 and 1e-2 of the largest reference value.  FP8 pools:
    the new rows' bytes equal the oracle's fixed-scale quantiser, attention against the
    oracle on the dequantised cache.  Raises ParityError on a miss."""
    import torch

    w = step.workload
    if w.batch == 0:
        return {"checked_layers": 0}
    device = step.device
    slots = w.slot_mapping
    slots_dev = slots.to(device)
    row_width = 2 * 128
    k_before = step.k_pools[layer].clone()
    v_before = step.v_pools[layer].clone()
    out = step.layer(layer)
    torch.cuda.synchronize(device)
    status = package.cabi.device_status()
    if status != 0:
        raise ParityError(f"the kernels recorded device status {status}")

    def untouched(after, before):
        changed = (after.view(-1, row_width) != before.view(-1, row_width)).any(dim=1)
        changed[slots_dev] = False
        return not bool(changed.any().item())

    rows_untouched = untouched(step.k_pools[layer], k_before) and untouched(step.v_pools[layer], v_before)
    packed = step.packed[layer].cpu()
    result = {"checked_layers": 1, "batch": w.batch, "untouched_rows_bit_exact": rows_untouched}
    if step.fp8:
        k_after, v_after = step.k_pools[layer].cpu(), step.v_pools[layer].cpu()
        k_scale, v_scale = step.k_scales[layer].cpu(), step.v_scales[layer].cpu()
        q_ref = oracle.rope(packed[:, :1536].view(-1, 12, 128), w.positions)
        k_rows = oracle.rope_f32(packed[:, 1536:1792].view(-1, 2, 128), w.positions)
        k_ref, v_ref = k_before.cpu(), v_before.cpu()
        oracle.write_fixed_scale(k_rows, slots, k_ref, k_scale)
        oracle.write_fixed_scale(packed[:, 1792:].view(-1, 2, 128).float(), slots, v_ref, v_scale)
        result["kv_rows_byte_exact"] = bool(torch.equal(k_after, k_ref) and torch.equal(v_after, v_ref))
        expected = oracle.paged_attention(q_ref, oracle.dequantize_pages(k_after, k_scale),
                                          oracle.dequantize_pages(v_after, v_scale), w.block_table, w.seq_lens)
        result["reference"] = "oracle on the dequantised e4m3 cache"
        ok = result["kv_rows_byte_exact"]
    else:
        k_ref, v_ref = k_before.cpu(), v_before.cpu()
        q_ref = oracle.packed_qkv_rope_cache(packed, w.positions, slots, k_ref, v_ref)
        expected = oracle.paged_attention(q_ref, k_ref, v_ref, w.block_table, w.seq_lens)
        v_exact = bool(torch.equal(step.v_pools[layer].cpu(), v_ref))
        written = step.k_pools[layer].view(-1, 2, 128)[slots_dev].cpu()
        wanted = k_ref.view(-1, 2, 128)[slots]
        k_ulp = float(oracle.ulp_distance_fp16(written, wanted, packed[:, 1536:1792].view(-1, 2, 128)).max())
        result.update({"v_bit_exact": v_exact, "k_ulp": k_ulp,
                       "k_max_abs": float((written.float() - wanted.float()).abs().max()),
                       "reference": "oracle (fp32 accumulate) on the same pools"})
        ok = v_exact and k_ulp <= 1.0
    del k_before, v_before
    difference = (out.cpu().float() - expected.float()).abs()
    scale = float(expected.float().abs().max())
    result["max_abs"] = float(difference.max())
    result["max_abs_over_largest_value"] = result["max_abs"] / scale if scale else 0.0
    ok = ok and rows_untouched and result["max_abs"] <= 2e-3 and result["max_abs_over_largest_value"] <= 1e-2
    result["passed"] = bool(ok)
    if not ok:
        raise ParityError(f"parity check failed for {w.name}: {json.dumps(result)}")
    return result


# --------------------------------------------------------------------------- CPU legs
def sample_indices(lengths, count):
    """`count` sequences spread evenly over the batch sorted by length (a sample whose mean
    length is close to the batch's)."""
    order = sorted(range(len(lengths)), key=lambda i: (lengths[i], i))
    if count >= len(order):
        return sorted(order)
    picks = [order[int((j + 0.5) * len(order) / count)] for j in range(count)]
    return sorted(picks)


def host_pools(workload, layers, seed):
    """`layers` pairs of CPU pools (N(0,1)*0.5, fp16) and the packed rows of every layer.
    One pool pair is drawn; the others are that pair with its pages rolled by a
    layer-dependent offset inside the live set (distinct memory per layer, same value
    distribution, seconds instead of minutes of CPU random numbers)."""
    import torch

    generator = torch.Generator().manual_seed(5000 + seed)
    shape = (workload.num_pages, 16, 2, 128)
    live = workload.live_pages
    base_k = (torch.randn((live.numel(), 16, 2, 128), generator=generator) * 0.5).half()
    base_v = (torch.randn((live.numel(), 16, 2, 128), generator=generator) * 0.5).half()
    pools = []
    for layer in range(layers):
        k_pool = torch.zeros(shape, dtype=torch.float16)
        v_pool = torch.zeros(shape, dtype=torch.float16)
        k_pool[live] = torch.roll(base_k, layer * 37, dims=0)
        v_pool[live] = torch.roll(base_v, layer * 37, dims=0)
        pools.append((k_pool, v_pool))
    packed = (torch.randn(layers, workload.batch, 2048, generator=generator) * 0.5).half()
    return packed, pools


def reference_step_runner(reference, workload, packed, pools, picks):
    """A callable that runs every layer of the step for the sampled sequences through the
    reference's own functions and returns the last layer's output."""
    import torch

    index = torch.tensor(picks, dtype=torch.long)
    positions, slots = workload.positions[index], workload.slot_mapping[index]
    table, lens = workload.block_table[index], workload.seq_lens[index]
    rows = [packed[layer][index] for layer in range(len(pools))]

    def run():
        out = None
        for layer, (k_pool, v_pool) in enumerate(pools):
            out = reference.layer(rows[layer], positions, slots, k_pool, v_pool, table, lens)
        return out

    return run


def port_layer_seconds(oracle, workload, packed_row, k_pool, v_pool, budget_seconds):
    """Median time of the C/OpenMP port of the same path on one layer of the full batch."""
    times = []
    deadline = time.perf_counter() + budget_seconds
    while len(times) < 3 or (time.perf_counter() < deadline and len(times) < 30):
        start = time.perf_counter()
        q = oracle.packed_qkv_rope_cache(packed_row, workload.positions, workload.slot_mapping, k_pool, v_pool)
        oracle.paged_attention(q, k_pool, v_pool, workload.block_table, workload.seq_lens)
        times.append(time.perf_counter() - start)
    return statistics.median(times), len(times)


def cpu_baseline(package, oracle, workload, seed, budget_seconds):
    """The reference's PyTorch path on the host cores: every layer of the step for a
    bounded sample of the batch's sequences, whole steps, within the budget; its C port on
    one layer of the full batch beside it."""
    import torch

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    reference = load_reference_path()
    layers = workload.layers
    packed, pools = host_pools(workload, layers, seed)
    port_seconds, port_passes = port_layer_seconds(oracle, workload, packed[0], *pools[0], min(3.0, budget_seconds / 4))
    port = {"value": workload.batch / (port_seconds * layers), "unit": UNIT,
            "sample": f"C/OpenMP port, full batch, 1 of {layers} layers per pass (median of {port_passes}), scaled x{layers}"}
    if reference is None:
        return {"value": port["value"], "unit": UNIT, "cores": cores, "kind": "port", "sample": port["sample"],
                "note": "oracle/_ref/ is not staged on this machine: the reference's own functions could not be timed"}
    lengths = workload.seq_lens.tolist()
    picks = sample_indices(lengths, min(workload.batch, 8))
    run = reference_step_runner(reference, workload, packed, pools, picks)
    run()  # warm-up step
    times = []
    deadline = time.perf_counter() + budget_seconds
    while len(times) < 2 or (time.perf_counter() < deadline and len(times) < 10):
        start = time.perf_counter()
        run()
        times.append(time.perf_counter() - start)
    step_seconds = statistics.median(times)
    sample_tokens = sum(lengths[i] for i in picks)
    return {
        "value": len(picks) / step_seconds, "unit": UNIT, "cores": cores, "kind": "reference",
        "sample": (f"the reference's apply_rotary_pos_emb + index_copy_ + decode_attention_sdpa, all {layers} layers, "
                   f"{len(picks)} of {workload.batch} sequences spread over the length range "
                   f"({sample_tokens} of {sum(lengths)} attended tokens), median of {len(times)} whole steps "
                   f"({step_seconds * 1e3:.0f} ms each)"),
        "port": port,
    }


def run_reference(args, rank, world):
    """--impl reference: the reference's own CPU implementation of the path (its PyTorch
    functions, staged under oracle/_ref/) on the host cores, whole 28-layer steps.  A step
    covers a fixed sample of the batch's sequences, sized so that --steps + --warmup of them
    end within minutes; tokens/s = sampled sequences / step time."""
    if rank != 0:
        return
    import torch

    package = entry.load_package()
    workload = package.workloads.build_workload(args.workload, seed=args.seed, layers=args.layers or None,
                                                world_size=world, scaling=args.scaling)
    config = workload_config(package, args.workload, workload, world, args.scaling)
    if workload.fp8:
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference has no per-page-scale FP8 paged attention to time"}))
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    reference = load_reference_path()
    lengths = workload.seq_lens.tolist()
    packed, pools = host_pools(workload, workload.layers, args.seed)
    if reference is not None:
        kind = "reference"
        picks = sample_indices(lengths, min(workload.batch, 64))
        run = reference_step_runner(reference, workload, packed, pools, picks)
        what = (f"the reference's apply_rotary_pos_emb + index_copy_ + decode_attention_sdpa on {len(pools)} host "
                f"pool pairs, all {workload.layers} layers per step, {len(picks)} of {workload.batch} sequences "
                f"spread over the length range")
    else:
        kind = "port"
        oracle = entry.load_oracle()
        picks = list(range(workload.batch))

        def run():
            for layer, (k_pool, v_pool) in enumerate(pools):
                q = oracle.packed_qkv_rope_cache(packed[layer], workload.positions, workload.slot_mapping, k_pool, v_pool)
                oracle.paged_attention(q, k_pool, v_pool, workload.block_table, workload.seq_lens)

        what = (f"C/OpenMP port of the reference's PyTorch path (oracle/_ref/ is not staged here), all "
                f"{workload.layers} layers per step, full batch")
    for _ in range(max(args.warmup, 1)):
        run()
    times, begin = [], time.perf_counter()
    for _ in range(args.steps):
        start = time.perf_counter()
        run()
        times.append(time.perf_counter() - start)
        if time.perf_counter() - begin > 200:
            break
    step_seconds = sum(times) / len(times)
    value = len(picks) / step_seconds
    sample = f"{what}; mean of {len(times)} steps ({step_seconds * 1e3:.0f} ms each)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": max(args.warmup, 1), "ms_per_step": step_seconds * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f16 storage, f32 accumulate",
        "data": "synthetic", "config": config,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_layer_glue(args):
    """--op layer_glue: the kernels that sit either side of the hot path in a decode layer.

    qkv_rope_cache: the QKV projection with the RoPE / cache epilogue (TMA + tcgen05), one
    call per layer with that layer's own weights (176 MB in all: beyond L2), against the
    library GEMM followed by the packed epilogue kernel.
    residual_add_rms_norm: (a) at decode sizes, 56 calls (two per layer) chained in one
    graph -- launch latency, reported as microseconds per call; (b) 4096 x 8192 rows
    (268 MB moved, larger than L2) -- HBM bound, reported against the measured copy peak.
    unrolled steps: `--steps` consecutive decode steps of the workload recorded as ONE
    graph with the metadata advanced on the device, against the same number of single-step
    graph replays; no host-to-device copy in either."""
    import torch

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    package = entry.load_package()
    generator = torch.Generator(device=device).manual_seed(args.seed)

    def time_graph(record, replays):
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            record()
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            record()
        torch.cuda.current_stream(device).wait_stream(side)
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(replays):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / replays

    def norm_inputs(rows, hidden):
        make = lambda *shape: torch.randn(shape, device=device, dtype=torch.float16, generator=generator)
        return make(rows, hidden), make(rows, hidden), make(hidden)

    decode_sizes = {}
    for rows in (64, 256):
        residual, branch, weight = norm_inputs(rows, 1536)
        calls = 2 * LAYERS
        ms = time_graph(lambda: [package.residual_add_rms_norm(residual, branch, weight) for _ in range(calls)],
                        args.steps)
        decode_sizes[f"{rows}x1536"] = {"us_per_call": ms * 1e3 / calls, "calls_per_graph": calls}

    rows, hidden = 4096, 8192
    sets = [norm_inputs(rows, hidden) for _ in range(3)]  # 3 x 134 MB of inputs: beyond L2
    ms = time_graph(lambda: [package.residual_add_rms_norm(*inputs) for inputs in sets], args.steps) / len(sets)
    moved = 4 * rows * hidden * 2 + hidden * 2
    peak, peak_kind = measured_peak_gbs()
    achieved = moved / (ms * 1e-3) / 1e9
    oracle = entry.load_oracle()
    cpu_inputs = [t.cpu() for t in sets[0]]
    cpu_start = time.perf_counter()
    oracle.residual_add_rms_norm(*cpu_inputs)
    cpu_seconds = time.perf_counter() - cpu_start

    # ---- QKV projection with the RoPE / cache epilogue: 28 layers' weights in turn ----
    # (28 x 6.3 MB of weights: beyond L2, so every launch streams its matrix from HBM)
    projection = {}
    weights = [torch.randn((2048, 1536), device=device, dtype=torch.float16, generator=generator) * 0.05
               for _ in range(LAYERS)]
    bias = torch.randn((2048,), device=device, dtype=torch.float16, generator=generator) * 0.1
    pool_k = torch.zeros((1024, 16, 2, 128), device=device, dtype=torch.float16)
    pool_v = torch.zeros_like(pool_k)
    gamma = torch.randn((1536,), device=device, dtype=torch.float16, generator=generator)
    for rows in (64, 256):
        x = torch.randn((rows, 1536), device=device, dtype=torch.float16, generator=generator) * 0.5
        branch = torch.randn((rows, 1536), device=device, dtype=torch.float16, generator=generator) * 0.5
        positions = torch.randint(0, 4096, (rows,), device=device, generator=generator)
        slots = torch.randperm(1024 * 16, device=device, generator=generator)[:rows]
        fused = lambda h, w: package.qkv_rope_cache(h, w, bias, None, positions=positions, slots=slots,
                                                    k_pool=pool_k, v_pool=pool_v)
        unfused = lambda h, w: package.packed_qkv_rope_cache(torch.nn.functional.linear(h, w, bias),
                                                             positions, slots, pool_k, pool_v)
        norm = lambda: package.residual_add_rms_norm(x, branch, gamma)[1]
        fused_ms = time_graph(lambda: [fused(x, w) for w in weights], args.steps) / LAYERS
        unfused_ms = time_graph(lambda: [unfused(x, w) for w in weights], args.steps) / LAYERS
        # as a layer runs it: the norm before the projection, whose tail the projection's
        # set-up and first weight tiles overlap
        norm_ms = time_graph(lambda: [norm() for _ in weights], args.steps) / LAYERS
        fused_pair_ms = time_graph(lambda: [fused(norm(), w) for w in weights], args.steps) / LAYERS
        unfused_pair_ms = time_graph(lambda: [unfused(norm(), w) for w in weights], args.steps) / LAYERS
        moved_gemm = 2048 * 1536 * 2 + rows * 1536 * 2 + rows * 2048 * 2 + 2048 * 2 + rows * 16
        projection[f"{rows}x1536"] = {
            "us_per_call": fused_ms * 1e3, "us_per_call_cublas_plus_epilogue": unfused_ms * 1e3,
            "us_after_norm": (fused_pair_ms - norm_ms) * 1e3,
            "us_after_norm_cublas_plus_epilogue": (unfused_pair_ms - norm_ms) * 1e3,
            "algorithmic_bytes": moved_gemm,
            "roofline": {"bound": "hbm", "achieved": moved_gemm / (fused_ms * 1e-3) / 1e9, "peak": peak,
                         "unit": "GB/s", "frac": moved_gemm / (fused_ms * 1e-3) / 1e9 / peak,
                         "peak_kind": f"of {peak_kind}"}}
    del weights

    # ---- consecutive decode steps without the host ---------------------------------
    steps = max(2, min(args.steps, 16))
    chained_replays = 3
    workload = package.workloads.build_workload(args.workload, seed=args.seed, layers=args.layers or None,
                                                reserve_tokens=steps * (chained_replays + 1))
    step = package.decode_step.DecodeStep(workload, device, split_k=args.split_k or None, package=package,
                                          fused_write=not args.unfused_write)
    step.load_packed_rows()
    step.capture(warmup=2)
    step.capture_steps(steps)
    torch.cuda.synchronize()

    def replay_ms(run, count):
        for _ in range(3):
            run()
            step.reset_metadata()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(count):
            run()
        end.record()
        torch.cuda.synchronize()
        step.reset_metadata()
        return start.elapsed_time(end) / count

    single_ms = replay_ms(step.replay, steps)
    # the reserved pages cover one warm-up replay and the timed ones back to back
    step.steps_graph.replay()
    step.reset_metadata()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(chained_replays):
        step.steps_graph.replay()
    end.record()
    torch.cuda.synchronize()
    step.reset_metadata()
    unrolled_ms = start.elapsed_time(end) / (chained_replays * steps)
    # ---- the front of every layer as the engine would run it: norm, projection, attention ----
    front = None
    if not step.fp8 and workload.batch:
        b = workload.batch
        hidden_in = torch.randn((b, 1536), device=device, dtype=torch.float16, generator=generator) * 0.5
        branch_in = torch.randn((b, 1536), device=device, dtype=torch.float16, generator=generator) * 0.5
        layer_weights = [torch.randn((2048, 1536), device=device, dtype=torch.float16, generator=generator) * 0.03
                         for _ in range(step.layers)]

        def layer_front(fused):
            for index, w in enumerate(layer_weights):
                h = package.residual_add_rms_norm(hidden_in, branch_in, gamma)[1]
                if fused:
                    q = package.qkv_rope_cache(h, w, bias, None, positions=step.positions, slots=step.slot_mapping,
                                               k_pool=step.k_pools[index], v_pool=step.v_pools[index])
                else:
                    q = package.packed_qkv_rope_cache(torch.nn.functional.linear(h, w, bias), step.positions,
                                                      step.slot_mapping, step.k_pools[index], step.v_pools[index])
                package.grouped_splitk_decode_attention(q, step.k_pools[index], step.v_pools[index], step.block_table,
                                                        step.seq_lens, split_k=step.split_k, partials=step.partials)

        fused_front_ms = time_graph(lambda: layer_front(True), args.steps)
        library_front_ms = time_graph(lambda: layer_front(False), args.steps)
        front = {"layers": step.layers, "batch": b,
                 "ms_per_step_fused_projection": fused_front_ms,
                 "ms_per_step_library_gemm_plus_epilogue": library_front_ms,
                 "tokens_per_s_fused_projection": b / (fused_front_ms * 1e-3)}
    status = package.cabi.device_status()
    print(json.dumps({
        "op": "layer_glue", "n_gpus": 1, "data": "synthetic", "dtype": "f16 storage, f32 accumulate",
        "residual_add_rms_norm": {
            "decode": decode_sizes,
            "large": {"rows": 4096, "hidden": 8192, "ms_per_call": ms, "algorithmic_bytes": moved,
                      "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                                   "frac": achieved / peak, "peak_kind": f"of {peak_kind}"},
                      "cpu_baseline": {"value": moved / cpu_seconds / 1e9, "unit": "GB/s", "cores": os.cpu_count(),
                                       "kind": "port", "sample": "numpy oracle, one call on the same rows"}},
        },
        "qkv_rope_cache": projection,
        "layer_front_norm_projection_attention": front,
        "unrolled_decode_steps": {
            "workload": args.workload, "steps_per_graph": steps, "batch": workload.batch,
            "fused_write": step.fused_write,
            "ms_per_step_single_step_graph": single_ms, "ms_per_step_unrolled_graph": unrolled_ms,
            "tokens_per_s_unrolled": workload.batch / (unrolled_ms * 1e-3),
            "h2d_bytes_per_step": 0, "kernel_launches_per_graph": steps * (step.kernel_launches_per_step + 1),
        },
        "device_status": status,
    }))



# --------------------------------------------------------------------------- GPU arm
class Timer:
    """CUDA-event timing of regions bracketed by a barrier and a device synchronize."""

    def __init__(self, device, local_rank, distributed):
        import torch
        import torch.distributed as dist

        self.torch, self.dist = torch, dist
        self.device, self.local_rank, self.distributed = device, local_rank, distributed

    def barrier(self):
        if self.distributed:
            self.dist.barrier(device_ids=[self.local_rank])
        self.torch.cuda.synchronize(self.device)

    def max_over_ranks(self, milliseconds):
        if not self.distributed:
            return milliseconds
        tensor = self.torch.tensor([milliseconds], dtype=self.torch.float64, device=self.device)
        self.dist.all_reduce(tensor, op=self.dist.ReduceOp.MAX)
        return float(tensor.item())

    def region(self, run_once, steps):
        """(max over ranks, this rank's own) milliseconds of `steps` calls of run_once."""
        torch = self.torch
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        start.record()
        for _ in range(steps):
            run_once()
        end.record()
        self.barrier()
        own = start.elapsed_time(end)
        return self.max_over_ranks(own), own

    def per_step(self, run_once, steps, repeats):
        """Per-step milliseconds of `repeats` regions: (max-over-ranks list, own list)."""
        both = [self.region(run_once, steps) for _ in range(max(1, repeats))]
        return [m / steps for m, _ in both], [o / steps for _, o in both]

    def evicted(self, run_once, count, flush):
        """Per-call milliseconds with a buffer larger than L2 rewritten before every call."""
        torch = self.torch
        samples = []
        for _ in range(count):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            run_once()
            end.record()
            torch.cuda.synchronize(self.device)
            samples.append(start.elapsed_time(end))
        return samples


def partial_pass_leg(package, step, timer, steps, repeats, seed, world):
    """The dominant kernel alone: one partial-pass launch per layer in one graph, timed with
    CUDA events on the launching stream; algorithmic bytes per launch over the mean launch time."""
    import ctypes

    import torch

    workload, device = step.workload, step.device
    cabi = package.cabi
    splitk = package.kernel_module("paged_decode_grouped_splitk")
    q = torch.randn(workload.batch, 12, 128, device=device).mul_(0.5).to(step.dtype)
    partials = step.partials or step._fp8_partials()
    out = torch.empty_like(q)
    arg_sets, plain_sets = [], []
    for layer in range(step.layers):
        scales = (step.k_scales[layer], step.v_scales[layer]) if step.fp8 else None
        source = q
        if step.fused_write:  # the partial pass reads the layer's packed rows and writes the new K/V rows
            source = step.packed[layer].as_strided((workload.batch, 12, 128), (step.packed.stride(1), 128, 1))
            plain_sets.append(splitk.fill_attention_args(
                cabi, q, step.k_pools[layer], step.v_pools[layer], step.block_table, step.seq_lens,
                split_k=step.split_k, scale=128 ** -0.5, partials=partials, out=out, kv_scales=scales))
        arg_sets.append(splitk.fill_attention_args(
            cabi, source, step.k_pools[layer], step.v_pools[layer], step.block_table, step.seq_lens,
            split_k=step.split_k, scale=128 ** -0.5, partials=partials, out=out, kv_scales=scales))
    lib = cabi.library()
    kernel_name, ctas_per_head = cabi.fused_kernel_plan(arg_sets[0])

    def launch_partials(with_write=True):
        # the partial pass of the fused attention call, without its combine
        stream = cabi.stream_pointer(device)
        for arg in (arg_sets if with_write or not step.fused_write else plain_sets):
            if step.fused_write and with_write:
                cabi.check(lib.qf_packed_rope_decode_attention(
                    ctypes.byref(arg), step.positions.data_ptr(), cabi.torch_index_code(step.positions.dtype),
                    1, step.rope_table.data_ptr(), step.rope_table.shape[0], cabi.STAGE_PARTIAL, stream))
            else:
                cabi.check(lib.qf_grouped_splitk_decode_attention_stages(
                    ctypes.byref(arg), cabi.STAGE_PARTIAL, stream))

    def per_launch_ms(with_write):
        side = torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            launch_partials(with_write)
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            launch_partials(with_write)
        torch.cuda.current_stream(device).wait_stream(side)
        for _ in range(3):
            graph.replay()
        _, own = timer.per_step(graph.replay, steps, repeats)
        return [ms / step.layers for ms in own]

    launch_ms = per_launch_ms(True)
    kernel_ms = statistics.median(launch_ms)
    peak, peak_kind = measured_peak_gbs()
    launch_bytes = partial_kernel_bytes(package, workload, step.split_k, step.fp8, kernel_name, ctas_per_head)
    without_write = None
    if step.fused_write:
        plain_ms = statistics.median(per_launch_ms(False))
        without_write = {"us_per_launch": plain_ms * 1e3, "algorithmic_bytes_per_launch": launch_bytes,
                         "achieved": launch_bytes / (plain_ms * 1e-3) / 1e9,
                         "frac": launch_bytes / (plain_ms * 1e-3) / 1e9 / peak}
        # instead of rotated Q (12 x 128 x 2 B, already counted): the packed row (2048 x 2 B), a position
        # and its 512 B of the rotation table are read, the new K and V rows (2 x 2 x 128 x 2 B) written
        launch_bytes += workload.batch * ((2048 - 1536) * 2 + 4 + 512 + 2 * 2 * 128 * 2)
    achieved = launch_bytes / (kernel_ms * 1e-3) / 1e9
    kv_bytes = package.kv_layout.kv_bytes_per_layer(workload.seq_lens.tolist(), elem_bytes=1 if step.fp8 else 2)
    traffic = None
    captured = NCU_TRAFFIC_BYTES_PER_LAUNCH.get((workload.name, seed, kernel_name + ("+rope" if step.fused_write else "")))
    if world == 1 and captured is not None and step.split_k == captured[1] and step.layers == LAYERS:
        traffic = captured[0]
    return {
        "bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peak,
        "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
        "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS, "traffic": traffic,
        "fused_write": step.fused_write, "same_pass_without_the_write": without_write,
        "algorithmic_bytes_per_launch": launch_bytes, "us_per_launch": kernel_ms * 1e3,
        "us_per_launch_min_max": [min(launch_ms) * 1e3, max(launch_ms) * 1e3],
        "kv_bytes_per_launch": kv_bytes,
        # the K/V bytes alone over the same time (the pieces a launch writes are not counted)
        "frac_kv_only": kv_bytes / (kernel_ms * 1e-3) / 1e9 / peak,
    }


def step_algorithmic_bytes(package, step, leg):
    """What a whole step moves: per layer the partial pass's bytes, the pieces read again by the
    combine, and the result rows; plus, when the write is its own kernel, that kernel's bytes."""
    batch = step.batch
    combine = 0 if step.split_k == 1 else (leg["algorithmic_bytes_per_launch"] - leg["kv_bytes_per_launch"]) // 2
    per_layer = leg["algorithmic_bytes_per_launch"] + combine + batch * 12 * 128 * 2
    if not step.fused_write:
        elem = 1 if step.fp8 else 2
        per_layer += batch * (2048 * 2 + 12 * 128 * 2 + 2 * 2 * 128 * elem + 12)
    return step.layers * per_layer


def measure_workload(package, oracle, name, device, timer, args, world, rank, scaling="weak"):
    """Build one configuration on this rank, check it against the oracle, time its step and its
    partial pass.  Returns (record, workload, step)."""
    import torch

    workload = package.workloads.build_workload(name, rank=rank, world_size=world, scaling=scaling,
                                                seed=args.seed, layers=args.layers or None)
    step = package.decode_step.DecodeStep(workload, device, package=package, fused_write=not args.unfused_write)
    step.load_packed_rows()
    record = {"config": workload_config(package, name, workload, world, scaling),
              "split_k": step.split_k, "fused_write": step.fused_write}
    if workload.batch == 0:
        return record, workload, step
    record["parity"] = preflight(package, oracle, step)
    step.capture(warmup=2)
    for _ in range(max(args.warmup, 3)):
        step.replay()
    across, own = timer.per_step(step.replay, args.steps, min(args.repeats, 5))
    record["ms_per_step"] = spread(across)
    record["own_ms_per_step"] = statistics.median(own)
    record["tokens_per_s"] = workload.batch / (statistics.median(own) * 1e-3)
    leg = partial_pass_leg(package, step, timer, args.steps, min(args.repeats, 5), args.seed, world)
    record["roofline"] = {k: leg[k] for k in ("bound", "kernel", "achieved", "peak", "unit", "frac", "peak_kind",
                                              "frac_of_nominal_8TBs", "traffic", "algorithmic_bytes_per_launch",
                                              "us_per_launch", "kv_bytes_per_launch", "frac_kv_only")}
    step_bytes = step_algorithmic_bytes(package, step, leg)
    record["step_gbs"] = step_bytes / (statistics.median(own) * 1e-3) / 1e9
    record["step_frac"] = record["step_gbs"] / leg["peak"]
    kv_step = step.layers * leg["kv_bytes_per_launch"]
    record["l2_resident"] = kv_step <= L2_BYTES
    if record["l2_resident"]:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
        cold = timer.evicted(step.replay, 20, flush)
        record["ms_per_step_l2_evicted"] = spread(cold)
        record["ms_per_step_l2_warm"] = record["ms_per_step"]
        del flush
    record["device_status"] = package.cabi.device_status()
    return record, workload, step


def release():
    """Return freed device memory to the driver (the next configuration may need most of the GPU)."""
    import gc

    import torch

    gc.collect()
    torch.cuda.empty_cache()


def run_cta_timeline(args):
    """--op cta_timeline: `--layers` (default 4) launches of the instrumented tensor-core partial
    pass, one per layer pool, chained in one graph as the layers of a step are.  Every CTA
    stamps %globaltimer at entry, when its share is known, when its page ids are known, when its
    first tile has landed and at exit.  Printed: per launch the min / mean / max of each stamp
    (microseconds from the first launch's first entry), the histogram of exit times relative to
    the launch's earliest exit in 1 us bins, and the range of units per CTA."""
    import ctypes

    import torch

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    package = entry.load_package()
    cabi = package.cabi
    launches = args.layers or 4
    if args.uniform_context:
        default_batch = package.workloads.WORKLOADS[args.workload]["batch"]
        package.workloads.context_lengths = (
            lambda name, seed=0, batch=None: [args.uniform_context] * (batch or default_batch))
    workload = package.workloads.build_workload(args.workload, seed=args.seed, layers=launches,
                                                world_size=args.shard_of, scaling="strong" if args.shard_of > 1 else "weak")
    cabi.set_tuning(force_generic=KERNEL_MODES[args.kernel])  # auto: the solo variant; persistent_mma: the interleaving one
    step = package.decode_step.DecodeStep(workload, device, split_k=args.split_k or None, package=package)
    splitk = package.kernel_module("paged_decode_grouped_splitk")
    q = torch.randn(workload.batch, 12, 128, device=device).mul_(0.5).to(step.dtype)
    out = torch.empty_like(q)
    scales = lambda layer: (step.k_scales[layer], step.v_scales[layer]) if step.fp8 else None
    arg_sets = [splitk.fill_attention_args(
        cabi, q, step.k_pools[layer], step.v_pools[layer], step.block_table, step.seq_lens, split_k=step.split_k,
        scale=128 ** -0.5, partials=step.partials, out=out, kv_scales=scales(layer)) for layer in range(launches)]
    kernel_name, ctas_per_head = cabi.fused_kernel_plan(arg_sets[0])
    ctas = ctas_per_head * 2
    stamps = [torch.zeros((ctas, 10), dtype=torch.int64, device=device) for _ in range(launches)]
    lib = cabi.library()

    def run():
        stream = cabi.stream_pointer(device)
        for layer in range(launches):
            cabi.check(lib.qf_grouped_splitk_persistent_timeline(
                ctypes.byref(arg_sets[layer]), stamps[layer].data_ptr(), stream))

    side = torch.cuda.Stream(device)
    side.wait_stream(torch.cuda.current_stream(device))
    with torch.cuda.stream(side):
        run()
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        run()
    torch.cuda.current_stream(device).wait_stream(side)
    for _ in range(max(args.warmup, 3)):
        graph.replay()
    torch.cuda.synchronize()
    tables = [t.cpu().double() for t in stamps]
    origin = tables[0][tables[0][:, 5] > 0, 0].min()  # CTAs without work leave no stamps
    names = ("entry", "share_known", "ids_known", "first_tile", "exit")
    rows = []
    for table in tables:
        busy = table[:, 5] > 0
        record = {name: [round(float(((table[busy, i] - origin) / 1e3).min()), 2),
                         round(float(((table[busy, i] - origin) / 1e3).mean()), 2),
                         round(float(((table[busy, i] - origin) / 1e3).max()), 2)] for i, name in enumerate(names)}
        exits = (table[busy, 4] - table[busy, 4].min()) / 1e3
        record["exit_histogram_1us_bins_from_earliest"] = torch.histc(exits.float(), bins=12, min=0, max=12).int().tolist()
        record["units_per_cta_min_max"] = [int(table[busy, 5].min()), int(table[busy, 5].max())]
        full = table[busy, 5] == table[busy, 5].max()
        record["exit_spread_us_of_ctas_with_a_full_share"] = round(
            float((table[busy, 4][full].max() - table[busy, 4][full].min()) / 1e3), 2)
        stream_phase = (table[busy, 4] - table[busy, 3]) / 1e3
        pieces = table[busy, 6]
        record["stream_phase_us_by_pieces_of_warp0"] = {
            int(n): [int((pieces == n).sum()), round(float(stream_phase[pieces == n].mean()), 2),
                     round(float(stream_phase[pieces == n].max()), 2)] for n in sorted(set(pieces.tolist()))}
        if kernel_name.endswith("(solo)"):
            # columns 7 to 9 of the solo variant: warp 0's wait at the barrier at the CTA's end, its merge
            # there (if it had one), and whether it had one
            record["warp0_wait_at_the_end_barrier_us_mean_max"] = [
                round(float(table[busy, 7].mean() / 1e3), 3), round(float(table[busy, 7].max() / 1e3), 3)]
            merging = table[busy, 9] > 0
            record["warp0_end_merges"] = int(merging.sum())
            record["warp0_us_per_end_merge"] = round(float(table[busy, 8][merging].mean() / 1e3), 3) if merging.any() else None
        else:
            record["warp0_deposit_us_per_piece"] = round(float(table[busy, 7].sum() / max(float(pieces.sum()), 1.0) / 1e3), 3)
            record["warp0_us_per_merge"] = round(float(table[busy, 8].sum() / max(float(table[busy, 9].sum()), 1.0) / 1e3), 3)
        rows.append(record)
    print(json.dumps({"op": "cta_timeline", "workload": args.workload, "kernel": kernel_name,
                      "uniform_context": args.uniform_context or None,
                      "batch": workload.batch, "split_k": step.split_k, "ctas": ctas, "launches": rows,
                      "columns": "min / mean / max microseconds over the CTAs, from the first launch's first entry",
                      "device_status": cabi.device_status()}))


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    if args.warmup < 3:
        args.warmup = 3
    if args.op == "layer_glue":
        if rank == 0:
            run_layer_glue(args)
        return
    if args.op == "cta_timeline":
        if rank == 0:
            run_cta_timeline(args)
        return
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    timer = Timer(device, local_rank, distributed)

    package = entry.load_package()
    oracle = entry.load_oracle()  # the checker of the parity gate and the CPU baseline's port; never timed as the product
    workload = package.workloads.build_workload(
        args.workload, rank=rank, world_size=world, scaling=args.scaling, seed=args.seed,
        layers=args.layers or None)
    package.cabi.set_tuning(force_generic=KERNEL_MODES[args.kernel])  # read at launch (and capture) time
    step = package.decode_step.DecodeStep(workload, device, split_k=args.split_k or None, package=package,
                                          fused_write=(not args.unfused_write and args.kernel in ("auto", "persistent_mma", "persistent_mma_solo")
                                                       and not (workload.fp8 and args.kernel == "persistent_mma")))  # FP8: folded in the solo variant only
    step.load_packed_rows()

    # ---- parity gate: nothing is timed unless the timed call gives the oracle's answers ----
    try:
        parity = preflight(package, oracle, step)
    except ParityError as error:
        print(json.dumps({"metric": METRIC, "value": None, "unit": UNIT, "n_gpus": world,
                          "refused": "parity gate", "detail": str(error)}))
        raise SystemExit(1)

    step.capture(warmup=2)
    step.host_buffers()
    torch.cuda.synchronize()

    # ---- device-resident throughput (graph replay) --------------------------------
    for _ in range(args.warmup):
        step.replay()
    with ClockSampler(local_rank) as sampler:
        across, own = timer.per_step(step.replay, args.steps, args.repeats)
        # The timed regions last a few tens of milliseconds each, about a sampling period:
        # keep the identical load running (untimed) until the sampler has seen it.
        deadline = time.perf_counter() + 0.5
        while time.perf_counter() < deadline:
            for _ in range(20):
                step.replay()
            torch.cuda.synchronize(device)
    clocks = sampler.summary()
    ms_per_step = statistics.median(across)

    # ---- end to end from pinned host buffers ---------------------------------------
    step.capture_from_host()  # copies of layer l + 1 overlap layer l inside one graph
    for _ in range(args.warmup):
        step.run_from_host()
    e2e_across, _ = timer.per_step(step.run_from_host, args.steps, args.repeats)
    e2e_ms = statistics.median(e2e_across)

    # ---- dominant kernel: one partial-pass launch per layer, in one graph ----------
    roofline = None
    if workload.batch:
        roofline = partial_pass_leg(package, step, timer, args.steps, args.repeats, args.seed, world)
        step_bytes = step_algorithmic_bytes(package, step, roofline)
        roofline["whole_step"] = {
            "algorithmic_bytes": step_bytes, "achieved": step_bytes / (statistics.median(own) * 1e-3) / 1e9,
            "frac": step_bytes / (statistics.median(own) * 1e-3) / 1e9 / roofline["peak"],
            "note": "bytes the step's launches move (partial pass, pieces re-read by the combine, result rows) "
                    "over this rank's step time"}
    if distributed:
        # every rank's own bytes over its own time (gathered after the timed regions)
        mine = {"rank": rank, "kv_tokens": int(workload.seq_lens.sum()), "ms_per_step": statistics.median(own),
                "partial_us": roofline["us_per_launch"] if roofline else None,
                "gbs": roofline["achieved"] if roofline else None, "frac": roofline["frac"] if roofline else None}
        per_rank = [None] * world
        dist.all_gather_object(per_rank, mine)
        if roofline:
            roofline["per_rank"] = per_rank
            roofline["min_frac_over_ranks"] = min(r["frac"] for r in per_rank if r["frac"] is not None)

    status = package.cabi.device_status()
    config = workload_config(package, args.workload, workload, world, args.scaling)
    kernel_launches_per_step = step.kernel_launches_per_step
    fused_write, split_k, fp8 = step.fused_write, step.split_k, step.fp8
    local_batch = torch.tensor([workload.batch], dtype=torch.int64, device=device)
    if distributed:
        dist.all_reduce(local_batch)
    global_batch = int(local_batch.item())

    baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not fp8:
        baseline = cpu_baseline(package, oracle, workload, args.seed, args.cpu_seconds)
    h2d_bytes, d2h_bytes = step.h2d_bytes(), step.d2h_bytes()
    del step
    release()

    # ---- the other configurations (one GPU) and the by-sequence split of the batch of 256 ----
    others, strong = None, None
    if not args.no_workloads and args.workload == "decode_b64" and args.scaling == "weak" and not args.layers:
        sweep_record = None
        if world == 1:
            others = {}
            for name in OTHER_WORKLOADS:
                try:
                    record, other_workload, other_step = measure_workload(
                        package, oracle, name, device, timer, args, 1, 0)
                except ParityError as error:
                    print(json.dumps({"metric": METRIC, "value": None, "unit": UNIT, "n_gpus": world,
                                      "refused": "parity gate", "detail": str(error)}))
                    raise SystemExit(1)
                del other_step, other_workload
                release()
                others[name] = record
                if name == "sweep_b256":
                    sweep_record = record
        if sweep_record is None:
            sweep_record, _, sweep_step = measure_workload(
                package, oracle, "sweep_b256", device, timer, args, world, rank, scaling="strong")
            del sweep_step
            release()
        mine = {"rank": rank, "sequences": sweep_record["config"]["batch_per_gpu"],
                "kv_tokens": sweep_record["roofline"]["kv_bytes_per_launch"] // 1024 if "roofline" in sweep_record else 0,
                "ms_per_step": sweep_record.get("own_ms_per_step"),
                "partial_us": sweep_record["roofline"]["us_per_launch"] if "roofline" in sweep_record else None,
                "gbs": sweep_record["roofline"]["achieved"] if "roofline" in sweep_record else None,
                "frac": sweep_record["roofline"]["frac"] if "roofline" in sweep_record else None,
                "parity": sweep_record.get("parity", {}).get("passed")}
        per_rank = [mine]
        if distributed:
            per_rank = [None] * world
            dist.all_gather_object(per_rank, mine)
        slowest = max(r["ms_per_step"] for r in per_rank if r["ms_per_step"])
        tokens = [r["kv_tokens"] for r in per_rank]
        strong = {
            "workload": "sweep_b256", "global_batch": 256, "partition": "sharding.partition_sequences(..., 'snake')",
            "n_gpus": world, "ms_per_step": slowest, "tokens_per_s": 256 / (slowest * 1e-3),
            "imbalance": max(tokens) / (sum(tokens) / len(tokens)) if sum(tokens) else 1.0,
            "bounded_by_rank": max(per_rank, key=lambda r: r["ms_per_step"] or 0)["rank"],
            "min_frac_over_ranks": min(r["frac"] for r in per_rank if r["frac"] is not None),
            "per_rank": per_rank,
        }

    if rank == 0:
        line = {
            "metric": METRIC, "value": global_batch / (ms_per_step * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "ms_per_step_spread": spread(across),
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f16 storage, f32 accumulate" if not fp8 else "e4m3 storage, f32 accumulate",
            "data": "synthetic",
            "config": config,
            "implementation": {
                "split_k": split_k, "kernel": args.kernel, "fused_write": fused_write,
                "timing": "CUDA graph replay; %d regions of %d replays, each between barriers, CUDA events on the "
                          "launching stream, max over ranks; the median region is the value" % (args.repeats, args.steps),
                "clock_sampling": "nvidia-smi every 50 ms over the timed regions and 0.5 s more of the same replays",
            },
            "parity": parity,
            "e2e": {"value": global_batch / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "ms_per_step_spread": spread(e2e_across),
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": d2h_bytes},
            "gpu_launches": args.steps * kernel_launches_per_step,
            "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            "roofline": roofline,
            "cpu_baseline": baseline,
            "workloads": others,
            "strong_sweep_b256": strong,
            "device_status": status,
        }
        print(json.dumps(line))
    if distributed:
        dist.barrier(device_ids=[local_rank])
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
