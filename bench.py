"""Benchmark of the decode-step attention hot path (fused RoPE + paged KV write, then
GQA paged decode attention with split-K combine, over all 28 layers).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--split-k S]
    python bench.py --impl reference ...        # the CPU implementation, same metric
    python bench.py --op layer_glue             # the small kernels either side of the path

A step is one pass of the hot path over one batch of synthetic input: for every
layer, the packed-QKV RoPE + KV write and the attention over the block tables.
Rank 0 prints ONE JSON line.

  value      decode tokens/s of the whole job with inputs resident in HBM: the step
             is replayed from one CUDA graph, timed with CUDA events on the
             launching stream between barriers, max over ranks.
  e2e        the same metric through DecodeStep.run_from_host: per step the packed
             QKV rows and the metadata are copied from pinned host memory, the step
             runs and the result is copied back, all inside the timed region (one
             graph in which the copy of layer l + 1's rows overlaps layer l).
  roofline   achieved HBM bandwidth of the dominant kernel (the attention partial
             pass): its algorithmic bytes per launch divided by its average launch
             time, measured here with CUDA events over a graph of one launch per
             layer (28 different pools, 3.9 GB: nothing is served from L2).
  cpu_baseline  the C oracle (a port of the reference's PyTorch path) on the host
             cores, on a bounded sample; reported, not a target.

With N > 1 (torchrun) every rank owns a full batch of its own sequences and their
KV pages (weak scaling, `--scaling strong` shards one global batch by sequence
instead); no collective runs inside the timed region.
"""

from __future__ import annotations

import argparse
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
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the dominant kernel, from the
# ncu capture summarised in profiles/ (same per-launch workload as a full-size launch: one
# layer of the named workload at seed 0).  Workloads without a capture report null.
NCU_TRAFFIC_BYTES_PER_LAUNCH = {
    ("decode_b64", 0, "decode_mma_kernel"): 137.52e6 + 4.00e6,          # RoPE / KV write as its own kernel
    ("decode_b64", 0, "decode_mma_kernel+rope"): 137.60e6 + 3.85e6,     # the default: write folded in
    ("decode_b64", 0, "decode_partial_kernel"): 137.92e6 + 5.0e6,
}


# --kernel -> qf_set_tuning mode: profiling and A/B runs of the other partial-pass kernels
KERNEL_MODES = {"auto": 0, "partitioned": 2, "persistent_cuda_core": 3, "persistent_mma": 4}


def parse_args():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("b200", "reference"), default="b200")
    parser.add_argument("--workload", default="decode_b64")
    parser.add_argument("--op", choices=("decode_step", "layer_glue"), default="decode_step",
                        help="layer_glue: residual-add + RMSNorm and the device-side metadata advance\n"
                             "(one GPU; prints its own JSON line)")
    parser.add_argument("--scaling", choices=("weak", "strong"), default="weak")
    parser.add_argument("--split-k", type=int, default=0, help="0: plan from host bounds")
    parser.add_argument("--layers", type=int, default=0, help="0: the workload's own (28)")
    parser.add_argument("--cpu-seconds", type=float, default=12.0, help="budget of the CPU baseline leg")
    parser.add_argument("--no-cpu-baseline", action="store_true")
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
    tensor_core = kernel == "decode_mma_kernel"
    _, pieces = package.kv_layout.persistent_schedule(
        lengths, split_k=split_k, ctas_per_head=ctas_per_head, unit_tokens=16 if tensor_core else 32,
        overhead_units=package.kv_layout.TENSOR_CORE_PIECE_OVERHEAD if tensor_core else 0)
    return total + 2 * len(pieces) * 6 * 130 * 4


def cpu_baseline(oracle, workload, packed_row, k_pool, v_pool, budget_seconds):
    """Time the oracle on one layer of the full batch (all host threads), repeat within
    the budget, scale the layer time to the step's layer count."""
    import torch

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    times = []
    deadline = time.perf_counter() + budget_seconds
    while len(times) < 3 or (time.perf_counter() < deadline and len(times) < 50):
        start = time.perf_counter()
        q = oracle.packed_qkv_rope_cache(packed_row, workload.positions, workload.slot_mapping, k_pool, v_pool)
        oracle.paged_attention(q, k_pool, v_pool, workload.block_table, workload.seq_lens)
        times.append(time.perf_counter() - start)
        if len(times) >= 3 and time.perf_counter() > deadline:
            break
    layer_seconds = statistics.median(times)
    return {
        "value": workload.batch / (layer_seconds * LAYERS),
        "unit": UNIT,
        "cores": cores,
        "kind": "port",
        "sample": (f"C/OpenMP oracle, full batch of {workload.batch} sequences, 1 of {LAYERS} layers per pass "
                   f"(median of {len(times)} passes, {layer_seconds * 1e3:.1f} ms/layer), scaled x{LAYERS}"),
    }, layer_seconds


def host_layer_inputs(workload, seed):
    """CPU pools and one packed row block for the CPU legs (N(0,1)*0.5, fp16)."""
    import torch

    generator = torch.Generator().manual_seed(5000 + seed)
    shape = (workload.num_pages, 16, 2, 128)
    k_pool = torch.empty(shape, dtype=torch.float16)
    v_pool = torch.empty(shape, dtype=torch.float16)
    live = workload.live_pages
    for pool in (k_pool, v_pool):
        pool.zero_()
        pool[live] = (torch.randn((live.numel(), 16, 2, 128), generator=generator) * 0.5).half()
    packed = (torch.randn(workload.batch, 2048, generator=generator) * 0.5).half()
    return packed, k_pool, v_pool


def run_reference(args, rank, world):
    """--impl reference: the CPU implementation of the path on the host cores.  The
    reference is a Python source tree with no build or install recipe, so what runs
    here is its port (oracle/); every step is one layer pass over the full batch."""
    if rank != 0:
        return
    package = entry.load_package()
    oracle = entry.load_oracle()
    workload = package.workloads.build_workload(args.workload, seed=args.seed)
    if workload.fp8:
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference has no per-page-scale FP8 paged attention to time"}))
        return
    packed, k_pool, v_pool = host_layer_inputs(workload, args.seed)
    for _ in range(max(args.warmup, 1)):
        cpu_baseline(oracle, workload, packed, k_pool, v_pool, 0.0)
    start = time.perf_counter()
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        q = oracle.packed_qkv_rope_cache(packed, workload.positions, workload.slot_mapping, k_pool, v_pool)
        oracle.paged_attention(q, k_pool, v_pool, workload.block_table, workload.seq_lens)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - start > 240:
            break
    layer_seconds = sum(times) / len(times)
    value = workload.batch / (layer_seconds * LAYERS)
    cores = os.cpu_count() or 1
    sample = (f"C/OpenMP port of the reference's PyTorch path; a step is one layer pass over the full batch "
              f"of {workload.batch} sequences ({layer_seconds * 1e3:.1f} ms), scaled x{LAYERS} layers")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": len(times), "warmup": max(args.warmup, 1), "ms_per_step": layer_seconds * LAYERS * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": args.workload, "batch": workload.batch,
                                        "layers": LAYERS, "page_size": 16},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
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
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    package = entry.load_package()
    workload = package.workloads.build_workload(
        args.workload, rank=rank, world_size=world, scaling=args.scaling, seed=args.seed,
        layers=args.layers or None)
    package.cabi.set_tuning(force_generic=KERNEL_MODES[args.kernel])  # read at launch (and capture) time
    step = package.decode_step.DecodeStep(workload, device, split_k=args.split_k or None, package=package,
                                          fused_write=not args.unfused_write and args.kernel in ("auto", "persistent_mma"))
    step.load_packed_rows()
    step.capture(warmup=2)
    host = step.host_buffers()
    torch.cuda.synchronize()

    def barrier():
        if distributed:
            dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()

    def max_over_ranks(milliseconds):
        if not distributed:
            return milliseconds
        tensor = torch.tensor([milliseconds], dtype=torch.float64, device=device)
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        return float(tensor.item())

    def timed(run_once, steps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for _ in range(steps):
            run_once()
        end.record()
        barrier()
        return max_over_ranks(start.elapsed_time(end))

    # ---- device-resident throughput (graph replay) --------------------------------
    for _ in range(args.warmup):
        step.replay()
    with ClockSampler(local_rank) as sampler:
        total_ms = timed(step.replay, args.steps)
        # The timed region lasts a few tens of milliseconds, less than a sampling period
        # or two: keep the identical load running (untimed) until the sampler has seen it.
        deadline = time.perf_counter() + 0.5
        while time.perf_counter() < deadline:
            for _ in range(20):
                step.replay()
            torch.cuda.synchronize(device)
    clocks = sampler.summary()
    ms_per_step = total_ms / args.steps

    # ---- end to end from pinned host buffers ---------------------------------------
    step.capture_from_host()  # copies of layer l + 1 overlap layer l inside one graph
    for _ in range(args.warmup):
        step.run_from_host()
    e2e_ms = timed(step.run_from_host, args.steps) / args.steps

    # ---- dominant kernel: one partial-pass launch per layer, in one graph ----------
    roofline = None
    if workload.batch:
        import ctypes

        cabi = package.cabi
        splitk = package.kernel_module("paged_decode_grouped_splitk")
        fp8 = package.kernel_module("fp8_paged_kv")
        q = torch.randn(workload.batch, 12, 128, device=device).mul_(0.5).to(step.dtype)
        partials = step.partials or step._fp8_partials()
        out = torch.empty_like(q)
        arg_sets = []
        for layer in range(step.layers):
            k_pool, v_pool = step.k_pools[layer], step.v_pools[layer]
            scales = (step.k_scales[layer], step.v_scales[layer]) if step.fp8 else None
            source = q
            if step.fused_write:  # the partial pass reads the layer's packed rows and writes the new K/V rows
                source = step.packed[layer].as_strided((workload.batch, 12, 128), (step.packed.stride(1), 128, 1))
            arg_sets.append(splitk.fill_attention_args(
                cabi, source, k_pool, v_pool, step.block_table, step.seq_lens, split_k=step.split_k,
                scale=128 ** -0.5, partials=partials, out=out, kv_scales=scales))
        del fp8
        lib = cabi.library()

        kernel_name, ctas_per_head = cabi.fused_kernel_plan(arg_sets[0])

        plain_sets = arg_sets
        if step.fused_write:  # the same pass without the write, on rotated queries, for comparison
            plain_sets = [splitk.fill_attention_args(
                cabi, q, step.k_pools[layer], step.v_pools[layer], step.block_table, step.seq_lens,
                split_k=step.split_k, scale=128 ** -0.5, partials=partials, out=out) for layer in range(step.layers)]

        def launch_partials(with_write=True):
            # the partial pass of the fused attention call, without its combine
            stream = cabi.stream_pointer(device)
            for arg in (arg_sets if with_write else plain_sets):
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
            return timed(graph.replay, args.steps) / args.steps / step.layers

        kernel_ms = per_launch_ms(True)
        peak, peak_kind = measured_peak_gbs()
        launch_bytes = partial_kernel_bytes(package, workload, step.split_k, step.fp8, kernel_name,
                                            ctas_per_head)
        without_write = None
        if step.fused_write:
            plain_ms = per_launch_ms(False)
            without_write = {"us_per_launch": plain_ms * 1e3, "algorithmic_bytes_per_launch": launch_bytes,
                             "achieved": launch_bytes / (plain_ms * 1e-3) / 1e9,
                             "frac": launch_bytes / (plain_ms * 1e-3) / 1e9 / peak}
        if step.fused_write:
            # instead of rotated Q (12 x 128 x 2 B, already counted): the packed row (2048 x 2 B), a position
            # and its 512 B of the rotation table are read, the new K and V rows (2 x 2 x 128 x 2 B) written
            launch_bytes += workload.batch * ((2048 - 1536) * 2 + 4 + 512 + 2 * 2 * 128 * 2)
        achieved = launch_bytes / (kernel_ms * 1e-3) / 1e9
        roofline = {
            "bound": "hbm", "kernel": kernel_name, "achieved": achieved, "peak": peak,
            "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
            "frac_of_nominal_8TBs": achieved / NOMINAL_HBM_GBS,
            "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH.get(
                (args.workload, args.seed, kernel_name + ("+rope" if step.fused_write else "")))
            if world == 1 and step.split_k == 10 else None,  # the captured launch used split_k 10
            "fused_write": step.fused_write,
            "same_pass_without_the_write": without_write,
            "algorithmic_bytes_per_launch": launch_bytes, "us_per_launch": kernel_ms * 1e3,
            "kv_bytes_per_launch": package.kv_layout.kv_bytes_per_layer(
                workload.seq_lens.tolist(), elem_bytes=1 if step.fp8 else 2),
        }

    status = package.cabi.device_status()
    local_batch = torch.tensor([workload.batch], dtype=torch.int64, device=device)
    if distributed:
        dist.all_reduce(local_batch)
    global_batch = int(local_batch.item())
    step_bytes = step.layers * package.kv_layout.algorithmic_bytes_per_layer(
        workload.seq_lens.tolist(), split_k=step.split_k, fp8=step.fp8)

    baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not step.fp8:
        oracle = entry.load_oracle()
        packed_cpu = step.packed[0].cpu()
        baseline, _ = cpu_baseline(oracle, workload, packed_cpu, step.k_pools[0].cpu(),
                                   step.v_pools[0].cpu(), args.cpu_seconds)

    if rank == 0:
        line = {
            "metric": METRIC, "value": global_batch / (ms_per_step * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "f16 storage, f32 accumulate" if not step.fp8 else "e4m3 storage, f32 accumulate",
            "data": "synthetic",
            "config": {
                "workload": args.workload, "doc": workload.meta["doc"], "global_batch": global_batch,
                "batch_per_gpu": workload.batch, "layers": step.layers, "page_size": 16,
                "heads": "12q/2kv x 128", "split_k": step.split_k, "parallelism": f"by-sequence x{world}",
                "kernel": args.kernel, "fused_write": step.fused_write,
                "l2": "inputs exceed L2: each step reads %.2f GB of K/V from %d per-layer pools (L2 is 126 MB)"
                      % (step.layers * package.kv_layout.kv_bytes_per_layer(
                          workload.seq_lens.tolist(), elem_bytes=1 if step.fp8 else 2) / 1e9, 2 * step.layers),
                "timing": "CUDA graph replay, CUDA events on the launching stream, max over ranks",
                "clock_sampling": "nvidia-smi every 50 ms over the timed region and 0.5 s more of the same replays",
            },
            "hot_path_gbs": step_bytes / (ms_per_step * 1e-3) / 1e9,
            "e2e": {"value": global_batch / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": step.h2d_bytes(), "d2h_bytes_per_step": step.d2h_bytes()},
            "gpu_launches": args.steps * step.kernel_launches_per_step,
            "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            "roofline": roofline,
            "cpu_baseline": baseline,
            "device_status": status,
        }
        print(json.dumps(line))
    if distributed:
        dist.barrier(device_ids=[local_rank])
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
