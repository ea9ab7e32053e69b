"""Generates tests/golden/*.npz by RUNNING the reference's own Python functions.

    python tests/golden/make_golden.py --reference <path of the qwen-frence tree>

Needs the benjaminW2025/qwen-frence tree on disk (it is imported, unmodified, on
CPU); the GPU test box has no such tree, which is why the vectors are committed.
Every file stores the exact inputs (as bit patterns for 16-bit tensors) and the
outputs of the named reference function, so the tests never regenerate inputs.

Reference functions exercised (paths inside the reference tree):
  experiments/decode/grouped_splitk_validation.py  make_inputs, attention_reference,
                                                   correctness_cases
  engine/kvcache/paged_decode_attention.py         decode_attention_reference,
                                                   decode_attention_sdpa,
                                                   select_splitk_config,
                                                   resolve_decode_attention_policy
  custom_kernels/rope.py                           rope_reference
  baseline/naive_forward.py                        apply_rotary_pos_emb
  engine/kvcache/paged_forward.py                  build_rope_from_positions
  engine/kvcache/paged_kv_cache.py                 PagedKVCache
  engine/graph/paged_graph_decoder.py              build_decode_step_inputs (one step, and
                                                   the consecutive steps of a stable cohort)
  experiments/quant/attention.py                   quantize, dequantize
  custom_kernels/fused_rms.py                      rms_norm_reference
"""

from __future__ import annotations

import argparse
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

GOLDEN_DIR = Path(__file__).resolve().parent


def bits(tensor):
    """16-bit tensors as int16 bit patterns (numpy has no bfloat16)."""
    tensor = tensor.detach().cpu().contiguous()
    if tensor.dtype in (torch.float16, torch.bfloat16):
        return tensor.view(torch.int16).numpy()
    return tensor.numpy()


def load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", required=True, help="path of the benjaminW2025/qwen-frence tree")
    root = Path(parser.parse_args().reference)
    sys.dont_write_bytecode = True
    for sub in ("baseline", "engine/kvcache", "engine/graph", "custom_kernels",
                "experiments/decode", "experiments/quant"):
        sys.path.insert(0, str(root / sub))
    torch.set_num_threads(4)

    validation = load(root / "experiments/decode/grouped_splitk_validation.py", "ref_validation")
    paged = load(root / "engine/kvcache/paged_decode_attention.py", "paged_decode_attention")
    rope_mod = load(root / "custom_kernels/rope.py", "ref_rope")
    naive = load(root / "baseline/naive_forward.py", "naive_forward")
    paged_forward = load(root / "engine/kvcache/paged_forward.py", "paged_forward")
    kv_cache = load(root / "engine/kvcache/paged_kv_cache.py", "paged_kv_cache")
    graph = load(root / "engine/graph/paged_graph_decoder.py", "paged_graph_decoder")
    quant = load(root / "experiments/quant/attention.py", "ref_quant_attention")

    # ------------------------------------------------------------ attention
    cases = {}

    def add_attention_case(name, tensors, options, dtype_name="float16"):
        q, k, v, table, lens = tensors
        expected = validation.attention_reference(q, k, v, table, lens, **options)
        safe_table = table.clone()
        safe_table[safe_table < 0] = 0  # engine oracles index with the padded table
        cases[name] = dict(
            q=bits(q), k=bits(k), v=bits(v), table=bits(table), lens=bits(lens),
            scale=np.float32(options.get("scale", q.shape[-1] ** -0.5)),
            dtype=dtype_name, expected=bits(expected),
            q_stride=np.asarray(q.stride()), v_stride=np.asarray(v.stride()),
        )
        if torch.isfinite(k.float()).all() and (lens > 0).all():
            cases[name]["expected_engine_reference"] = bits(
                paged.decode_attention_reference(q, k, v, safe_table, lens, **options))
            cases[name]["expected_engine_sdpa"] = bits(
                paged.decode_attention_sdpa(q, k, v, safe_table, lens, **options))

    for dtype, dtype_name in ((torch.float16, "float16"), (torch.bfloat16, "bfloat16")):
        tensors = validation.make_inputs([0, 1, 15, 16, 17, 33, 81], dtype=dtype, device="cpu",
                                         strided=True, poison_padding=True, seed=42)
        add_attention_case(f"ragged_strided_matrix_{dtype_name}", tensors, {}, dtype_name)
        for name, tensors, options in validation.correctness_cases(dtype=dtype, device="cpu"):
            add_attention_case(f"{name}_{dtype_name}", tensors, options, dtype_name)
    add_attention_case("graph_replay_70_70", validation.make_inputs([70, 70], device="cpu"), {})
    add_attention_case("preallocated_1_17_81", validation.make_inputs([1, 17, 81], device="cpu"), {})
    add_attention_case("clean_0_1_17_70", validation.make_inputs([0, 1, 17, 70], device="cpu", seed=42), {})
    # engine boundary sweep (correctness/checks/check_paged_decode_attention.py:12-20),
    # inputs built the way check_correctness builds them (seed 0, own block run per sequence)
    for page, lengths in ((16, [1]), (16, [15, 16]), (16, [16, 17]), (16, [1, 15, 16, 17]),
                          (16, [31, 32, 33, 100]), (32, [31, 32, 33, 129])):
        torch.manual_seed(0)
        lens = torch.tensor(lengths, dtype=torch.int32)
        max_blocks = (max(lengths) + page - 1) // page
        table = torch.zeros(len(lengths), max_blocks, dtype=torch.int32)
        for b, length in enumerate(lengths):
            nb = (length + page - 1) // page
            table[b, :nb] = torch.arange(b * max_blocks, b * max_blocks + nb, dtype=torch.int32)
        k = torch.randn(len(lengths) * max_blocks, page, 2, 128, dtype=torch.float16)
        v = torch.randn(len(lengths) * max_blocks, page, 2, 128, dtype=torch.float16)
        q = torch.randn(len(lengths), 12, 128, dtype=torch.float16)
        add_attention_case(f"boundary_page{page}_" + "_".join(map(str, lengths)),
                           (q, k, v, table, lens), {})
    flat = {f"{case}/{key}": value for case, fields in cases.items() for key, value in fields.items()}
    np.savez_compressed(GOLDEN_DIR / "attention_cases.npz", **flat)
    print("attention cases:", len(cases))

    # ----------------------------------------------------------------- rope
    generator = torch.Generator().manual_seed(7)
    rope_cases = {}
    for name, positions in (
        ("pos0", [0, 0, 0]),
        ("small", [1, 2, 3, 17, 512]),
        ("check_custom_kernels", list(range(4096, 4096 + 9))),
        ("large", [8191, 16384, 32767]),
    ):
        rows = len(positions)
        x = torch.randn(rows, 14, 128, generator=generator).mul(0.5).to(torch.float16)
        pos = torch.tensor(positions, dtype=torch.int32)
        # rope_reference wants (batch, heads, seq, dim) with positions (batch, seq)
        as_bhsd = x.permute(1, 0, 2)[None]                               # (1, 14, rows, 128)
        fp32_path = rope_mod.rope_reference(as_bhsd, 1_000_000.0, pos[None].long())
        fp32_path = fp32_path[0].permute(1, 0, 2).contiguous()
        cfg = naive.Qwen2Config()
        cos, sin = paged_forward.build_rope_from_positions(cfg, pos, torch.float16)
        decode_layout = x[:, :, None, :]                                   # (rows, 14, 1, 128)
        fp16_table_path = naive.apply_rotary_pos_emb(decode_layout, cos, sin)[:, :, 0, :]
        rope_cases[name] = dict(x=bits(x), positions=pos.numpy(), expected_fp32_path=bits(fp32_path),
                                expected_fp16_table_path=bits(fp16_table_path.contiguous()))
    flat = {f"{case}/{key}": value for case, fields in rope_cases.items() for key, value in fields.items()}
    np.savez_compressed(GOLDEN_DIR / "rope_cases.npz", **flat)
    print("rope cases:", len(rope_cases))

    # ---------------------------------------- allocator + decode-step metadata
    cfg = naive.Qwen2Config(n_layers=1)
    cache = kv_cache.PagedKVCache(cfg, 4, 64, 16, "cpu", torch.float16)
    trace = []
    cache.allocate_block([5, 16, 17, 1])
    cache.allocate_block([1, 1, 0, 40])
    cache.free(1)
    cache.allocate_block([0, 33, 1, 0])
    cache.truncate(3, 20)
    cache.allocate_block([1, 1, 1, 1])
    max_blocks = 6
    ids, positions, seq_lens, table, slots = graph.build_decode_step_inputs(
        cache, [1, 2, 3, 4], max_blocks, "cpu")
    np.savez_compressed(
        GOLDEN_DIR / "metadata_case.npz",
        cur_lens=np.asarray(cache.cur_lens), free_blocks=np.asarray(cache.free_blocks),
        tables=np.asarray([bt + [-1] * (max_blocks - len(bt)) for bt in cache.block_tables]),
        positions=positions.numpy(), seq_lens=seq_lens.numpy(), block_table=table.numpy(),
        slot_mapping=slots.numpy(), max_blocks=np.int64(max_blocks),
    )
    del trace

    # ------------------------- metadata of consecutive steps of a stable cohort
    # Pages are reserved for the whole run at admission (what the device-side advance of
    # engine/cpp/src/iteration_loop.cpp:500-528 relies on); build_decode_step_inputs is
    # then evaluated at every step's lengths.  Step s + 1 must equal the advance of step s.
    steps, start_lens = 40, [7, 16, 33, 1, 250]
    cache = kv_cache.PagedKVCache(cfg, len(start_lens), 128, 16, "cpu", torch.float16)
    generator = torch.Generator().manual_seed(5)
    cache.free_blocks = [cache.free_blocks[i] for i in torch.randperm(128, generator=generator).tolist()]
    cache.allocate_block([n + steps - 1 for n in start_lens])
    max_blocks = max(len(t) for t in cache.block_tables) + 1
    rows = {"positions": [], "seq_lens": [], "slot_mapping": []}
    for step in range(steps):
        cache.cur_lens = [n + step for n in start_lens]
        _, positions, seq_lens, table, slots = graph.build_decode_step_inputs(
            cache, [0] * len(start_lens), max_blocks, "cpu")
        rows["positions"].append(positions.numpy())
        rows["seq_lens"].append(seq_lens.numpy())
        rows["slot_mapping"].append(slots.numpy())
    np.savez_compressed(
        GOLDEN_DIR / "metadata_steps.npz", block_table=table.numpy(),
        **{key: np.stack(value) for key, value in rows.items()})

    # --------------------------------------- RMSNorm, residual-add + RMSNorm
    # rms_norm_reference is the CPU statement the reference checks its Triton kernel
    # against (custom_kernels/fused_rms.py:137-140, :166-180); the residual form is the
    # model-dtype add followed by it (experiments/decode/benchmark_fa3_fusion_kernels.py:71-78);
    # nn.RMSNorm is what the model runs without custom kernels (baseline/naive_forward.py:59-64).
    fused_rms = load(root / "custom_kernels/fused_rms.py", "ref_fused_rms")
    generator = torch.Generator().manual_seed(21)
    norm_cases = {}
    for name, rows, hidden, dtype, epsilon in (
            ("decode_b16_f16", 16, 1536, torch.float16, 1e-6),
            ("decode_b8_bf16", 8, 1536, torch.bfloat16, 1e-6),
            ("odd_width_f16", 5, 1000, torch.float16, 1e-5),
            ("wide_rows_f16", 2, 8192 + 264, torch.float16, 1e-6),
            ("tiny_values_bf16", 4, 96, torch.bfloat16, 1e-6)):
        residual = torch.randn(rows, hidden, generator=generator).to(dtype)
        branch = torch.randn(rows, hidden, generator=generator).to(dtype)
        weight = torch.randn(hidden, generator=generator).to(dtype)
        if name.startswith("tiny"):
            residual, branch = residual * 1e-3, branch * 1e-3
            residual[0], branch[0] = 0, 0  # a zero row: epsilon alone under the root
        summed = residual + branch
        module = torch.nn.RMSNorm(hidden, eps=epsilon, dtype=dtype)
        with torch.no_grad():
            module.weight.copy_(weight)
            torch_norm = module(summed)
        norm_cases[name] = dict(
            residual=bits(residual), branch=bits(branch), weight=bits(weight), epsilon=np.float64(epsilon),
            dtype="bfloat16" if dtype == torch.bfloat16 else "float16", summed=bits(summed),
            normalized=bits(fused_rms.rms_norm_reference(summed, weight, epsilon)),
            plain=bits(fused_rms.rms_norm_reference(residual, weight, epsilon)),
            torch_rmsnorm=bits(torch_norm))
    np.savez_compressed(GOLDEN_DIR / "rms_norm_cases.npz",
                        **{f"{name}/{key}": value for name, case in norm_cases.items()
                           for key, value in case.items()})
    print("rms norm cases:", len(norm_cases))

    # ------------------------------------------------------- split-K policy
    contexts = [1, 16, 1023, 1024, 1280, 1281, 2048, 4096, 32768]
    policy = {
        "contexts": np.asarray(contexts),
        "split_k": np.asarray([paged.select_splitk_config(c)["split_k"] for c in contexts]),
        "num_stages": np.asarray([paged.select_splitk_config(c)["num_stages"] for c in contexts]),
        "resolved_native": np.asarray(
            [paged.resolve_decode_attention_policy("native_grouped", c) for c in contexts]),
    }
    np.savez_compressed(GOLDEN_DIR / "splitk_policy.npz", **policy)

    # ------------------------------------------------------------- FP8 codec
    all_bytes = torch.arange(256, dtype=torch.int32).to(torch.uint8).reshape(1, 1, 2, 128)
    decoded = quant.dequantize(all_bytes, torch.ones(1, 1, 2))
    generator = torch.Generator().manual_seed(11)
    values = torch.randn(2, 2, 48, 128, generator=generator).mul(0.5).half()
    values[0, 0, 0] = 0
    token_bits, token_scales = quant.quantize(values, "token")
    head_bits, head_scales = quant.quantize(values, "head")
    np.savez_compressed(
        GOLDEN_DIR / "fp8_codec.npz",
        decode_table=bits(decoded.reshape(256)),
        values=bits(values),
        token_bits=token_bits.numpy(), token_scales=token_scales.numpy(),
        head_bits=head_bits.numpy(), head_scales=head_scales.numpy(),
        token_dequant=bits(quant.dequantize(token_bits, token_scales)),
        head_dequant=bits(quant.dequantize(head_bits, head_scales)),
    )

    # --------------------- one decode step through the reference's CPU path
    # B=2 slice of the CPU-runnable configuration: context 512, page 16, pool
    # permuted, new token written with RoPE at position 512, then attention over
    # 513 tokens.  Two reference routes: the engine default (fp16 cos/sin tables,
    # apply_rotary_pos_emb + index_copy_ + decode_attention_sdpa) and the fused
    # kernels' arithmetic (rope_reference fp32 + index_copy_ + attention_reference).
    generator = torch.Generator().manual_seed(0)
    batch, context, pages_per_seq = 2, 512, 33
    pool_pages = batch * pages_per_seq
    k_pool = torch.randn(pool_pages, 16, 2, 128, generator=generator).mul(0.5).half()
    v_pool = torch.randn(pool_pages, 16, 2, 128, generator=generator).mul(0.5).half()
    table = torch.randperm(pool_pages, generator=generator).view(batch, pages_per_seq).int()
    packed = torch.randn(batch, 2048, generator=generator).mul(0.5).half()
    positions = torch.full((batch,), context, dtype=torch.int32)
    seq_lens = positions + 1
    slots = (table[:, context // 16].long() * 16 + context % 16)
    q = packed[:, :1536].view(batch, 12, 128)
    k = packed[:, 1536:1792].view(batch, 2, 128)
    v = packed[:, 1792:].view(batch, 2, 128)
    out = {}
    for route in ("engine_fp16_tables", "fused_fp32"):
        kp, vp = k_pool.clone(), v_pool.clone()
        if route == "engine_fp16_tables":
            cos, sin = paged_forward.build_rope_from_positions(naive.Qwen2Config(), positions, torch.float16)
            q_rot = naive.apply_rotary_pos_emb(q[:, :, None, :], cos, sin)[:, :, 0, :]
            k_rot = naive.apply_rotary_pos_emb(k[:, :, None, :], cos, sin)[:, :, 0, :]
        else:
            q_rot = rope_mod.rope_reference(q.permute(1, 0, 2)[None], 1_000_000.0, positions[None].long())[0].permute(1, 0, 2)
            k_rot = rope_mod.rope_reference(k.permute(1, 0, 2)[None], 1_000_000.0, positions[None].long())[0].permute(1, 0, 2)
        kp.view(-1, 2, 128).index_copy_(0, slots, k_rot.contiguous())
        vp.view(-1, 2, 128).index_copy_(0, slots, v.contiguous())
        if route == "engine_fp16_tables":
            attn = paged.decode_attention_sdpa(q_rot.contiguous(), kp, vp, table, seq_lens)
        else:
            attn = validation.attention_reference(q_rot.contiguous(), kp, vp, table, seq_lens)
        out[f"{route}/q_rot"] = bits(q_rot.contiguous())
        out[f"{route}/k_rows"] = bits(kp.view(-1, 2, 128)[slots])
        out[f"{route}/v_rows"] = bits(vp.view(-1, 2, 128)[slots])
        out[f"{route}/attention"] = bits(attn)
    np.savez_compressed(
        GOLDEN_DIR / "decode_step_b2_ctx512.npz",
        k_pool=bits(k_pool), v_pool=bits(v_pool), table=table.numpy(), packed=bits(packed),
        positions=positions.numpy(), seq_lens=seq_lens.numpy(), slots=slots.numpy(), **out)
    print("wrote", sorted(p.name for p in GOLDEN_DIR.glob("*.npz")))


if __name__ == "__main__":
    main()
