"""Drop-in proof through the reference's OWN callers: its decode layer loop
(`graph_decode_forward`, engine/graph/paged_graph_decoder.py:173-347) and its CUDA-graph
decoder (`CUDAGraphDecoder`, :32-169) run unmodified, with the one documented change --
`baseline/kernel_dispatch.py`'s `_KERNEL_DIR` pointing at this package's `custom_kernels/` --
on a Qwen2.5-1.5B-geometry model with random weights, its own `PagedKVCache` and its own
`build_decode_step_inputs`.

The reference files are the unmodified copies that `oracle/build_ref.py` stages under
oracle/_ref/ (they are imported, not read from the reference tree, which does not exist on
the GPU machine).  The expected logits come from the same loop with no custom kernel: the
reference's torch RoPE + `index_copy_` branch and its `decode_attention_sdpa`."""

from __future__ import annotations

import copy
import importlib.util
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

REPO_ROOT = Path(__file__).resolve().parents[1]
REF_DIR = REPO_ROOT / "oracle" / "_ref"
KERNEL_DIR = REPO_ROOT / "qwen-frence_b200" / "custom_kernels"
NEEDED = ("baseline/naive_forward.py", "baseline/kernel_dispatch.py", "engine/kvcache/paged_kv_cache.py",
          "engine/kvcache/paged_decode_attention.py", "engine/graph/paged_graph_decoder.py")


@pytest.fixture(scope="module")
def reference():
    if not all((REF_DIR / name).is_file() for name in NEEDED):
        pytest.skip("oracle/_ref/ is not staged (run `python oracle/build_ref.py` where the reference tree is)")
    sys.dont_write_bytecode = True
    for sub in ("baseline", "engine/kvcache", "engine/graph"):
        path = str(REF_DIR / sub)
        if path not in sys.path:
            sys.path.insert(0, path)

    def load(relative, name):
        if name in sys.modules and getattr(sys.modules[name], "__file__", "").startswith(str(REF_DIR)):
            return sys.modules[name]
        spec = importlib.util.spec_from_file_location(name, REF_DIR / relative)
        module = importlib.util.module_from_spec(spec)
        sys.modules[name] = module
        spec.loader.exec_module(module)
        return module

    modules = {
        "kv_cache": load("baseline/kv_cache.py", "kv_cache"),
        "naive_forward": load("baseline/naive_forward.py", "naive_forward"),
        "kernel_dispatch": load("baseline/kernel_dispatch.py", "kernel_dispatch"),
        "paged_decode_attention": load("engine/kvcache/paged_decode_attention.py", "paged_decode_attention"),
        "paged_forward": load("engine/kvcache/paged_forward.py", "paged_forward"),
        "paged_kv_cache": load("engine/kvcache/paged_kv_cache.py", "paged_kv_cache"),
        "decoder": load("engine/graph/paged_graph_decoder.py", "paged_graph_decoder"),
    }
    # the one change a maintainer makes: the loader's kernel directory
    dispatch = modules["kernel_dispatch"]
    dispatch._KERNEL_DIR = KERNEL_DIR
    dispatch._load.cache_clear()
    return modules


def _setup(reference, device, lengths, layers=2, seed=0):
    """Model (random weights, packed projections), the reference's paged cache holding
    `lengths[b]` tokens per sequence (the last one is the token of this step), metadata."""
    naive, paged = reference["naive_forward"], reference["paged_kv_cache"]
    torch.manual_seed(seed)
    cfg = naive.Qwen2Config(n_layers=layers, vocab=2048)
    model = naive.Model(cfg)
    for parameter in model.parameters():  # checkpoint-like magnitudes (no checkpoint is available offline)
        if parameter.dim() >= 2:
            torch.nn.init.normal_(parameter, std=0.02)
        elif parameter.numel() != cfg.d_model:  # projection biases; the RMSNorm weights stay at one
            torch.nn.init.normal_(parameter, std=0.02)
    model = model.to(device=device, dtype=torch.float16).eval()
    model.pack_projections_()
    batch = len(lengths)
    pages = sum(-(-n // 16) for n in lengths) + 8
    cache = paged.PagedKVCache(cfg, batch, pages, 16, device, torch.float16)
    generator = torch.Generator().manual_seed(seed + 1)
    cache.free_blocks = torch.randperm(pages, generator=generator).tolist()  # permuted block tables
    cache.allocate_block(list(lengths))
    for layer in range(layers):
        for pool in (cache.k_pool[layer], cache.v_pool[layer]):
            pool.copy_((torch.randn(pool.shape, generator=generator) * 0.5).half())
    max_blocks = max(len(table) for table in cache.block_tables) + 3
    tokens = torch.randint(0, cfg.vocab, (batch,), generator=generator).tolist()
    inputs = reference["decoder"].build_decode_step_inputs(cache, tokens, max_blocks, device)
    return cfg, model, cache, max_blocks, inputs


def _clone_cache(cache):
    clone = copy.copy(cache)
    clone.k_pool = [pool.clone() for pool in cache.k_pool]
    clone.v_pool = [pool.clone() for pool in cache.v_pool]
    return clone


@torch.no_grad()
def test_reference_layer_loop_and_graph_decoder_drive_these_kernels(reference, package, cuda_device):
    decoder = reference["decoder"]
    lengths = [1100, 37, 2049, 513, 1, 16, 17, 1500]
    cfg, model, cache, max_blocks, inputs = _setup(reference, cuda_device, lengths)
    slots = inputs[4]

    # (a) the reference's own torch path: RoPE tables + index_copy_ + decode_attention_sdpa
    plain_cache = _clone_cache(cache)
    original = decoder.paged_decode_attention_dispatch
    decoder.paged_decode_attention_dispatch = (
        lambda q, k, v, table, lens, **_: reference["paged_decode_attention"].decode_attention_sdpa(q, k, v, table, lens))
    try:
        expected = decoder.graph_decode_forward(model, plain_cache, *inputs)
    finally:
        decoder.paged_decode_attention_dispatch = original

    # (b) the same loop, unmodified, on this package's kernels: packed-QKV RoPE / cache
    # epilogue, then grouped split-K attention chosen by the reference's own policy table
    calls = {}
    dispatch = reference["kernel_dispatch"]
    for name in ("packed_qkv_rope_cache", "paged_decode_grouped_splitk", "paged_decode_native_grouped",
                 "rope_kv_write"):
        module = dispatch._load(name)
        assert Path(module.__file__).parent == KERNEL_DIR  # the drop-in files, not the reference's Triton ones
        calls[name] = module
    ours_cache = _clone_cache(cache)
    logits = decoder.graph_decode_forward(
        model, ours_cache, *inputs, decode_attention_policy="splitk", max_decode_context_length=4096,
        enable_packed_qkv_rope_cache=True)
    assert logits.shape == expected.shape == (len(lengths), 1, cfg.vocab)
    # the reference's own logit gate for this fusion (experiments/model/benchmark_native_decode_rope_kv.py:22-23)
    torch.testing.assert_close(logits.float(), expected.float(), atol=0.05, rtol=0.01)
    for layer in range(cfg.n_layers):
        # V placement bit-exact where both runs saw the same hidden state (layer 0; later layers
        # inherit the last-bit differences of the layers before them: same slots, close values);
        # K within the bound the reference holds its own fused write to
        if layer == 0:
            assert torch.equal(ours_cache.v_pool[layer], plain_cache.v_pool[layer])
        changed = (ours_cache.v_pool[layer] != cache.v_pool[layer]).view(-1, 256).any(dim=1).nonzero().flatten()
        assert set(changed.tolist()) <= set(slots.tolist())  # nothing but the step's slots was written
        torch.testing.assert_close(ours_cache.v_pool[layer].float(), plain_cache.v_pool[layer].float(),
                                   atol=2e-2, rtol=2e-2)
        torch.testing.assert_close(ours_cache.k_pool[layer].view(-1, 2, 128)[slots].float(),
                                   plain_cache.k_pool[layer].view(-1, 2, 128)[slots].float(), atol=2e-2, rtol=2e-2)

    # (c) native decode layout write + native grouped attention (the reference's other two entry points)
    native_cache = _clone_cache(cache)
    native = decoder.graph_decode_forward(
        model, native_cache, *inputs, decode_attention_policy="native_grouped", max_decode_context_length=4096,
        enable_native_decode_qkv_postprocess=True)
    torch.testing.assert_close(native.float(), expected.float(), atol=0.05, rtol=0.01)

    # (d) the reference's CUDA-graph decoder captures the step on these kernels and replays it
    graph_cache = _clone_cache(cache)
    graphed = decoder.CUDAGraphDecoder(
        model, graph_cache, len(lengths), max_blocks, cuda_device, torch.float16,
        decode_attention_policy="splitk", max_decode_context_length=4096,
        enable_packed_qkv_rope_cache=True).capture()
    for pool, source in zip(graph_cache.k_pool + graph_cache.v_pool, cache.k_pool + cache.v_pool):
        pool.copy_(source)  # capture's warm-up wrote slot zero
    replayed = graphed.decode(*inputs)
    torch.cuda.synchronize()
    assert torch.equal(replayed, logits)
    assert package.cabi.device_status() == 0
