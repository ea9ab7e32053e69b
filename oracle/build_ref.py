"""Stages the reference's own CPU (PyTorch) implementation of the hot path under
oracle/_ref/, so that it can be timed on a machine that has no copy of the
benjaminW2025/qwen-frence tree.

    python oracle/build_ref.py [--reference <tree>] [--force]

Test and benchmark infrastructure only: nothing in the product imports this, and
oracle/_ref/ is git-ignored (it holds unmodified files of another project; they are
never committed, only carried beside the built libraries to the machine that runs
`bench.py --impl reference`).  The files are copied byte for byte, each under its
path inside the reference tree, and listed with their SHA-256 in MANIFEST.json.

What is staged is the PyTorch path the reference runs when no custom kernel is
selected, i.e. the last branch of its decode layer loop
(engine/graph/paged_graph_decoder.py:264-274) followed by the attention it checks its
kernels against:

    build_rope_from_positions   engine/kvcache/paged_forward.py:32-44
    apply_rotary_pos_emb        baseline/naive_forward.py:38-48
    index_copy_ placement       engine/graph/paged_graph_decoder.py:271-274 (two torch
                                calls on the flat pool view; restated in `ReferencePath`)
    decode_attention_sdpa       engine/kvcache/paged_decode_attention.py:293-314
    decode_attention_reference  engine/kvcache/paged_decode_attention.py:268-290
"""

from __future__ import annotations

import argparse
import hashlib
import importlib.util
import json
import os
import shutil
import sys
from pathlib import Path

ORACLE_DIR = Path(__file__).resolve().parent
REF_DIR = ORACLE_DIR / "_ref"
MANIFEST = REF_DIR / "MANIFEST.json"
# where the build machine keeps the reference tree; override with --reference or QF_REFERENCE_TREE
DEFAULT_REFERENCE = Path(os.environ.get("QF_REFERENCE_TREE", "/root/reference"))

# module files the staged functions need at import time (paths inside the reference tree)
REFERENCE_FILES = (
    "baseline/kv_cache.py",
    "baseline/naive_forward.py",
    "engine/kvcache/paged_decode_attention.py",
    "engine/kvcache/paged_prefill_attention.py",
    "engine/kvcache/paged_forward.py",
    # the callers of the path, for the drop-in test (tests/test_gpu_reference_caller.py): the
    # reference's decode layer loop and graph decoder, its page allocator and its kernel loader
    "engine/kvcache/paged_kv_cache.py",
    "engine/graph/paged_graph_decoder.py",
    "baseline/kernel_dispatch.py",
)


def _sha256(path: Path) -> str:
    return hashlib.sha256(path.read_bytes()).hexdigest()


def build_ref(reference: Path | str | None = None, force: bool = False) -> Path | None:
    """Copy REFERENCE_FILES from the reference tree into oracle/_ref/.  Returns the
    directory, or None when neither the tree nor an earlier copy is present."""
    root = Path(reference) if reference is not None else DEFAULT_REFERENCE
    if not root.is_dir():
        return REF_DIR if MANIFEST.is_file() else None
    entries = {}
    for relative in REFERENCE_FILES:
        source = root / relative
        if not source.is_file():
            raise RuntimeError(f"the reference tree at {root} has no {relative}")
        target = REF_DIR / relative
        target.parent.mkdir(parents=True, exist_ok=True)
        if force or not target.is_file() or _sha256(target) != _sha256(source):
            shutil.copyfile(source, target)
        entries[relative] = _sha256(target)
    MANIFEST.write_text(json.dumps({"project": "benjaminW2025/qwen-frence", "files": entries}, indent=1) + "\n")
    return REF_DIR


def available() -> bool:
    return MANIFEST.is_file() and all((REF_DIR / name).is_file() for name in REFERENCE_FILES)


class ReferencePath:
    """The staged reference functions, imported from oracle/_ref/ on CPU tensors."""

    def __init__(self):
        if not available():
            raise RuntimeError("oracle/_ref/ is not staged: run `python oracle/build_ref.py` where the "
                               "reference tree is on disk")
        sys.dont_write_bytecode = True
        for sub in ("baseline", "engine/kvcache"):
            path = str(REF_DIR / sub)
            if path not in sys.path:
                sys.path.insert(0, path)

        def load(relative, name):
            spec = importlib.util.spec_from_file_location(name, REF_DIR / relative)
            module = importlib.util.module_from_spec(spec)
            sys.modules[name] = module
            spec.loader.exec_module(module)
            return module

        self.naive_forward = load("baseline/naive_forward.py", "naive_forward")
        self.paged_decode_attention = load("engine/kvcache/paged_decode_attention.py", "paged_decode_attention")
        self.paged_forward = load("engine/kvcache/paged_forward.py", "paged_forward")
        self.cfg = self.naive_forward.Qwen2Config()

    def layer(self, packed, positions, slot_mapping, k_pool, v_pool, block_table, seq_lens, attention="sdpa"):
        """One layer of the hot path as the reference's decode loop runs it without custom
        kernels: split the packed projection output, RoPE on Q and K with fp16 cos / sin
        tables, place K and V in the pools with index_copy_, attend over the block table."""
        cfg = self.cfg
        rows = packed.shape[0]
        q = packed[:, :1536].view(rows, 1, cfg.n_heads, cfg.d_head).transpose(1, 2)
        k = packed[:, 1536:1792].view(rows, 1, cfg.n_kv_heads, cfg.d_head).transpose(1, 2)
        v = packed[:, 1792:].view(rows, 1, cfg.n_kv_heads, cfg.d_head).transpose(1, 2)
        cos, sin = self.paged_forward.build_rope_from_positions(cfg, positions, packed.dtype)
        q = self.naive_forward.apply_rotary_pos_emb(q, cos, sin)
        k = self.naive_forward.apply_rotary_pos_emb(k, cos, sin)
        k_flat = k_pool.view(-1, cfg.n_kv_heads, cfg.d_head)
        v_flat = v_pool.view(-1, cfg.n_kv_heads, cfg.d_head)
        k_flat.index_copy_(0, slot_mapping, k[:, :, 0, :].contiguous())
        v_flat.index_copy_(0, slot_mapping, v[:, :, 0, :].contiguous())
        attend = (self.paged_decode_attention.decode_attention_sdpa if attention == "sdpa"
                  else self.paged_decode_attention.decode_attention_reference)
        return attend(q[:, :, 0, :], k_pool, v_pool, block_table, seq_lens)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    parser.add_argument("--reference", default=str(DEFAULT_REFERENCE))
    parser.add_argument("--force", action="store_true")
    args = parser.parse_args()
    print(build_ref(args.reference, force=args.force))


if __name__ == "__main__":
    main()
