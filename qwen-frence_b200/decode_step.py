"""One decode step of the hot path over all layers: for every layer, the packed-QKV
RoPE + paged KV write, then GQA paged decode attention over the block tables.

This is the loop body of the reference's graph decoder restricted to the two
stages this package owns (engine/graph/paged_graph_decoder.py:234-289):
the write for position p precedes, on the same stream, the attention that
reads seq_len = p + 1 tokens.  The projections around it (QKV GEMM, o_proj,
MLP) are outside the path; the packed QKV rows arrive as an input.

`DecodeStep` owns the device state of one rank (per-layer pools, static
metadata buffers at fixed addresses, partial buffers), can capture the whole
step in a CUDA graph as the reference engine does
(engine/graph/paged_graph_decoder.py:124-142), and offers `run_from_host`,
the end-to-end call that takes pinned host buffers, copies them in, replays
and copies the result out.  `capture_from_host` records that whole call as one
graph in which the host-to-device copy of layer l + 1's rows runs on a second
stream while layer l computes.
"""

from __future__ import annotations

import torch

from . import kv_layout


class DecodeStep:
    # sequences up to which the RoPE / KV write is folded into the partial pass: the persistent
    # kernels' batch limit (measured per 28-layer step, folded against separate: 64 sequences
    # 0.789 / 0.878 ms, 256 log-uniform lengths 2.089 / 2.151, 512 x 100 tokens 0.538 / 0.590)
    FUSED_WRITE_MAX_BATCH = 1024

    def __init__(self, workload, device, *, split_k=None, dtype=torch.float16,
                 fill_pools=True, package=None, fused_write=False):
        import sys

        self.package = package if package is not None else sys.modules[__package__]
        self.workload = workload
        self.device = torch.device(device)
        self.dtype = dtype
        self.fp8 = workload.fp8
        self.layers = workload.layers
        self.batch = workload.batch
        self.split_k = int(split_k) if split_k else kv_layout.plan_split_k(
            max(self.batch, 1), workload.max_context,
            sm_count=torch.cuda.get_device_properties(self.device).multi_processor_count)
        # fused_write: RoPE + KV write inside the attention partial pass (two launches per layer
        # instead of three) where the tensor-core kernel applies
        self.fused_write = (bool(fused_write) and self.split_k > 1
                            and (fused_write == "always" or self.batch <= self.FUSED_WRITE_MAX_BATCH))
        self.kernel_launches_per_step = self.layers * (2 if self.split_k == 1 or self.fused_write else 3)
        self.rope_table = None
        if self.fused_write:  # (cos, sin) of every position the block tables can hold
            with torch.cuda.device(self.device):
                self.rope_table = self.package.build_rope_table(
                    workload.block_table.shape[1] * kv_layout.PAGE_SIZE, device=self.device)

        shape = (workload.num_pages, kv_layout.PAGE_SIZE, kv_layout.KV_HEADS, kv_layout.HEAD_DIM)
        pool_dtype = torch.uint8 if self.fp8 else dtype
        self.k_pools = [torch.empty(shape, dtype=pool_dtype, device=self.device) for _ in range(self.layers)]
        self.v_pools = [torch.empty(shape, dtype=pool_dtype, device=self.device) for _ in range(self.layers)]
        self.k_scales = self.v_scales = None
        if self.fp8:
            scale_shape = (workload.num_pages, kv_layout.KV_HEADS)
            self.k_scales = [torch.ones(scale_shape, dtype=torch.float32, device=self.device) for _ in range(self.layers)]
            self.v_scales = [torch.ones(scale_shape, dtype=torch.float32, device=self.device) for _ in range(self.layers)]
        if fill_pools:
            self._fill_pools()

        # Static buffers: a captured graph reads these addresses on every replay.
        b = self.batch
        self.packed = torch.zeros((self.layers, b, 2048), dtype=dtype, device=self.device)
        # The four metadata tensors are views of ONE byte buffer (slot mapping first: it is
        # the 8-byte type), so that the end-to-end call brings them in with one copy.
        self._metadata = self._pack_metadata(workload, self.device)
        self.positions, self.seq_lens, self.slot_mapping, self.block_table = self._metadata_views(
            self._metadata, workload)
        for name in ("positions", "seq_lens", "slot_mapping", "block_table"):
            getattr(self, name).copy_(getattr(workload, name))
        # attention output of the last layer (what the step hands on); under capture
        # it lives at a fixed address in the graph's private pool
        self.result = torch.zeros((b, kv_layout.Q_HEADS, kv_layout.HEAD_DIM), dtype=dtype, device=self.device)
        k = self.split_k
        self.partials = None
        if k > 1:
            self.partials = (
                torch.empty((b, k, kv_layout.Q_HEADS, kv_layout.HEAD_DIM), dtype=torch.float32, device=self.device),
                torch.empty((b, k, kv_layout.Q_HEADS), dtype=torch.float32, device=self.device),
                torch.empty((b, k, kv_layout.Q_HEADS), dtype=torch.float32, device=self.device),
            )
        self.graph = None
        self.steps_graph = None
        self.host_graph = None
        self._host = None

    # ------------------------------------------------------------------ setup
    @staticmethod
    def _metadata_layout(workload):
        """(name, dtype, shape, byte offset) of the metadata tensors inside one buffer."""
        layout, offset = [], 0
        for name in ("slot_mapping", "positions", "seq_lens", "block_table"):
            tensor = getattr(workload, name)
            size = tensor.numel() * tensor.element_size()
            layout.append((name, tensor.dtype, tuple(tensor.shape), offset))
            offset += -(-size // 8) * 8
        return layout, max(offset, 8)

    @classmethod
    def _pack_metadata(cls, workload, device, pin=False):
        _, size = cls._metadata_layout(workload)
        return torch.zeros(size, dtype=torch.uint8, device=device, pin_memory=pin)

    @classmethod
    def _metadata_views(cls, buffer, workload):
        layout, _ = cls._metadata_layout(workload)
        views = {}
        for name, dtype, shape, offset in layout:
            count = 1
            for extent in shape:
                count *= extent
            size = count * torch.empty((), dtype=dtype).element_size()
            views[name] = buffer[offset:offset + size].view(dtype).view(shape)
        return views["positions"], views["seq_lens"], views["slot_mapping"], views["block_table"]

    def _fill_pools(self):
        """Random N(0,1)*0.5 K/V in the live pages (the rest of the pool is never
        read); FP8 pools are quantised page by page with the library's quantiser."""
        w = self.workload
        live = w.live_pages.to(self.device)
        generator = torch.Generator(device=self.device).manual_seed(4000 + w.value_seed)
        chunk = 4096
        for layer in range(self.layers):
            for pool, scales in ((self.k_pools[layer], self.k_scales), (self.v_pools[layer], self.v_scales)):
                for start in range(0, live.numel(), chunk):
                    index = live[start:start + chunk]
                    values = torch.randn((index.numel(), *pool.shape[1:]), generator=generator,
                                         device=self.device, dtype=torch.float32).mul_(0.5).to(self.dtype)
                    if self.fp8:
                        bits, scale = self.package.quantize_kv_pool_e4m3(values)
                        pool[index] = bits
                        scales[layer][index] = scale
                    else:
                        pool[index] = values

    def load_packed_rows(self):
        """Setup: fill the static packed-QKV buffer of every layer (untimed)."""
        from . import workloads

        for layer in range(self.layers):
            self.packed[layer].copy_(workloads.packed_qkv_rows(self.workload, layer, self.device, self.dtype))

    # ------------------------------------------------------------------- step
    def layer(self, index):
        """RoPE + KV write, then attention, for one layer, on the current stream."""
        pkg = self.package
        if self.fp8 and self.fused_write:
            out = pkg.packed_qkv_rope_attention_fp8(
                self.packed[index], self.positions, self.slot_mapping, self.k_pools[index], self.v_pools[index],
                self.k_scales[index], self.v_scales[index], self.block_table, self.seq_lens, split_k=self.split_k,
                partials=self._fp8_partials(), rope_table=self.rope_table, require_fused=True)
        elif self.fp8:
            q = pkg.packed_qkv_rope_cache_fp8(
                self.packed[index], self.positions, self.slot_mapping, self.k_pools[index],
                self.v_pools[index], self.k_scales[index], self.v_scales[index])
            out = pkg.grouped_splitk_decode_attention_fp8(
                q, self.k_pools[index], self.v_pools[index], self.k_scales[index], self.v_scales[index],
                self.block_table, self.seq_lens, split_k=self.split_k,
                partials=self._fp8_partials())
        elif self.fused_write:
            out = pkg.packed_qkv_rope_attention(
                self.packed[index], self.positions, self.slot_mapping, self.k_pools[index], self.v_pools[index],
                self.block_table, self.seq_lens, split_k=self.split_k, partials=self.partials,
                rope_table=self.rope_table, require_fused=True)  # a silent fallback would miscount launches
        else:
            q = pkg.packed_qkv_rope_cache(
                self.packed[index], self.positions, self.slot_mapping, self.k_pools[index], self.v_pools[index])
            out = pkg.grouped_splitk_decode_attention(
                q, self.k_pools[index], self.v_pools[index], self.block_table, self.seq_lens,
                split_k=self.split_k, partials=self.partials)
        return out

    def _fp8_partials(self):
        if self.partials is not None:
            return self.partials
        b = self.batch
        self.partials = (
            torch.empty((b, 1, kv_layout.Q_HEADS, kv_layout.HEAD_DIM), dtype=torch.float32, device=self.device),
            torch.empty((b, 1, kv_layout.Q_HEADS), dtype=torch.float32, device=self.device),
            torch.empty((b, 1, kv_layout.Q_HEADS), dtype=torch.float32, device=self.device),
        )
        return self.partials

    def step(self):
        """All layers, eagerly, on the current stream."""
        if self.batch == 0:
            return self.result
        for index in range(self.layers):
            out = self.layer(index)
        self.result = out
        return out

    def capture(self, warmup=3):
        """Warm up on a side stream, then record the whole step into one CUDA graph."""
        if self.batch == 0:
            return None
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                self.step()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            self.step()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        self.graph = graph
        return graph

    def advance(self):
        """Move the step metadata on by one token on the device, in place (no host
        rebuild, no copy): positions and lengths + 1, slots looked up in the block
        table, which must already hold the pages of the coming tokens."""
        if self.batch:
            self.package.advance_decode_state(
                self.positions, self.seq_lens, self.slot_mapping, self.block_table,
                num_pages=self.workload.num_pages)

    def capture_steps(self, count, warmup=1):
        """Record `count` consecutive decode steps, each followed by the device-side
        metadata advance, into one graph -- the shape of the reference's unrolled
        decoder (engine/graph/unrolled_graph_decoder.py:92-130) with its per-step
        metadata tensors replaced by one set advanced in place.  Warm-up runs advance
        the metadata too; it is restored from the workload before recording."""
        if self.batch == 0:
            return None
        stream = torch.cuda.Stream(self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))

        def run():
            for _ in range(count):
                self.step()
                self.advance()

        with torch.cuda.stream(stream):
            for _ in range(warmup):
                run()
            self.reset_metadata()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            run()
        torch.cuda.current_stream(self.device).wait_stream(stream)
        self.steps_graph = graph
        return graph

    def reset_metadata(self):
        """Step metadata back to the workload's first step."""
        for name in ("positions", "seq_lens", "slot_mapping", "block_table"):
            getattr(self, name).copy_(getattr(self.workload, name))

    def replay(self):
        if self.batch == 0 or self.graph is None:
            return self.step()
        self.graph.replay()
        return self.result

    # ------------------------------------------------------------- end to end
    def host_buffers(self):
        """Pinned host staging: the step's inputs and its result."""
        if self._host is None:
            pin = dict(pin_memory=True)
            metadata = self._pack_metadata(self.workload, "cpu", pin=True)
            positions, seq_lens, slot_mapping, block_table = self._metadata_views(metadata, self.workload)
            self._host = dict(
                packed=torch.empty(self.packed.shape, dtype=self.dtype, **pin),
                metadata=metadata, positions=positions, seq_lens=seq_lens, slot_mapping=slot_mapping,
                block_table=block_table,
                out=torch.empty(self.result.shape, dtype=self.dtype, **pin),
            )
            for key in ("packed", "positions", "seq_lens", "slot_mapping", "block_table"):
                self._host[key].copy_(getattr(self, key))
        return self._host

    def h2d_bytes(self):
        host = self.host_buffers()  # what run_from_host copies: the rows and the metadata buffer
        return sum(host[k].numel() * host[k].element_size() for k in ("packed", "metadata"))

    def d2h_bytes(self):
        host = self.host_buffers()
        return host["out"].numel() * host["out"].element_size()

    def capture_from_host(self, warmup=2):
        """Record the end-to-end call as ONE graph with the copies pipelined: a copy
        stream brings in the metadata and then the packed rows a few layers at a time,
        the compute stream waits only for the rows of the layer it is about to run, and
        the result goes back to pinned memory at the end.  Same reads and writes as the
        sequential `run_from_host`; the host buffers are read when the graph replays."""
        if self.batch == 0:
            return None
        host = self.host_buffers()
        main = torch.cuda.Stream(self.device)
        copier = torch.cuda.Stream(self.device)

        # Rows travel in a few copies of growing size (1, 3, 9, ... layers): the first one
        # is short, so the first layer starts early, and there are few cross-stream
        # dependencies, each of which costs the waiting kernel its early start.
        chunks, first = [], 0
        while first < self.layers:
            size = min(max(1, len(chunks) and 3 * chunks[-1][1]), self.layers - first)
            chunks.append((first, size))
            first += size

        def record():
            copier.wait_stream(main)  # fork
            with torch.cuda.stream(copier):
                self._metadata.copy_(host["metadata"], non_blocking=True)  # all four tensors at once
                arrived = {}
                for start, size in chunks:
                    self.packed[start:start + size].copy_(host["packed"][start:start + size], non_blocking=True)
                    arrived[start] = torch.cuda.Event()
                    arrived[start].record(copier)
            out = None
            for index in range(self.layers):
                if index in arrived:
                    main.wait_event(arrived[index])  # metadata was copied before the first rows
                out = self.layer(index)
            main.wait_stream(copier)  # join
            self.result = out
            host["out"].copy_(out, non_blocking=True)

        main.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(main):
            for _ in range(warmup):
                record()
        main.synchronize()
        copier.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=main):
            record()
        torch.cuda.current_stream(self.device).wait_stream(main)
        self.host_graph = graph
        return graph

    def run_from_host(self):
        """Host inputs in, result out: H2D copies of the step's inputs from pinned
        memory, the step, D2H of the last layer's attention output.  One pipelined
        graph when `capture_from_host` was called, else copies, `replay`, copy.
        Asynchronous on the current stream; the caller synchronises."""
        host = self.host_buffers()
        if self.host_graph is not None:
            self.host_graph.replay()
            return host["out"]
        self.packed.copy_(host["packed"], non_blocking=True)
        self._metadata.copy_(host["metadata"], non_blocking=True)
        result = self.replay()
        host["out"].copy_(result, non_blocking=True)
        return host["out"]
