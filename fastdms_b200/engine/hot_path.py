"""One decode step of the compact-DMS path for a fixed batch, captured as a CUDA graph.

Order of work inside a step (the reference's order: engine/model_runner.py:713-772 prepare_decode,
models/llama.py:138-201 per layer, model_runner.py:681-711 record):

    expiry (all layers)  ->  decode metadata (all layers, live += 1)
    ->  per layer: DMS decision + RoPE + FP8 store + compact attention (one launch when the pools
        are FP8 and head_dim is 64/128, else a store launch and an attention launch)
    ->  decision recording (all layers)  ->  positions += 1

Everything is a launch on device-resident state, so the whole step is ONE graph replay:
2 + layers + 1 kernels of this library (2 + 2 * layers + 1 unfused); the recording launch also
advances the positions.

`DecodeHotPath` is driven either with activations that already sit in its device buffers
(`step_device`) or with host buffers (`step_host`: pinned host -> device copies of the step's
q/k/v and positions, graph replay, device -> host copy of the attention output).  For a stream of
host-driven steps, `submit_host_block` / `wait_host_block` pipeline them: two banks of device
buffers, the upload of step n+1 and the download of step n-1 on copy streams of their own while the
kernels of step n run.
"""
from __future__ import annotations

import torch

from fastdms_b200 import _lib
from fastdms_b200.engine.compact_kv import CompactKVManager
from fastdms_b200.layers.compact_attention import (compact_decode_attention,
                                                   fused_dms_rope_store_compact_decode,
                                                   fused_store_decode_attention)


class DecodeHotPath:
    def __init__(self, manager: CompactKVManager, seqs: list, *, num_q_heads: int, window_size: int,
                 alpha_scale: float, alpha_offset: float, cos_sin_cache: torch.Tensor,
                 act_dtype: torch.dtype = torch.bfloat16, scale: float | None = None,
                 expire_every_step: bool = True, use_cuda_graph: bool = True, overlap: bool = True,
                 fuse_store: bool | None = None):
        self.m = manager
        self.seqs = list(seqs)
        self.states = manager._states(self.seqs)
        dev = manager.device
        L, Hk, D = manager.num_layers, manager.num_kv_heads, manager.head_dim
        B = len(self.seqs)
        self.L, self.B, self.Hq, self.Hk, self.D = L, B, int(num_q_heads), Hk, D
        self.window_size = int(window_size)
        self.alpha_scale, self.alpha_offset = float(alpha_scale), float(alpha_offset)
        self.scale = scale
        self.expire_every_step = expire_every_step
        self.overlap = overlap      # attention may start while the layer's store kernel still runs
        self.cos_sin_cache = cos_sin_cache.to(device=dev, dtype=torch.float32).contiguous()
        self.slots_t = manager._slots_tensor(self.states)
        # device-resident step state
        # q | k | v | positions live in ONE device block so that a host-driven step needs one copy
        self._act_dtype = act_dtype
        self._in_block = torch.zeros((self._block_bytes(),), device=dev, dtype=torch.uint8)
        self.q, self.k, self.v, self.positions = self._block_views(self._in_block)
        self.out = torch.zeros((L, B, self.Hq, D), device=dev, dtype=act_dtype)
        self.evict_all = torch.zeros((L, B, Hk), device=dev, dtype=torch.bool)
        self.base = torch.zeros((L, B, Hk), device=dev, dtype=torch.int32)
        self.live = torch.zeros_like(self.base)
        self.slot = torch.zeros_like(self.base)
        self.cu_live = torch.zeros((L, B * Hk + 1), device=dev, dtype=torch.int32)
        # Block tables of the batch.  With contiguous active slots this is a VIEW of the manager's
        # table, which the metadata and expiry kernels update in place (a new page every 16 tokens,
        # released pages at expiry).  With gaps in the slots it has to be a gathered copy; the copy is
        # refreshed inside every step, after the metadata launch (see _enqueue).
        # second bank of activation / output buffers for pipelined host-driven steps (made on first use)
        self._banks = [(self.q, self.k, self.v, self.positions, self.out, self._in_block)]
        self._bank_graphs: list = [None, None]
        self._pipe = None
        self.block_tables = manager.decode_block_tables(self.seqs)
        self._bt_gathered = (self.block_tables is not None
                             and manager._contiguous_active_slot_start(self.states) is None)
        self._slots_long = self.slots_t.long()
        # pinned staging for the host-driven step
        self._h_q = self._h_k = self._h_v = self._h_out = self._h_pos = None
        self.graph = None
        self._host_graphs: dict = {}
        self.use_cuda_graph = use_cuda_graph
        can_fuse = (manager.compact_dtype == torch.float8_e4m3fn and D in (64, 128)
                    and act_dtype in (torch.bfloat16, torch.float16, torch.float32))
        if fuse_store and not can_fuse:
            raise ValueError("fuse_store needs FP8 e4m3 pools and head_dim 64 or 128")
        self.fuse_store = can_fuse if fuse_store is None else bool(fuse_store)
        self.launches_per_step = 2 + (1 if self.fuse_store else 2) * L + 1
        _lib.attn_workspace(dev, B, Hk, D)          # allocate outside any capture

    # ---------------------------------------------------------------- input block layout
    def _block_sizes(self):
        e = torch.empty((), dtype=self._act_dtype).element_size()
        nq = self.L * self.B * self.Hq * self.D * e
        nk = self.L * self.B * self.Hk * self.D * e
        return nq, nk, self.B * 8

    def _block_bytes(self) -> int:
        nq, nk, npos = self._block_sizes()
        return nq + 2 * nk + npos                    # every part is a multiple of 16 bytes for head_dim >= 8

    def _block_views(self, block: torch.Tensor):
        nq, nk, npos = self._block_sizes()
        L, B, D = self.L, self.B, self.D
        q = block[:nq].view(self._act_dtype).view(L, B, self.Hq, D)
        k = block[nq:nq + nk].view(self._act_dtype).view(L, B, self.Hk, D)
        v = block[nq + nk:nq + 2 * nk].view(self._act_dtype).view(L, B, self.Hk, D)
        pos = block[nq + 2 * nk:nq + 2 * nk + npos].view(torch.int64)
        return q, k, v, pos

    def new_host_block(self):
        """A pinned host block with the layout of the device input block and its (q, k, v, positions)
        views: fill the views, then `step_host_block(block)` moves all of it with one copy."""
        block = torch.zeros((self._block_bytes(),), dtype=torch.uint8).pin_memory()
        return (block, *self._block_views(block))

    # ---------------------------------------------------------------- the step itself
    def _enqueue(self, bank: int = 0) -> None:
        m = self.m
        q_all, k_all, v_all, positions, out_all, _ = self._banks[bank]
        if self.expire_every_step:
            m.expire_device(self.slots_t, positions, window_size=self.window_size)
        m.decode_metadata_device(self.slots_t, self.base, self.live, self.slot, self.cu_live)
        if self._bt_gathered:
            torch.index_select(m.block_tables, 1, self._slots_long, out=self.block_tables)
        for l in range(self.L):
            ks, vs = m.layer_scales(l)
            ck, cv = m.compact_k_per_layer[l], m.compact_v_per_layer[l]
            bt = None if self.block_tables is None else self.block_tables[l]
            if self.fuse_store:
                # Layer 0 follows the metadata kernel, whose outputs (live counts, bases) the attention
                # prologue reads before its dependency wait: no overlap there.  Later layers follow the
                # previous layer's attention, which writes nothing this launch reads before the wait.
                fused_store_decode_attention(
                    q_all[l], k_all[l], v_all[l], self.cos_sin_cache, ck, cv, self.base[l], self.live[l],
                    self.evict_all[l], positions, num_kv_heads=self.Hk, alpha_scale=self.alpha_scale,
                    alpha_offset=self.alpha_offset, scale=self.scale, block_tables=bt, k_scale=ks, v_scale=vs,
                    out=out_all[l], overlap_previous_kernel=self.overlap and l > 0)
                continue
            fused_dms_rope_store_compact_decode(
                q_all[l], k_all[l], v_all[l], self.cos_sin_cache, ck, cv, self.slot[l], self.evict_all[l],
                positions, num_kv_heads=self.Hk, alpha_scale=self.alpha_scale, alpha_offset=self.alpha_offset,
                store_q=True, store_transient_k=False, k_scale=ks, v_scale=vs)
            compact_decode_attention(
                q_all[l], ck, cv, self.base[l], self.live[l], scale=self.scale, block_tables=bt,
                k_scale=ks, v_scale=vs, out=out_all[l], overlap_previous_kernel=self.overlap)
        m.record_device(self.slots_t, positions, self.evict_all, advance_positions=True)

    def capture(self) -> None:
        """Runs one eager step (warm-up; it advances the state like any step) and records the graph."""
        if not self.use_cuda_graph or self.graph is not None:
            return
        self._enqueue()
        torch.cuda.synchronize(self.m.device)
        g = torch.cuda.CUDAGraph()
        # Capturing enqueues nothing on the device, but the Python-side calls are the same; the
        # captured launches read the state at replay time.
        with torch.cuda.graph(g):
            self._enqueue()
        self.graph = g

    def step_device(self) -> None:
        """One step on the activations currently in self.q / self.k / self.v at self.positions."""
        if self.use_cuda_graph:
            if self.graph is None:
                raise RuntimeError("call capture() before step_device()")
            self.graph.replay()
        else:
            self._enqueue()

    def set_positions(self, positions) -> None:
        self.positions.copy_(torch.as_tensor(positions, dtype=torch.int64), non_blocking=True)

    # ---------------------------------------------------------------- host-driven step
    def _ensure_pinned(self) -> None:
        if self._h_q is None:
            pin = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
            self._h_q, self._h_k, self._h_v, self._h_out = pin(self.q), pin(self.k), pin(self.v), pin(self.out)
            self._h_pos = torch.empty((self.B,), dtype=torch.int64, pin_memory=True)

    def step_host(self, q_host: torch.Tensor, k_host: torch.Tensor, v_host: torch.Tensor,
                  positions_host: torch.Tensor) -> torch.Tensor:
        """Host buffers in, host buffer out.  Inputs that already sit in pinned memory are copied to
        the device directly; pageable ones are staged through pinned buffers first.  The step runs
        and the attention output [layers, batch, q_heads, head_dim] is copied back.  Returns the
        pinned result tensor (overwritten by the next call)."""
        self._ensure_pinned()
        for dst, stage, src in ((self.q, self._h_q, q_host), (self.k, self._h_k, k_host), (self.v, self._h_v, v_host),
                                (self.positions, self._h_pos, positions_host)):
            if not (src.is_pinned() and src.dtype == dst.dtype and src.is_contiguous()):
                stage.copy_(src)
                src = stage
            dst.copy_(src, non_blocking=True)
        self.step_device()
        self._h_out.copy_(self.out, non_blocking=True)
        torch.cuda.current_stream(self.m.device).synchronize()
        return self._h_out

    def step_host_block(self, block: torch.Tensor) -> torch.Tensor:
        """Like `step_host`, for inputs prepared in a block from `new_host_block()`: one host-to-device
        copy, the step, one device-to-host copy of the outputs.  With CUDA graphs enabled the two
        copies are nodes of a graph captured once per block (the block's address is part of it), so a
        call is one graph launch and one stream synchronisation."""
        if block.dtype != torch.uint8 or block.numel() != self._in_block.numel() or not block.is_pinned():
            raise ValueError("step_host_block takes a pinned block made by new_host_block()")
        self._ensure_pinned()
        stream = torch.cuda.current_stream(self.m.device)
        if not self.use_cuda_graph:
            self._in_block.copy_(block, non_blocking=True)
            self._enqueue()
            self._h_out.copy_(self.out, non_blocking=True)
            stream.synchronize()
            return self._h_out
        if self.graph is None:
            raise RuntimeError("call capture() before step_host_block()")
        g = self._host_graphs.get(block.data_ptr())
        if g is None:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._in_block.copy_(block, non_blocking=True)
                self._enqueue()
                self._h_out.copy_(self.out, non_blocking=True)
            self._host_graphs[block.data_ptr()] = (g, block)        # keeps the block alive with its graph
            g = self._host_graphs[block.data_ptr()]
        g[0].replay()
        torch.cuda.current_stream(self.m.device).synchronize()
        return self._h_out

    # ---------------------------------------------------------------- pipelined host-driven steps
    def _ensure_pipeline(self) -> None:
        if self._pipe is not None:
            return
        if not self.use_cuda_graph or self.graph is None:
            raise RuntimeError("call capture() before submit_host_block()")
        dev = self.m.device
        block2 = torch.zeros_like(self._in_block)
        q2, k2, v2, pos2 = self._block_views(block2)
        self._banks.append((q2, k2, v2, pos2, torch.zeros_like(self.out), block2))
        self._bank_graphs[0] = self.graph
        # The kernels keep running on the stream the path was captured on; capturing the second bank's
        # graph executes nothing.
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._enqueue(bank=1)
        self._bank_graphs[1] = g
        pin = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        self._pipe = {
            "up": torch.cuda.Stream(dev), "down": torch.cuda.Stream(dev), "h_out": [pin(self.out), pin(self.out)],
            "uploaded": [torch.cuda.Event(), torch.cuda.Event()], "computed": [torch.cuda.Event(), torch.cuda.Event()],
            "downloaded": [torch.cuda.Event(), torch.cuda.Event()], "count": 0,
        }

    def submit_host_block(self, block: torch.Tensor) -> int:
        """Enqueues one host-driven step without waiting for it and returns a ticket for
        `wait_host_block`.  Steps alternate between two banks of device buffers: the upload of this
        step's block runs on a copy stream while the previous step's kernels are still running, the
        kernels wait for the upload, and the download of the outputs runs on a third stream.  At most
        two steps may be outstanding: wait for ticket n-1 before submitting n+1.  The block must stay
        unchanged until its step's ticket has been waited for."""
        if block.dtype != torch.uint8 or block.numel() != self._in_block.numel() or not block.is_pinned():
            raise ValueError("submit_host_block takes a pinned block made by new_host_block()")
        self._ensure_pipeline()
        pp = self._pipe
        n = pp["count"]
        bank = n & 1
        main = torch.cuda.current_stream(self.m.device)
        up, down = pp["up"], pp["down"]
        if n >= 2:
            up.wait_event(pp["computed"][bank])       # the bank's previous kernels have read their inputs
        with torch.cuda.stream(up):
            self._banks[bank][5].copy_(block, non_blocking=True)
            pp["uploaded"][bank].record(up)
        main.wait_event(pp["uploaded"][bank])
        if n >= 2:
            main.wait_event(pp["downloaded"][bank])   # the bank's previous outputs have left the device
        self._bank_graphs[bank].replay()
        pp["computed"][bank].record(main)
        down.wait_event(pp["computed"][bank])
        with torch.cuda.stream(down):
            pp["h_out"][bank].copy_(self._banks[bank][4], non_blocking=True)
            pp["downloaded"][bank].record(down)
        pp["count"] = n + 1
        return n

    def wait_host_block(self, ticket: int) -> torch.Tensor:
        """Outputs [layers, batch, q_heads, head_dim] of the step `ticket` in pinned host memory
        (overwritten when the second step after it is submitted)."""
        pp = self._pipe
        if pp is None or not (pp["count"] - 2 <= ticket < pp["count"]):
            raise ValueError("unknown or expired ticket")
        pp["downloaded"][ticket & 1].synchronize()
        return pp["h_out"][ticket & 1]

    @property
    def h2d_bytes_per_step(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.q, self.k, self.v, self.positions))

    @property
    def d2h_bytes_per_step(self) -> int:
        return self.out.numel() * self.out.element_size()
