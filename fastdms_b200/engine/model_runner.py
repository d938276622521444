"""Per-rank model runner for compact-DMS serving.

Follows the reference's `fastdms/engine/model_runner.py` for the step order:
  prefill: allocate -> forward (per layer: decisions, RoPE, prefill pack, dense attention) -> sample
  decode : expire -> decode metadata (live += 1) -> forward (per layer: fused store, compact
           attention) -> record decisions -> sample
The whole decode step, including expiry, metadata, recording and the greedy argmax, is ONE CUDA
graph per batch size (the reference graphs only the model forward and re-captures when its lazily
grown pools move; the pools here never move).  Tensor parallelism is SPMD: one process per GPU
(torchrun), every rank runs the same schedule on its share of the KV heads and the row-parallel
linears all-reduce over NCCL.
"""
from __future__ import annotations

import os
from glob import glob

import torch
import torch.distributed as dist

from fastdms_b200.config import Config
from fastdms_b200.engine.compact_kv import CompactKVManager
from fastdms_b200.engine.dms import DMSMetadata, load_dms_metadata
from fastdms_b200.engine.sequence import Sequence
from fastdms_b200.layers.sampler import Sampler, argmax_workspace, greedy_argmax
from fastdms_b200.models.registry import build_model
from fastdms_b200.utils.context import reset_context, set_context
from fastdms_b200.utils.loader import load_model, load_state_dict
from fastdms_b200.utils.profiler import get_profiler


class _DecodeGraph:
    """Static buffers (and the captured graph) of the decode step for one batch size."""

    def __init__(self, runner: "ModelRunner", batch: int):
        dev = runner.device
        m = runner.compact_kv_manager
        L, Hk = m.num_layers, m.num_kv_heads
        self.batch = batch
        self.ids = torch.zeros((batch,), device=dev, dtype=torch.int64)
        self.pos = torch.zeros((batch,), device=dev, dtype=torch.int64)
        self.slots = torch.zeros((batch,), device=dev, dtype=torch.int32)
        self.base = torch.zeros((L, batch, Hk), device=dev, dtype=torch.int32)
        self.live = torch.zeros_like(self.base)
        self.slot = torch.zeros_like(self.base)
        self.cu = torch.zeros((L, batch * Hk + 1), device=dev, dtype=torch.int32)
        self.evict_all = torch.zeros((L, batch, Hk), device=dev, dtype=torch.bool)
        self.h_in = torch.zeros((3, batch), dtype=torch.int64, pin_memory=True)
        self.d_in = torch.zeros((3, batch), device=dev, dtype=torch.int64)
        self.argmax_scratch = argmax_workspace(batch, dev)
        self.logits = None
        self.tokens = None
        self.graph = None
        # run-ahead decode: token read-back of the last two steps (pinned) and the events that guard them
        self.h_tok = torch.zeros((2, batch), dtype=torch.int64, pin_memory=True)
        self.tok_events = [torch.cuda.Event(), torch.cuda.Event()]
        self.tok_turn = 0


class ModelRunner:
    def __init__(self, config: Config, device: torch.device | None = None):
        self.config = config
        hf = config.hf_config
        from fastdms_b200.layers.linear import set_replica_mode, tp_world
        # tensor_parallel_size 1 inside a multi-rank job = one full replica per rank (sequence sharding)
        set_replica_mode(config.tensor_parallel_size == 1)
        self.world_size, self.rank = tp_world()
        if self.world_size != config.tensor_parallel_size:
            raise RuntimeError(
                f"tensor_parallel_size={config.tensor_parallel_size} needs that many ranks (torchrun); "
                f"the process group has {self.world_size}")
        if not torch.cuda.is_available():
            raise RuntimeError("fastdms_b200 requires a CUDA device (there is no CPU fallback)")
        if device is None:
            device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", torch.cuda.current_device())))
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.dtype = config.model_dtype()
        if self.world_size > 1:
            # small tensor-parallel sums go through NVLink peer memory instead of NCCL
            from fastdms_b200.layers.peer_allreduce import init_fused_row_parallel, init_peer_all_reduce
            self.peer_all_reduce = init_peer_all_reduce(self.device)
            self.fused_row_parallel = init_fused_row_parallel(self.device)
        self.dms_metadata = self._load_dms_metadata()
        default_dtype = torch.get_default_dtype()
        torch.set_default_dtype(self.dtype)
        try:
            with torch.device(self.device):
                self.model = build_model(hf)
        finally:
            torch.set_default_dtype(default_dtype)
        self.model.to(self.device)       # also moves the (float32, CPU-built) rotary tables
        self._load_weights()
        if config.fp8_weights:
            from fastdms_b200.layers.linear import LinearBase
            for mod in self.model.modules():
                if isinstance(mod, LinearBase) and mod.weight.dtype in (torch.bfloat16, torch.float16):
                    mod.quantize_fp8()
        self.model.eval()
        for p in self.model.parameters():
            p.requires_grad_(False)
        self.sampler = Sampler()
        self.num_kv_heads = hf.num_key_value_heads // self.world_size
        self.num_q_heads = hf.num_attention_heads // self.world_size
        self.head_dim = hf.head_dim
        self.compact_kv_manager = self._allocate_kv()
        self.compact_kv_manager.attach_attention_modules(self.model.attention_modules())
        self.graphs: dict[int, _DecodeGraph] = {}
        self.last_dms_decode_stats: list[dict] = []

    # ------------------------------------------------------------------ set-up
    def _load_dms_metadata(self) -> DMSMetadata:
        c = self.config
        try:
            md = load_dms_metadata(c.model, c.dms_metadata_path)
            w, a, o = md.window_size, md.alpha_scale, md.alpha_offset
            src = (md.source_path, md.source_kind, md.packaged_metadata_found)
        except (FileNotFoundError, NotADirectoryError):
            w, a, o, src = 256, 100.0, 5.0, ("", "config_defaults", False)
        w = c.dms_window_size if c.dms_window_size is not None else w
        a = c.dms_alpha_scale if c.dms_alpha_scale is not None else a
        o = c.dms_alpha_offset if c.dms_alpha_offset is not None else o
        return DMSMetadata(model_path=str(c.model), source_path=str(src[0]), source_kind=src[1],
                           packaged_metadata_found=src[2], window_size=int(w), alpha_scale=float(a),
                           alpha_offset=float(o))

    def _load_weights(self) -> None:
        c = self.config
        if os.path.isdir(os.fspath(c.model)) and glob(os.path.join(os.fspath(c.model), "*.safetensors")):
            load_model(self.model, os.fspath(c.model))
            return
        if c.random_init_seed is None:
            raise FileNotFoundError(f"no *.safetensors under {c.model!r} and random_init_seed is not set")
        hf = c.hf_config
        if getattr(hf, "synthetic_hash_weights", False):
            from fastdms_b200.utils.synth import synth_llama_state_dict
            sd = synth_llama_state_dict(vars(hf), seed=c.random_init_seed, alpha_scale=self.dms_metadata.alpha_scale,
                                        alpha_offset=self.dms_metadata.alpha_offset)
            load_state_dict(self.model, sd)
            return
        # large random-init models: draw on the device (same seed on every rank, then sharded values
        # differ per rank only through the shard they keep, which is what a loader would give)
        g = torch.Generator(device=self.device).manual_seed(int(c.random_init_seed) + 7919 * self.rank)
        for name, p in self.model.named_parameters():
            if p.ndim == 1:
                if "norm" in name:
                    p.data.fill_(1.0)
                else:
                    p.data.zero_()
            else:
                std = p.shape[-1] ** -0.5 if "embed" not in name else 1.0
                p.data.copy_(torch.randn(p.shape, device=self.device, generator=g, dtype=torch.float32) * std)
        self._wire_decision_channel()

    def _wire_decision_channel(self, evict_rate: float = 7.0 / 8.0) -> None:
        """Random-init models: give the DMS decision channel a bias so that about `evict_rate` of
        the tokens are marked for eviction (needs attention_bias or is skipped)."""
        import math
        lo, hi = -6.0, 6.0
        for _ in range(60):
            mid = 0.5 * (lo + hi)
            if 0.5 * (1.0 + math.erf(mid / math.sqrt(2.0))) < evict_rate:
                lo = mid
            else:
                hi = mid
        shift = self.dms_metadata.alpha_offset / self.dms_metadata.alpha_scale + 0.5 * (lo + hi)
        for layer in self.model.model.layers:
            att = layer.self_attn
            if att.qkv_proj.bias is None:
                continue
            G = att.num_heads // att.num_kv_heads
            for h in range(att.num_kv_heads):
                att.qkv_proj.bias.data[(h * G) * att.head_dim + att.head_dim - 1] = shift

    def _allocate_kv(self) -> CompactKVManager:
        c, hf = self.config, self.config.hf_config
        kv_dtype = c.resolve_kv_cache_dtype()
        elem = torch.empty((), dtype=kv_dtype).element_size()
        L = hf.num_hidden_layers
        per_row = L * 2 * self.head_dim * elem
        per_seq = c.compact_kv_target_live_tokens_per_seq or c.max_model_len
        rows = c.compact_kv_capacity_tokens or c.max_num_seqs * min(per_seq, c.max_model_len) * self.num_kv_heads
        if c.compact_kv_budget_bytes:
            rows = min(rows, max(256, c.compact_kv_budget_bytes // per_row))
        free, _ = torch.cuda.mem_get_info(self.device)
        rows = int(min(rows, max(256, int(free * c.gpu_memory_utilization * 0.8) // per_row)))
        return CompactKVManager(
            num_layers=L, num_kv_heads=self.num_kv_heads, capacity_tokens=rows, max_model_len=c.max_model_len,
            device=self.device, target_live_tokens_per_seq=c.compact_kv_target_live_tokens_per_seq,
            head_dim=self.head_dim, compact_dtype=kv_dtype, max_active_seqs=c.max_num_seqs, paged=c.compact_kv_paged,
            dms_expiry_interval=c.dms_expiry_interval,
            row_indirection=c.compact_kv_row_indirection, admission=c.compact_kv_admission,
            admission_keep_estimate=c.compact_kv_admission_keep_estimate,
            admission_window=self.dms_metadata.window_size)

    # ------------------------------------------------------------------ prefill
    @torch.inference_mode()
    def run_prefill(self, seqs: list[Sequence]) -> torch.Tensor:
        """One prefill forward: whole prompts, or -- with `Config.prefill_chunk_size` -- the next
        `num_scheduled_tokens` prompt tokens of every sequence (tokens before `num_cached_tokens` are
        already in its compact spans).  Returns the logits of each sequence's last token of the batch."""
        md, m, dev = self.dms_metadata, self.compact_kv_manager, self.device
        ids, pos, cu = [], [], [0]
        starts, remaining = [], []
        for seq in seqs:
            total = len(seq)
            a = int(seq.num_cached_tokens) if self.config.prefill_chunk_size else 0
            n = int(seq.num_scheduled_tokens) if self.config.prefill_chunk_size and seq.num_scheduled_tokens else total - a
            ids.extend(seq[a:a + n])
            pos.extend(range(a, a + n))
            cu.append(cu[-1] + n)
            starts.append(a)
            remaining.append(total - a - n)
            m.allocate(seq)
        chunked = bool(self.config.prefill_chunk_size)
        prefix_slots = None
        if chunked and any(a > 0 for a in starts):
            prefix_slots = m._slots_tensor(m._states(seqs))
        ids_t = torch.tensor(ids, dtype=torch.int64, pin_memory=True).to(dev, non_blocking=True)
        pos_t = torch.tensor(pos, dtype=torch.int64, pin_memory=True).to(dev, non_blocking=True)
        cu_t = torch.tensor(cu, dtype=torch.int32, pin_memory=True).to(dev, non_blocking=True)
        set_context(True, cu_t, cu_t, max(cu[i + 1] - cu[i] for i in range(len(seqs))), 0,
                    compact_kv_enabled=True, dms_capture_enabled=True, dms_alpha_scale=md.alpha_scale,
                    dms_alpha_offset=md.alpha_offset, dms_layer_evictions={}, streaming_pack_manager=m,
                    streaming_pack_seq_ids=[s.seq_id for s in seqs], streaming_pack_window_size=md.window_size,
                    cu_seqlens_host=cu, prefill_chunk_starts=starts if chunked else None,
                    prefill_chunk_remaining=remaining if chunked else None, compact_prefix_slots=prefix_slots)
        try:
            with get_profiler().cuda_phase("model_forward_prefill"):
                hidden = self.model(ids_t, pos_t)
            last = hidden[cu_t[1:].long() - 1]
            logits = self.model.compute_logits(last)
            if m.paged and m.admission == "optimistic":
                # pages are popped on the device: a stack that ran dry shows in the status word
                from fastdms_b200 import _lib
                if _lib.read_device_status(dev) & _lib.DEV_BAD_INDEX:
                    raise RuntimeError("compact KV capacity exhausted: the page pool ran dry during a prefill")
            if chunked:
                # prompts that are now complete give back what the chunked reservation did not use
                m.trim_spans([s.seq_id for s, rest, a in zip(seqs, remaining, starts) if rest == 0 and a > 0])
            return logits
        finally:
            reset_context()

    # ------------------------------------------------------------------ decode
    def _decode_body(self, g: _DecodeGraph) -> None:
        md, m = self.dms_metadata, self.compact_kv_manager
        if m.dms_expiry_interval == 1:
            m.expire_device(g.slots, g.pos, window_size=md.window_size)
        m.decode_metadata_device(g.slots, g.base, g.live, g.slot, g.cu)
        bt = m.block_tables.index_select(1, g.slots.long()) if m.paged else None
        set_context(False, compact_kv_enabled=True, compact_base_offsets=g.base, compact_live_counts=g.live,
                    compact_slot_mapping=g.slot, compact_max_live_count=m.max_model_len, dms_capture_enabled=True,
                    dms_alpha_scale=md.alpha_scale, dms_alpha_offset=md.alpha_offset,
                    dms_layer_evictions_buffer=g.evict_all, compact_block_tables=bt,
                    overlap_store_and_attention=True)
        try:
            hidden = self.model(g.ids, g.pos)
        finally:
            reset_context()
        # With run-ahead the step leaves the NEXT step's inputs on the device: the recording launch
        # advances the positions and the argmax writes the greedy tokens into the id buffer (the
        # reference feeds tokens back on the device for a single sequence only,
        # fastdms/engine/model_runner.py:971-1053).  Host-provided inputs simply overwrite them.
        feed = self.config.decode_run_ahead
        m.record_device(g.slots, g.pos, g.evict_all, advance_positions=feed)
        g.logits = self.model.compute_logits(hidden)
        g.tokens = greedy_argmax(g.logits, g.argmax_scratch, out=g.ids if feed else None)

    def _decode_inputs(self, g: _DecodeGraph, seqs: list[Sequence]) -> None:
        m = self.compact_kv_manager
        states = m._states(seqs)
        for i, (seq, st) in enumerate(zip(seqs, states)):
            g.h_in[0, i] = seq.last_token
            g.h_in[1, i] = len(seq) - 1
            g.h_in[2, i] = st.active_slot
        g.d_in.copy_(g.h_in, non_blocking=True)
        g.ids.copy_(g.d_in[0])
        g.pos.copy_(g.d_in[1])
        g.slots.copy_(g.d_in[2])

    def can_run_ahead(self, seqs: list[Sequence]) -> bool:
        """Whether the decode step of `seqs` can be replayed from device-resident inputs: greedy
        requests only, expiry inside the graph, and the graph of this batch size already captured."""
        g = self.graphs.get(len(seqs))
        return (self.config.decode_run_ahead and not self.config.enforce_eager
                and self.compact_kv_manager.dms_expiry_interval == 1
                and g is not None and isinstance(g.graph, torch.cuda.CUDAGraph)
                and all(seq.temperature <= 1e-10 for seq in seqs))

    @torch.inference_mode()
    def launch_decode(self, seqs: list[Sequence], device_fed: bool):
        """Enqueues one decode step and the read-back of its greedy tokens without waiting for
        either; `resolve_decode` returns the tokens.  With `device_fed` the step reads the token
        ids, positions and slots the previous step of the same batch left on the device."""
        g = self.run_decode(seqs, device_fed=device_fed)
        turn = g.tok_turn
        g.tok_turn ^= 1
        g.h_tok[turn].copy_(g.tokens, non_blocking=True)
        g.tok_events[turn].record()
        return g, turn

    def resolve_decode(self, handle) -> list[int]:
        g, turn = handle
        g.tok_events[turn].synchronize()
        return g.h_tok[turn].tolist()

    @torch.inference_mode()
    def run_decode(self, seqs: list[Sequence], device_fed: bool = False) -> _DecodeGraph:
        """One decode step for `seqs`; returns the buffers holding logits and greedy tokens."""
        m, md = self.compact_kv_manager, self.dms_metadata
        B = len(seqs)
        g = self.graphs.get(B)
        if g is None:
            g = _DecodeGraph(self, B)
            self.graphs[B] = g
        if device_fed:
            with get_profiler().cuda_phase("model_forward_decode"):
                g.graph.replay()
            return g
        if m.dms_expiry_interval != 1:
            with get_profiler().cuda_phase("dms_decode_expire"):
                self.last_dms_decode_stats.append(m.apply_dms_evictions(
                    seqs, [len(s) - 1 for s in seqs], window_size=md.window_size, sync_stats=False))
        self._decode_inputs(g, seqs)
        if self.config.enforce_eager:
            self._decode_body(g)
            return g
        if g.graph is None:
            # One eager step doubles as warm-up (lazy allocations, cuBLAS handles); it is a real
            # step, so the graph is captured for the NEXT call and this one returns the eager result.
            self._decode_body(g)
            torch.cuda.synchronize(self.device)
            g.graph = "pending"
            return g
        if g.graph == "pending":
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):          # nothing executes during capture: the state does not advance
                self._decode_body(g)
            g.graph = graph
        with get_profiler().cuda_phase("model_forward_decode"):
            g.graph.replay()
        return g

    # ------------------------------------------------------------------ run / free
    @torch.inference_mode()
    def run(self, seqs: list[Sequence], is_prefill: bool) -> list[int]:
        if is_prefill:
            logits = self.run_prefill(seqs)
            greedy = None
        else:
            g = self.run_decode(seqs)
            logits, greedy = g.logits, g.tokens
        temps = [seq.temperature for seq in seqs]
        if all(t <= 1e-10 for t in temps):
            tokens = greedy if greedy is not None else greedy_argmax(logits)
        else:
            t = torch.tensor([max(x, 1e-10) for x in temps], dtype=torch.float32, device=self.device)
            tokens = self.sampler(logits, t)
            if any(x <= 1e-10 for x in temps):
                arg = greedy_argmax(logits)
                mask = torch.tensor([x <= 1e-10 for x in temps], device=self.device)
                tokens = torch.where(mask, arg, tokens)
        return tokens.tolist()

    def free_compact(self, seq_ids: list[int]) -> None:
        for sid in seq_ids:
            self.compact_kv_manager.free(sid)
