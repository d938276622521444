"""Generate the end-to-end golden trace of the tiny CPU-runnable model by running the REFERENCE model classes
and its CompactKVManager on CPU.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_model.py --reference /path/to/FastDMS

Tiny Llama-style DMS model, float32, 2 layers, hidden 256, 4 q / 2 KV heads, head_dim 64, MLP
1024, vocab 1024, RoPE theta 500000, DMS window 16, eviction rate ~7/8; four ragged prompts of
37/128/200/511 tokens; 128 greedy decode steps; compact KV in float32 and in FP8 e4m3.  Logits are
kept for the first 32 steps and every 8th step after that (`logit_steps`), everything else for all
steps.  `*_top2_gap` / `*_runner_up` give the margin of every greedy choice (a model with random
weights produces near-ties: with 1024 logits of spread 1.6 about one choice in a hundred has a
margin below 5e-3, which is the size of FP8 rounding effects, so a test can only demand the
reference's token where the margin is larger than the logit tolerance).

A third run ("bf16") loads the same weights rounded to bfloat16 (the LM head scaled by 0.05 so that
logits stay below 0.5 in magnitude: two bfloat16 runs of the same model differ by a few units in the last
place of their logits, and only at that scale are a few such units well under the 2e-2 tolerance), keeps the
FP8 compact KV and additionally records the raw DMS decision value of every (step, layer, sequence,
KV head) -- the number that is compared with the threshold -- so that a test can tell a decision
that sits on the threshold from one that does not.  Its greedy tokens are the history a test forces
on the implementation under test.
Weights and prompts come from `fastdms_b200.utils.synth` (an integer hash), so the tests rebuild
the identical model without a checkpoint.

Everything on the path is the reference's code (models/llama.py, engine/compact_kv.py,
engine/dms.py, layers/*), driven in the order of engine/model_runner.py:594-772,1105-1145
(allocate -> prefill; per step: apply_dms_evictions -> prepare_decode_metadata -> forward ->
record_appended_dms_decisions).  Three callees exist only as CUDA code and are substituted:
  flash_attn_varlen_func     -> per-sequence causal softmax attention in float32
  store_compact_kvcache      -> indexed row assignment
  compact_decode_attention   -> the reference's own compact_decode_attention_ref
"""
from __future__ import annotations

import argparse
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

MODEL_CFG = dict(
    model_type="llama", hidden_size=256, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
    num_key_value_heads=2, head_dim=64, vocab_size=1024, rms_norm_eps=1e-5, max_position_embeddings=1024,
    rope_theta=500000.0, attention_bias=True, tie_word_embeddings=False, hidden_act="silu", lm_head_std=0.1,
    synthetic_hash_weights=True, torch_dtype="float32",
)
PROMPT_LENS = [37, 128, 200, 511]
DECODE_STEPS = 128
LOGIT_STEPS = sorted(set(range(32)) | set(range(32, DECODE_STEPS, 8)) | {DECODE_STEPS - 1})
BF16_LM_HEAD_FACTOR = 0.05
WINDOW, ALPHA_SCALE, ALPHA_OFFSET = 16, 100.0, 5.0
SEED = 0


def make_prompts():
    from fastdms_b200.utils.synth import hashed_uniform
    out = []
    for i, n in enumerate(PROMPT_LENS):
        u = hashed_uniform(f"prompt{i}", (n,), SEED)
        out.append(np.minimum(((u + 1.0) * 0.5 * MODEL_CFG["vocab_size"]).astype(np.int64), MODEL_CFG["vocab_size"] - 1).tolist())
    return out


def sdpa_varlen(q, k, v, max_seqlen_q, cu_seqlens_q, max_seqlen_k, cu_seqlens_k, softmax_scale, causal, block_table=None):
    out = torch.empty_like(q)
    cu = cu_seqlens_q.tolist()
    G = q.shape[1] // k.shape[1]
    for i in range(len(cu) - 1):
        s, e = cu[i], cu[i + 1]
        qq = q[s:e].float().transpose(0, 1)                       # [Hq, T, D]
        kk = k[s:e].float().transpose(0, 1).repeat_interleave(G, dim=0)
        vv = v[s:e].float().transpose(0, 1).repeat_interleave(G, dim=0)
        sc = torch.matmul(qq, kk.transpose(1, 2)) * softmax_scale
        mask = torch.ones(e - s, e - s, dtype=torch.bool).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
        out[s:e] = torch.matmul(torch.softmax(sc, dim=-1), vv).transpose(0, 1).to(q.dtype)
    return out


def index_store(key, value, compact_k, compact_v, slot_mapping):
    flat = slot_mapping.reshape(-1).long()
    compact_k[flat] = key.reshape(-1, key.shape[-1]).to(compact_k.dtype)
    compact_v[flat] = value.reshape(-1, value.shape[-1]).to(compact_v.dtype)


def run(reference: str, kv_dtype: torch.dtype, tag: str, out: dict, model_dtype: torch.dtype = torch.float32) -> None:
    import torch.distributed as dist
    from transformers import LlamaConfig

    import fastdms.layers.attention as ref_attention
    from fastdms.engine.compact_kv import CompactKVManager
    from fastdms.engine.sequence import Sequence
    from fastdms.layers.compact_attention import compact_decode_attention_ref
    from fastdms.models.llama import LlamaForCausalLM
    from fastdms.sampling_params import SamplingParams
    import fastdms.models.llama as ref_llama
    from fastdms.utils.context import get_context, reset_context, set_context
    from fastdms_b200.utils.synth import synth_llama_state_dict

    if not dist.is_initialized():
        dist.init_process_group("gloo", init_method="tcp://127.0.0.1:29611", rank=0, world_size=1)
    ref_attention.flash_attn_varlen_func = sdpa_varlen
    ref_attention.store_compact_kvcache = index_store
    ref_attention.compact_decode_attention = (
        lambda q, ck, cv, base, live, scale=None, **kw: compact_decode_attention_ref(q, ck, cv, base, live, scale=scale))

    # raw decision values, in call order (one call per layer per forward)
    decision_log: list[torch.Tensor] = []
    original_extract = getattr(ref_llama.extract_dms_eviction_decisions, "__wrapped__", ref_llama.extract_dms_eviction_decisions)

    def recording_extract(q, *, num_kv_heads, num_qo_heads, head_dim, **kw):
        view = q.view(q.shape[0], num_kv_heads, num_qo_heads // num_kv_heads, head_dim)
        decision_log.append(view[:, :, 0, -1].float().clone())
        return original_extract(q, num_kv_heads=num_kv_heads, num_qo_heads=num_qo_heads, head_dim=head_dim, **kw)

    recording_extract.__wrapped__ = original_extract
    ref_llama.extract_dms_eviction_decisions = recording_extract

    cfg = {k: v for k, v in MODEL_CFG.items() if k not in ("lm_head_std", "synthetic_hash_weights", "torch_dtype", "model_type")}
    hf = LlamaConfig(**cfg)
    torch.set_default_dtype(model_dtype)
    model = LlamaForCausalLM(hf)
    torch.set_default_dtype(torch.float32)
    synth_cfg = dict(MODEL_CFG)
    if model_dtype != torch.float32:
        synth_cfg["lm_head_factor"] = BF16_LM_HEAD_FACTOR
    sd = synth_llama_state_dict(synth_cfg, seed=SEED, alpha_scale=ALPHA_SCALE, alpha_offset=ALPHA_OFFSET)
    packed = model.packed_modules_mapping
    for name, tensor in sd.items():
        for key, (target, shard) in packed.items():
            if f".{key}." in name:
                p = model.get_parameter(name.replace(key, target))
                p.weight_loader(p, tensor, shard)
                break
        else:
            p = model.get_parameter(name)
            getattr(p, "weight_loader", lambda pp, t: pp.data.copy_(t))(p, tensor)
    model.eval()
    L, Hk, D = hf.num_hidden_layers, hf.num_key_value_heads, MODEL_CFG["head_dim"]
    manager = CompactKVManager(num_layers=L, num_kv_heads=Hk, capacity_tokens=8192, max_model_len=1024, device="cpu",
                               head_dim=D, compact_dtype=kv_dtype, per_layer_storage=True)
    attn_modules = [layer.self_attn.attn for layer in model.model.layers]
    for i, mod in enumerate(attn_modules):
        mod.layer_id = i
    manager.attach_attention_modules(attn_modules)
    prompts = make_prompts()
    seqs = [Sequence(p, SamplingParams(temperature=0.0, max_tokens=DECODE_STEPS + 1, ignore_eos=True)) for p in prompts]
    B = len(seqs)
    cache = model.model.layers[0].self_attn.rotary_emb.cos_sin_cache
    out["cos_sin_cache"] = cache[: max(PROMPT_LENS) + DECODE_STEPS + 2, 0].float().numpy().copy()

    with torch.inference_mode():
        # ---- prefill (engine/model_runner.py:594-679) ----
        ids, pos, cu = [], [], [0]
        for s in seqs:
            ids.extend(s.token_ids)
            pos.extend(range(len(s)))
            cu.append(cu[-1] + len(s))
            manager.allocate(s)
        cu_t = torch.tensor(cu, dtype=torch.int32)
        set_context(True, cu_t, cu_t, max(PROMPT_LENS), max(PROMPT_LENS), torch.full((cu[-1],), -1, dtype=torch.int32),
                    None, None, dms_capture_enabled=True, dms_alpha_scale=ALPHA_SCALE, dms_alpha_offset=ALPHA_OFFSET,
                    dms_layer_evictions={}, streaming_pack_manager=manager,
                    streaming_pack_seq_ids=[s.seq_id for s in seqs], streaming_pack_window_size=WINDOW)
        decision_log.clear()
        hidden = model(torch.tensor(ids), torch.tensor(pos))
        logits = model.compute_logits(hidden).float()
        ctx = get_context()
        out[f"{tag}_prefill_evict"] = torch.stack([ctx.dms_layer_evictions[l] for l in range(L)]).numpy().copy()
        out[f"{tag}_prefill_decision_values"] = torch.stack(decision_log).numpy().copy()     # [L, tokens, Hk]
        reset_context()
        out[f"{tag}_prefill_logits"] = logits.numpy().copy()
        live0 = torch.stack([manager.seq_states[s.seq_id].live_counts for s in seqs], dim=1)     # [L, B, Hk]
        out[f"{tag}_prefill_live"] = live0.numpy().copy()
        tokens = logits.argmax(dim=-1).tolist()
        top2 = [logits.topk(2, dim=-1)]              # per step: the two largest logits and their ids
        all_tokens, step_logits, step_evict, step_live, step_slot, step_values = [tokens], [], [], [], [], []
        for s, t in zip(seqs, tokens):
            s.append_token(t)
        # ---- decode (engine/model_runner.py:713-772, 1105-1145) ----
        for step in range(DECODE_STEPS):
            positions = [len(s) - 1 for s in seqs]
            manager.apply_dms_evictions(seqs, positions, window_size=WINDOW, sync_stats=False)
            base, live, slot, cap = manager.prepare_decode_metadata(seqs)
            set_context(False, compact_kv_enabled=True, compact_base_offsets=base, compact_live_counts=live,
                        compact_slot_mapping=slot, compact_max_live_count=cap, dms_capture_enabled=True,
                        dms_alpha_scale=ALPHA_SCALE, dms_alpha_offset=ALPHA_OFFSET, dms_layer_evictions={})
            decision_log.clear()
            hidden = model(torch.tensor([s.last_token for s in seqs]), torch.tensor(positions))
            logits = model.compute_logits(hidden).float()
            step_values.append(torch.stack(decision_log).numpy().copy())                         # [L, B, Hk]
            ctx = get_context()
            ev = torch.stack([ctx.dms_layer_evictions[l] for l in range(L)])                     # [L, B, Hk]
            manager.record_appended_dms_decisions(seqs, positions, ctx.dms_layer_evictions, sync_stats=False)
            reset_context()
            tokens = logits.argmax(dim=-1).tolist()
            top2.append(logits.topk(2, dim=-1))
            for s, t in zip(seqs, tokens):
                s.append_token(t)
            all_tokens.append(tokens)
            if step in LOGIT_STEPS:
                step_logits.append(logits.numpy().copy())
            step_evict.append(ev.numpy().copy())
            step_live.append(live.numpy().copy())
            step_slot.append((slot - base).numpy().copy())         # logical slot index of the appended row
    out[f"{tag}_tokens"] = np.array(all_tokens, dtype=np.int64)                 # [steps + 1, B]
    # margin of every greedy choice: top logit minus runner-up, and the runner-up's id
    out[f"{tag}_top2_gap"] = np.stack([(t.values[:, 0] - t.values[:, 1]).numpy() for t in top2]).astype(np.float32)
    out[f"{tag}_runner_up"] = np.stack([t.indices[:, 1].numpy() for t in top2]).astype(np.int64)
    out[f"{tag}_logits"] = np.stack(step_logits)                               # [len(LOGIT_STEPS), B, V]
    out[f"{tag}_decision_values"] = np.stack(step_values)                      # [steps, L, B, Hk]
    out[f"{tag}_evict"] = np.stack(step_evict)                                 # [steps, L, B, Hk]
    out[f"{tag}_live"] = np.stack(step_live)                                   # [steps, L, B, Hk]
    out[f"{tag}_slot"] = np.stack(step_slot)                                   # [steps, L, B, Hk]
    for i, s in enumerate(seqs):
        st = manager.seq_states[s.seq_id]
        out[f"{tag}_final_pos_s{i}"] = st.token_positions.numpy().copy()
        out[f"{tag}_final_ev_s{i}"] = st.evict_mask.numpy().copy()
        out[f"{tag}_final_live_s{i}"] = st.live_counts.numpy().copy()
    for s in seqs:
        manager.free(s.seq_id)
    assert manager.free_tokens == L * 8192
    print(tag, "tokens of seq 0:", [t[0] for t in all_tokens][:12], "evict rate", float(np.stack(step_evict).mean()),
          "live after prefill", live0.flatten().tolist())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of a FastDMS checkout (the directory that holds the fastdms package)")
    args = ap.parse_args()
    os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")
    os.environ.setdefault("FASTDMS_DMS_EXPIRY_TRITON", "0")
    os.environ.setdefault("FASTDMS_DMS_FUSED_DECODE_PREPROCESS", "0")
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    torch.set_num_threads(4)
    out: dict[str, np.ndarray] = {}
    run(args.reference, torch.float32, "f32", out)
    run(args.reference, torch.float8_e4m3fn, "fp8", out)
    run(args.reference, torch.float8_e4m3fn, "bf16", out, model_dtype=torch.bfloat16)
    out["prompt_lens"] = np.array(PROMPT_LENS)
    out["logit_steps"] = np.array(LOGIT_STEPS)
    path = HERE / "model_golden.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size / 1024:.1f} KiB)")


if __name__ == "__main__":
    main()
