"""Model shapes of the reference's published benchmarks, as synthetic HF-style config dicts."""
from __future__ import annotations

SHAPES = {
    # Llama-3.2-1B: 16 layers, hidden 2048, 32 q / 8 KV heads of 64, MLP 8192, vocab 128256
    "llama-1b": dict(model_type="llama", hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                     num_attention_heads=32, num_key_value_heads=8, head_dim=64, vocab_size=128256,
                     rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=False, hidden_act="silu"),
    # Qwen3-8B: 36 layers, hidden 4096, 32 q / 8 KV heads of 128, q/k RMSNorm, MLP 12288, vocab 151936
    "qwen3-8b": dict(model_type="qwen3", hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                     num_attention_heads=32, num_key_value_heads=8, head_dim=128, vocab_size=151936,
                     rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, hidden_act="silu"),
    # small shape for tests
    "tiny": dict(model_type="llama", hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                 num_attention_heads=8, num_key_value_heads=2, head_dim=64, vocab_size=1024,
                 rms_norm_eps=1e-5, rope_theta=500000.0, tie_word_embeddings=False, hidden_act="silu"),
}
