"""qwen3 family: the llama-style block with per-head RMSNorm on q and k (``qk_norm``), untied head.
Family parity: reference ``src/dataflow_training/model_families/qwen3/``."""
from .._llama_like import register_llama_like

PRESETS = {
    "tiny": dict(name="tiny", n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=512, vocab_size=1024,
                 seq_len=128, batch=2, grad_accum_rounds=2),
    "qwen3_0p6b": dict(name="qwen3_0p6b", n_layers=28, d_model=1024, n_heads=16, n_kv_heads=8, head_dim=128, d_ff=3072,
                       vocab_size=151936, rope_theta=1e6, rms_eps=1e-6, seq_len=2048, batch=4, grad_accum_rounds=8),
    "qwen3_1p7b": dict(name="qwen3_1p7b", n_layers=28, d_model=2048, n_heads=16, n_kv_heads=8, head_dim=128, d_ff=6144,
                       vocab_size=151936, rope_theta=1e6, rms_eps=1e-6, seq_len=2048, batch=4, grad_accum_rounds=8),
    "qwen3_8b": dict(name="qwen3_8b", n_layers=36, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128, d_ff=12288,
                     vocab_size=151936, rope_theta=1e6, rms_eps=1e-6, seq_len=4096, batch=4, grad_accum_rounds=8,
                     dtype_policy="bf16_split_master"),
}
FAMILY = register_llama_like("qwen3", PRESETS, qk_norm=True)
