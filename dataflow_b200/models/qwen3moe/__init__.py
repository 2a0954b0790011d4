"""qwen3moe family: qwen3 attention (q/k RMSNorm) with a mixture-of-experts MLP, top-k then softmax over the
selection (normalised route weights).  Family parity: reference ``src/dataflow_training/model_families/qwen3moe/``."""
from .._llama_like import register_llama_like

PRESETS = {
    "tiny": dict(name="tiny", n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, d_ff=0, vocab_size=1024,
                 seq_len=128, batch=2, grad_accum_rounds=2, n_experts=8, top_k=2, d_ff_expert=128),
    "qwen3_30b_a3b": dict(name="qwen3_30b_a3b", n_layers=48, d_model=2048, n_heads=32, n_kv_heads=4, head_dim=128, d_ff=0,
                          vocab_size=151936, rope_theta=1e6, rms_eps=1e-6, seq_len=4096, batch=2, grad_accum_rounds=8,
                          n_experts=128, top_k=8, d_ff_expert=768, aux_coef=0.001, dtype_policy="bf16_split_master"),
}
FAMILY = register_llama_like("qwen3moe", PRESETS, qk_norm=True, routing_mode="topk_then_softmax")
