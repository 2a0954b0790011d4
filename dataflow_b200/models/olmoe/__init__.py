"""olmoe family: llama-style attention with an RMSNorm over the whole projected q row and k row
(all heads at once, ``qk_norm="full"``) and a mixture-of-experts MLP (softmax over all
experts, then top-k, un-normalised), load-balance auxiliary gradient.  ``olmoe_1b_7b`` is the 16-layer, 64-expert,
top-8 model.  Family parity: reference ``src/dataflow_training/model_families/olmoe/``."""
from .._llama_like import register_llama_like

PRESETS = {
    "tiny": dict(name="tiny", n_layers=2, d_model=256, n_heads=4, n_kv_heads=4, head_dim=64, d_ff=0, vocab_size=1024,
                 seq_len=128, batch=2, grad_accum_rounds=2, n_experts=8, top_k=2, d_ff_expert=128),
    "olmoe_smoke": dict(name="olmoe_smoke", n_layers=4, d_model=256, n_heads=4, n_kv_heads=4, head_dim=64, d_ff=0,
                        vocab_size=50304, seq_len=1024, batch=2, grad_accum_rounds=2, n_experts=8, top_k=2, d_ff_expert=512),
    "olmoe_1b_7b": dict(name="olmoe_1b_7b", n_layers=16, d_model=2048, n_heads=16, n_kv_heads=16, head_dim=128, d_ff=0,
                        vocab_size=50304, rope_theta=10000.0, seq_len=4096, batch=4, grad_accum_rounds=4, n_experts=64,
                        top_k=8, d_ff_expert=1024, aux_coef=0.01, dtype_policy="bf16_split_master"),
}
FAMILY = register_llama_like("olmoe", PRESETS, qk_norm="full", routing_mode="softmax_then_topk")
