"""Small configurations for the tests.  A and B differ in every size and option:
depth, layer pattern, width, head counts and grouping, head size, feed-forward kind and
width, vocabulary, rope base, convolution length, eps, tied or own output matrix.
C is A's shape with the reference's own lfm3 options switched on (norms after mixer and
feed-forward, per-head output gate, a sliding window with its own rope base).
D has the two optional tensors: a bias in the short convolution and the model's rotary frequency
factors (which the layer with a window must not use), three query heads per kv head, a rotation
over half of the head only, and a convolution of length 5.
"""

TINY_A = {
    "architectures": ["Lfm3ForCausalLM"], "model_type": "lfm3",
    "vocab_size": 256, "hidden_size": 64, "num_hidden_layers": 4,
    "layer_types": ["conv", "attention", "conv", "attention"],
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 128, "block_auto_adjust_ff_dim": False,
    "rope_theta": 10000.0, "conv_L_cache": 3, "norm_eps": 1e-5, "tie_embedding": True,
    "max_position_embeddings": 4096, "eos_token_id": 7,
}

TINY_B = {
    "architectures": ["Lfm3ForCausalLM"], "model_type": "lfm3",
    "vocab_size": 384, "hidden_size": 96, "num_hidden_layers": 6,
    "layer_types": ["conv", "conv", "attention", "conv", "conv", "attention"],
    "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32,
    "intermediate_size": 240, "block_auto_adjust_ff_dim": True, "block_multiple_of": 32,
    "block_ffn_dim_multiplier": 1.0,                     # 240 -> 160 -> 160
    "num_experts": 8, "num_experts_per_tok": 2, "moe_intermediate_size": 48, "num_dense_layers": 1,
    "norm_topk_prob": True, "use_expert_bias": True, "routed_scaling_factor": 1.0,
    "rope_theta": 1000000.0, "conv_L_cache": 4, "norm_eps": 1e-6, "tie_embedding": False,
    "max_position_embeddings": 4096,
}

TINY_C = {
    "architectures": ["Lfm3ForCausalLM"], "model_type": "lfm3",
    "vocab_size": 200, "hidden_size": 80, "num_hidden_layers": 3,
    "layer_types": ["sliding_attention", "conv", "attention"],
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48, "rope_dim": 32,
    "intermediate_size": 72, "rope_theta": 50000.0, "rope_theta_swa": 10000.0,
    "sliding_window": 24, "conv_L_cache": 2, "norm_eps": 1e-5, "tie_embedding": True,
    "sandwich_norms": True, "attn_output_gate": True,
    "num_experts": 4, "num_experts_per_tok": 1, "moe_intermediate_size": 40, "num_dense_layers": 2,
    "norm_topk_prob": False, "use_expert_bias": False, "routed_scaling_factor": 1.5,
}

TINY_D = {
    "architectures": ["Lfm3ForCausalLM"], "model_type": "lfm3",
    "vocab_size": 300, "hidden_size": 72, "num_hidden_layers": 4,
    "layer_types": ["conv", "attention", "sliding_attention", "conv"],
    "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32, "rope_dim": 16,
    "intermediate_size": 104, "rope_theta": 200000.0, "rope_theta_swa": 30000.0,
    "sliding_window": 40, "conv_L_cache": 5, "conv_bias": True, "norm_eps": 1e-6, "tie_embedding": False,
}
