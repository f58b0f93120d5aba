"""The LFM3 hybrid decoder as a plan: which parts each layer has, in which order layers run,
and what their tensors are called.

Layer l (src/dense.rs:178-194): operator_norm -> mixer -> (+) -> ffn_norm -> feed-forward -> (+).
The mixer is the short convolution where layer_types[l] is conv, grouped-query attention
with per-head q/k norm and split-half rotary positions where it is attention
(src/dense.rs:61-64 decides the same from the kv-head count).  The feed-forward is dense
SwiGLU, or routed experts from layer num_dense_layers on.  Tensor names are the
architecture's checkpoint names; a leading "model." is accepted and dropped.
"""
from __future__ import annotations

from ..config.lfm3 import CONV, SLIDING, Lfm3Config
from ..parts.base import LayerSpec, ModelPlan, PartSpec, ScheduleEntry
from ..registry import ARCHITECTURES

NAMES = ("Lfm3ForCausalLM", "lfm3", "Lfm2ForCausalLM", "lfm2", "Lfm2MoeForCausalLM", "lfm2_moe")


def _alias(name: str) -> str:
    return name[len("model."):] if name.startswith("model.") else name


def lfm3_plan(cfg: Lfm3Config) -> ModelPlan:
    D = cfg.hidden_size
    norm = PartSpec("rmsnorm", {"size": D, "eps": cfg.norm_eps})
    layers: list[LayerSpec] = []
    for l, kind in enumerate(cfg.layer_types):
        if kind == CONV:
            mixer = PartSpec("shortconv", {"hidden_size": D, "L_cache": cfg.conv_L_cache, "bias": cfg.conv_bias})
            mixer_name = "conv"
        else:
            sliding = kind == SLIDING
            theta = cfg.rope_theta_swa if sliding else cfg.rope_theta  # src/dense.rs:124
            mixer = PartSpec("attention", {
                "hidden_size": D, "num_heads": cfg.num_attention_heads,
                "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                "norm_eps": cfg.norm_eps, "qk_norm": True,
                # the model's frequency factors divide the angles of layers without a window (src/dense.rs:125)
                "position": PartSpec("rope", {"rope_dim": cfg.rope_dim, "theta": theta, "style": "neox",
                                              "freq_factors": not sliding}),
                "window": cfg.sliding_window if sliding else 0,
                "output_gate": cfg.attn_output_gate})
            mixer_name = "self_attn"
        if cfg.layer_is_moe(l):
            ffn = PartSpec("sigmoid_topk_moe", {
                "hidden_size": D, "num_experts": cfg.num_experts, "top_k": cfg.num_experts_per_tok,
                "expert_size": cfg.moe_intermediate_size, "norm_topk": cfg.norm_topk_prob,
                "use_bias": cfg.use_expert_bias, "scaling": cfg.routed_scaling_factor})
        else:
            ffn = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": cfg.ffn_dim})
        layers.append(LayerSpec(
            prefix=f"layers.{l}", mixer=mixer, ffn=ffn, mixer_norm=norm, ffn_norm=norm,
            post_mixer_norm=norm if cfg.sandwich_norms else None,
            post_ffn_norm=norm if cfg.sandwich_norms else None,
            names={"mixer": mixer_name, "ffn": "feed_forward", "mixer_norm": "operator_norm",
                   "ffn_norm": "ffn_norm", "post_mixer_norm": "post_mixer_norm",
                   "post_ffn_norm": "post_ffn_norm"}))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab_size,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": D}),
        final_norm=norm,
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "hidden_size": D,
                                      "tied": cfg.tie_embedding}),
        layers=layers, schedule=[ScheduleEntry(i) for i in range(len(layers))],
        eos_token_ids=cfg.eos_token_ids,
        names={"embedding": "embed_tokens", "final_norm": "embedding_norm", "head": "lm_head"},
        tensor_aliases=_alias,
        # the rotary frequency factors belong to the layers without a window; a model without such a
        # layer may still carry them (the reference reads them if present and uses them there only,
        # src/dense.rs:125)
        unused_tensors=("rope_freqs.weight",))


@ARCHITECTURES.register(*NAMES)
def build_lfm3(raw: dict) -> ModelPlan:
    return lfm3_plan(Lfm3Config.from_dict(raw))
