"""Configuration of the LFM3 hybrid decoder, read from the architecture's own config.json keys.

The reference fills the same quantities from `lfm3.*` GGUF keys (src/dense.rs:52-77):
layer kinds per layer (`:61-64`), head counts (`:57-65`), head size with the default
hidden/heads (`:69`), rope dimension (`:72`), norm epsilon default 1e-5 and rope base
default 10000 (`:73`), the sliding window and its own rope base (`:74-75`) and the
short convolution's length (`:76`).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from .base import ConfigError, KeyReader

CONV = "conv"
ATTENTION = "attention"
SLIDING = "sliding_attention"

# spellings of a layer's kind that config.json files of this family use
_LAYER_KIND = {
    "conv": CONV,
    "attention": ATTENTION,
    "full_attention": ATTENTION,
    "sliding_attention": SLIDING,
}


@dataclass(frozen=True)
class Lfm3Config:
    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    layer_types: tuple[str, ...]
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rope_dim: int
    rope_theta: float
    rope_theta_swa: float
    norm_eps: float
    max_position_embeddings: int
    # short convolution
    conv_L_cache: int
    conv_bias: bool
    # dense feed-forward: the width actually used, after the block_* adjustment
    intermediate_size: int
    ffn_dim: int
    # experts (num_experts == 0: every layer is dense)
    num_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    num_dense_layers: int
    norm_topk_prob: bool
    use_expert_bias: bool
    routed_scaling_factor: float
    # output
    tie_embedding: bool
    # options of the reference's own lfm3 (off unless config.json turns them on)
    sandwich_norms: bool
    attn_output_gate: bool
    sliding_window: int
    # generation defaults
    eos_token_ids: tuple[int, ...]
    bos_token_id: int | None
    raw: dict = field(compare=False, repr=False, default_factory=dict)

    @property
    def attention_layers(self) -> list[int]:
        return [i for i, k in enumerate(self.layer_types) if k != CONV]

    @property
    def conv_layers(self) -> list[int]:
        return [i for i, k in enumerate(self.layer_types) if k == CONV]

    def layer_is_moe(self, layer: int) -> bool:
        return self.num_experts > 0 and layer >= self.num_dense_layers

    @staticmethod
    def from_dict(raw: dict[str, Any], where: str = "config.json") -> "Lfm3Config":
        r = KeyReader(raw, where)
        from .base import architecture_name

        arch = architecture_name(raw)
        V = r.integer("vocab_size", minimum=1)
        D = r.integer("hidden_size", minimum=1)
        L = r.integer("num_hidden_layers", minimum=1)
        nh = r.integer("num_attention_heads", minimum=1)
        nkv = r.integer("num_key_value_heads", default=nh, minimum=1)

        if r.has("layer_types"):
            lt = r.array("layer_types", item=lambda e: isinstance(e, str))
            kinds = []
            for i, name in enumerate(lt):
                if name not in _LAYER_KIND:
                    raise ConfigError(
                        f"{where}: 'layer_types'[{i}] is '{name}'; known kinds: {sorted(_LAYER_KIND)}")
                kinds.append(_LAYER_KIND[name])
        elif r.has("full_attn_idxs"):
            idx = r.array("full_attn_idxs", item=lambda e: isinstance(e, int) and not isinstance(e, bool))
            bad = [i for i in idx if not 0 <= i < L]
            if bad:
                raise ConfigError(f"{where}: 'full_attn_idxs' names layers {bad} outside 0..{L - 1}")
            kinds = [ATTENTION if i in set(idx) else CONV for i in range(L)]
        else:
            raise ConfigError(f"{where}: missing required key 'layer_types' (one of "
                              f"{sorted(set(_LAYER_KIND))} per layer)")
        if len(kinds) != L:
            raise ConfigError(f"{where}: 'layer_types' has {len(kinds)} entries but "
                              f"'num_hidden_layers' is {L}")

        if nh % nkv != 0:
            raise ConfigError(f"{where}: 'num_attention_heads' ({nh}) must be a multiple of "
                              f"'num_key_value_heads' ({nkv})")
        if r.has("head_dim"):
            hd = r.integer("head_dim", minimum=1)
        else:
            if D % nh != 0:
                raise ConfigError(f"{where}: 'hidden_size' ({D}) is not a multiple of "
                                  f"'num_attention_heads' ({nh}); give 'head_dim'")
            hd = D // nh
        rope_dim = r.integer("rope_dim", default=hd, minimum=2)
        if rope_dim > hd or rope_dim % 2 != 0:
            raise ConfigError(f"{where}: 'rope_dim' ({rope_dim}) must be even and at most "
                              f"'head_dim' ({hd})")

        theta = None
        if r.has("rope_theta"):
            theta = r.number("rope_theta")
        elif isinstance(raw.get("rope_parameters"), dict) and "rope_theta" in raw["rope_parameters"]:
            r.used.add("rope_parameters")
            theta = float(raw["rope_parameters"]["rope_theta"])
        if theta is None:
            theta = 10000.0  # the reference's default (src/dense.rs:73)
        if theta <= 0:
            raise ConfigError(f"{where}: 'rope_theta' must be positive, got {theta}")
        theta_swa = r.number("rope_theta_swa", default=10000.0)  # src/dense.rs:74
        eps = r.number("norm_eps", "rms_norm_eps", default=1e-5)
        if eps < 0:
            raise ConfigError(f"{where}: 'norm_eps' must not be negative, got {eps}")
        max_pos = r.integer("max_position_embeddings", default=128000, minimum=1)

        has_conv = any(k == CONV for k in kinds)
        lc = r.integer("conv_L_cache", default=0 if not has_conv else None)
        if has_conv:
            if lc is None:
                raise ConfigError(f"{where}: missing required key 'conv_L_cache' "
                                  f"(layer_types has conv layers)")
            if lc < 2:
                raise ConfigError(f"{where}: 'conv_L_cache' must be at least 2, got {lc}")
        conv_bias = r.boolean("conv_bias", default=False)

        inter = r.integer("intermediate_size", "block_ff_dim", minimum=1)
        ffn = inter
        if r.boolean("block_auto_adjust_ff_dim", default=False):
            ffn = int(2 * ffn / 3)
            mult = r.number("block_ffn_dim_multiplier", default=None)
            if mult is not None:
                ffn = int(mult * ffn)
            mo = r.integer("block_multiple_of", default=1, minimum=1)
            ffn = mo * ((ffn + mo - 1) // mo)

        E = r.integer("num_experts", default=0, minimum=0)
        if E > 0:
            k = r.integer("num_experts_per_tok", minimum=1)
            fe = r.integer("moe_intermediate_size", minimum=1)
            nd = r.integer("num_dense_layers", default=0, minimum=0)
            if k > E:
                raise ConfigError(f"{where}: 'num_experts_per_tok' ({k}) exceeds 'num_experts' ({E})")
        else:
            k, fe, nd = 0, 0, L
        norm_topk = r.boolean("norm_topk_prob", default=True)
        use_bias = r.boolean("use_expert_bias", default=True)
        scale = r.number("routed_scaling_factor", default=1.0)

        tie = r.boolean("tie_embedding", "tie_word_embeddings", default=True)
        sandwich = r.boolean("sandwich_norms", default=False)
        gate = r.boolean("attn_output_gate", default=False)
        window = r.integer("sliding_window", default=0, minimum=0)
        if r.has("sliding_window_pattern"):
            pat = r.array("sliding_window_pattern")
            if len(pat) != L:
                raise ConfigError(f"{where}: 'sliding_window_pattern' has {len(pat)} entries, "
                                  f"expected {L}")
            for i, p in enumerate(pat):
                if p in (1, True) and kinds[i] == ATTENTION:
                    kinds[i] = SLIDING  # the reference's per-layer flag, src/dense.rs:60-63
        if any(k_ == SLIDING for k_ in kinds) and window <= 0:
            raise ConfigError(f"{where}: a layer is '{SLIDING}' but 'sliding_window' is not set")

        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"{where}: 'eos_token_id' must be an integer or a list of integers")
        bos = r.integer("bos_token_id", default=None)

        return Lfm3Config(
            architecture=arch, vocab_size=V, hidden_size=D, num_hidden_layers=L,
            layer_types=tuple(kinds), num_attention_heads=nh, num_key_value_heads=nkv,
            head_dim=hd, rope_dim=rope_dim, rope_theta=theta, rope_theta_swa=theta_swa,
            norm_eps=eps, max_position_embeddings=max_pos, conv_L_cache=lc or 0,
            conv_bias=conv_bias, intermediate_size=inter, ffn_dim=ffn, num_experts=E,
            num_experts_per_tok=k, moe_intermediate_size=fe, num_dense_layers=nd,
            norm_topk_prob=norm_topk, use_expert_bias=use_bias, routed_scaling_factor=scale,
            tie_embedding=tie, sandwich_norms=sandwich, attn_output_gate=gate,
            sliding_window=window, eos_token_ids=eos_ids, bos_token_id=bos, raw=dict(raw))
