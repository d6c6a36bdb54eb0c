"""Typed configuration of the Llama 4 text decoder, read from its config.json keys.

What giveen/spite reads from GGUF metadata into one flat struct
(crates/spite-loader/src/config.rs:124-344, crates/spite-models/src/lib.rs:58-144)
and partly hard-codes in the model (NoPE period 4, temperature constants 8192 and
0.1, QK-norm by expert count: crates/spite-models/src/llama/llama4.rs:95-96,179) is
all configuration data here.
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import Optional

from .registry import register_architecture
from .specs import BlockSpec, ConfigError, LayerCall, ModelPlan, PartSpec


@dataclass(frozen=True)
class WeightBinding:
    """A parameter of the plan and the checkpoint tensor that fills it."""
    target: str                 # e.g. "layers.3.ffn.experts_down"
    source: str                 # checkpoint tensor name
    source_shape: tuple         # exact shape expected in the file
    transform: Optional[str] = None   # a registered weight transform (spite_b200.weights.register_weight_transform)
    init: str = "normal"        # how the random-weights mode fills it: "normal" | "ones"


@dataclass(frozen=True)
class RopeScaling:
    """`rope_scaling` of rope_type "llama3"."""
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int


def _need(d, key):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key `{key}` is missing")
    return d[key]


@register_architecture("Llama4ForCausalLM", "Llama4ForConditionalGeneration", model_types=("llama4_text", "llama4"))
@dataclass(frozen=True)
class Llama4Config:
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int               # width of one routed expert and of the shared expert
    intermediate_size_mlp: int           # width of the dense feed-forward of non-MoE layers
    num_local_experts: int
    num_experts_per_tok: int
    moe_layers: tuple                    # indices of the layers whose feed-forward is MoE
    no_rope_layers: tuple                # per layer: 1 = rotary + chunked attention, 0 = NoPE + global attention
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    attention_chunk_size: int
    use_qk_norm: bool
    attn_temperature_tuning: bool
    floor_scale: float
    attn_scale: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    interleave_moe_layer_step: int = 1
    no_rope_layer_interval: int = 4
    architecture: str = "Llama4ForCausalLM"
    eos_token_id: Optional[tuple] = None
    extra: dict = field(default_factory=dict, compare=False)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, raw: dict) -> "Llama4Config":
        arch = (raw.get("architectures") or ["Llama4ForCausalLM"])[0]
        d = dict(raw.get("text_config") or raw)
        n_layers = int(_need(d, "num_hidden_layers"))
        hidden = int(_need(d, "hidden_size"))
        nq = int(_need(d, "num_attention_heads"))
        nkv = int(d.get("num_key_value_heads") or nq)
        if nq <= 0:
            raise ConfigError("num_attention_heads must be positive")
        head_dim = int(d.get("head_dim") or hidden // nq)
        step = int(d.get("interleave_moe_layer_step", 1))
        if d.get("moe_layers") is not None:
            moe_layers = tuple(int(x) for x in d["moe_layers"])
        else:
            # crates/spite-models/src/llama/llama4.rs:44-47
            moe_layers = tuple(L for L in range(n_layers) if step > 0 and (L + 1) % step == 0)
        interval = int(d.get("no_rope_layer_interval", 4))
        if d.get("no_rope_layers"):
            no_rope = tuple(int(x) for x in d["no_rope_layers"])
        else:
            # crates/spite-models/src/llama/llama4.rs:155
            if interval < 1:
                raise ConfigError("no_rope_layer_interval must be >= 1")
            no_rope = tuple(int((L + 1) % interval != 0) for L in range(n_layers))
        sc = d.get("rope_scaling")
        scaling = None
        if sc:
            kind = sc.get("rope_type", sc.get("type", "llama3"))
            if kind != "llama3":
                raise ConfigError(f"rope_scaling type {kind!r} is not supported (only 'llama3')")
            scaling = RopeScaling(
                factor=float(_need(sc, "factor")),
                low_freq_factor=float(sc.get("low_freq_factor", 1.0)),
                high_freq_factor=float(sc.get("high_freq_factor", 4.0)),
                original_max_position_embeddings=int(_need(sc, "original_max_position_embeddings")))
        n_experts = int(d.get("num_local_experts", 0) or 0)
        eos = d.get("eos_token_id", raw.get("eos_token_id"))
        if isinstance(eos, int):
            eos = (eos,)
        elif eos is not None:
            eos = tuple(int(x) for x in eos)
        cfg = cls(
            vocab_size=int(_need(d, "vocab_size")),
            hidden_size=hidden,
            num_hidden_layers=n_layers,
            num_attention_heads=nq,
            num_key_value_heads=nkv,
            head_dim=head_dim,
            intermediate_size=int(d.get("intermediate_size") or 0),
            intermediate_size_mlp=int(d.get("intermediate_size_mlp") or d.get("intermediate_size") or 0),
            num_local_experts=n_experts,
            num_experts_per_tok=int(d.get("num_experts_per_tok", 1)),
            moe_layers=moe_layers,
            no_rope_layers=no_rope,
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=scaling,
            attention_chunk_size=int(d.get("attention_chunk_size") or 8192),
            use_qk_norm=bool(d.get("use_qk_norm", True)),
            attn_temperature_tuning=bool(d.get("attn_temperature_tuning", True)),
            floor_scale=float(d.get("floor_scale", 8192)),
            attn_scale=float(d.get("attn_scale", 0.1)),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", raw.get("tie_word_embeddings", False))),
            max_position_embeddings=int(d.get("max_position_embeddings", 131072)),
            interleave_moe_layer_step=step,
            no_rope_layer_interval=interval,
            architecture=arch,
            eos_token_id=eos,
        )
        cfg.validate()
        return cfg

    def validate(self):
        c = self
        pos = {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size,
               "num_hidden_layers": c.num_hidden_layers, "num_attention_heads": c.num_attention_heads,
               "num_key_value_heads": c.num_key_value_heads, "head_dim": c.head_dim,
               "attention_chunk_size": c.attention_chunk_size,
               "max_position_embeddings": c.max_position_embeddings}
        for k, v in pos.items():
            if v <= 0:
                raise ConfigError(f"`{k}` must be positive, got {v}")
        if c.num_attention_heads % c.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {c.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {c.num_key_value_heads}")
        if c.head_dim % 2:
            raise ConfigError(f"head_dim {c.head_dim} must be even (rotary pairs)")
        if len(c.no_rope_layers) != c.num_hidden_layers:
            raise ConfigError(
                f"no_rope_layers has {len(c.no_rope_layers)} entries for {c.num_hidden_layers} layers")
        for L in c.moe_layers:
            if not 0 <= L < c.num_hidden_layers:
                raise ConfigError(f"moe_layers names layer {L}, model has {c.num_hidden_layers}")
        if c.moe_layers:
            if c.num_local_experts < 1:
                raise ConfigError("MoE layers need num_local_experts >= 1")
            if not 1 <= c.num_experts_per_tok <= c.num_local_experts:
                raise ConfigError(
                    f"num_experts_per_tok {c.num_experts_per_tok} must lie in 1..{c.num_local_experts}")
            if c.intermediate_size <= 0:
                raise ConfigError("MoE layers need intermediate_size > 0")
        if len(c.moe_layers) < c.num_hidden_layers and c.intermediate_size_mlp <= 0:
            raise ConfigError("dense layers need intermediate_size_mlp > 0")
        if c.rms_norm_eps <= 0:
            raise ConfigError("rms_norm_eps must be positive")
        if c.floor_scale < 1:
            raise ConfigError("floor_scale must be >= 1")
        s = c.rope_scaling
        if s is not None:
            if s.factor <= 0 or s.low_freq_factor <= 0 or s.high_freq_factor <= 0:
                raise ConfigError("rope_scaling factors must be positive")
            if s.high_freq_factor < s.low_freq_factor:
                raise ConfigError("rope_scaling: high_freq_factor < low_freq_factor")
            if s.original_max_position_embeddings <= 0:
                raise ConfigError("rope_scaling.original_max_position_embeddings must be positive")

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = asdict(self)
        d.pop("extra")
        arch = d.pop("architecture")
        d["architectures"] = [arch]
        d["model_type"] = "llama4_text"
        d["moe_layers"] = list(self.moe_layers)
        d["no_rope_layers"] = list(self.no_rope_layers)
        if self.rope_scaling is not None:
            d["rope_scaling"] = dict(asdict(self.rope_scaling), rope_type="llama3")
        if self.eos_token_id is not None:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    # ------------------------------------------------------------------ the plan
    def is_moe_layer(self, L: int) -> bool:
        return L in self.moe_layers

    def uses_rope(self, L: int) -> bool:
        return bool(self.no_rope_layers[L])

    def plan(self) -> ModelPlan:
        c = self
        norm = PartSpec("rms_norm", {"size": c.hidden_size, "eps": c.rms_norm_eps})
        rope = PartSpec("rotary_interleaved", {
            "head_dim": c.head_dim, "theta": c.rope_theta,
            "scaling": None if c.rope_scaling is None else asdict(c.rope_scaling)})
        nope = PartSpec("no_position", {})
        blocks = []
        for L in range(c.num_hidden_layers):
            common = {"hidden_size": c.hidden_size, "num_heads": c.num_attention_heads,
                      "num_kv_heads": c.num_key_value_heads, "head_dim": c.head_dim}
            if c.uses_rope(L):
                mixer = PartSpec("paged_attention", dict(
                    common, position=rope, window=("chunk", c.attention_chunk_size),
                    qk_norm_eps=c.rms_norm_eps if c.use_qk_norm else None,
                    temperature_tuning=None))
            else:
                mixer = PartSpec("paged_attention", dict(
                    common, position=nope, window=("full", 0), qk_norm_eps=None,
                    temperature_tuning=(c.floor_scale, c.attn_scale) if c.attn_temperature_tuning else None))
            if c.is_moe_layer(L):
                ffn = PartSpec("moe_sigmoid_prescaled", {
                    "hidden_size": c.hidden_size, "num_experts": c.num_local_experts,
                    "top_k": c.num_experts_per_tok, "expert_size": c.intermediate_size,
                    "shared_size": c.intermediate_size})
            else:
                ffn = PartSpec("dense_swiglu", {
                    "hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size_mlp})
            blocks.append(BlockSpec("prenorm_residual", {"mixer_norm": norm, "mixer": mixer, "ffn_norm": norm, "ffn": ffn}))
        order = tuple(LayerCall(L, L, True) for L in range(c.num_hidden_layers))
        return ModelPlan(hidden_size=c.hidden_size, vocab_size=c.vocab_size, blocks=tuple(blocks),
                         order=order, final_norm=norm, tie_word_embeddings=c.tie_word_embeddings,
                         max_positions=c.max_position_embeddings).validate()

    # ------------------------------------------------------------------ tensor names
    def weight_bindings(self) -> list[WeightBinding]:
        """Checkpoint tensor names and shapes (the public checkpoint convention:
        projections `[out, in]`; the stacked experts input-major, `gate_up_proj
        [E, d, 2f]` with the gate columns first and `down_proj [E, f, d]`), bound
        to the plan's parameters, which are all `[out, in]`."""
        c = self
        d, hd = c.hidden_size, c.head_dim
        nq, nkv = c.num_attention_heads, c.num_key_value_heads
        B = WeightBinding
        out = [B("embed.weight", "model.embed_tokens.weight", (c.vocab_size, d))]
        for L in range(c.num_hidden_layers):
            s, t = f"model.layers.{L}.", f"layers.{L}."
            out += [
                B(t + "mixer_norm.weight", s + "input_layernorm.weight", (d,), init="ones"),
                B(t + "mixer.q_proj", s + "self_attn.q_proj.weight", (nq * hd, d)),
                B(t + "mixer.k_proj", s + "self_attn.k_proj.weight", (nkv * hd, d)),
                B(t + "mixer.v_proj", s + "self_attn.v_proj.weight", (nkv * hd, d)),
                B(t + "mixer.o_proj", s + "self_attn.o_proj.weight", (d, nq * hd)),
                B(t + "ffn_norm.weight", s + "post_attention_layernorm.weight", (d,), init="ones"),
            ]
            if c.is_moe_layer(L):
                E, f = c.num_local_experts, c.intermediate_size
                out += [
                    B(t + "ffn.router", s + "feed_forward.router.weight", (E, d)),
                    B(t + "ffn.experts_gate_up", s + "feed_forward.experts.gate_up_proj", (E, d, 2 * f),
                      transform="transpose_last2"),
                    B(t + "ffn.experts_down", s + "feed_forward.experts.down_proj", (E, f, d),
                      transform="transpose_last2"),
                    B(t + "ffn.shared_gate_proj", s + "feed_forward.shared_expert.gate_proj.weight", (f, d)),
                    B(t + "ffn.shared_up_proj", s + "feed_forward.shared_expert.up_proj.weight", (f, d)),
                    B(t + "ffn.shared_down_proj", s + "feed_forward.shared_expert.down_proj.weight", (d, f)),
                ]
            else:
                f = c.intermediate_size_mlp
                out += [
                    B(t + "ffn.gate_proj", s + "feed_forward.gate_proj.weight", (f, d)),
                    B(t + "ffn.up_proj", s + "feed_forward.up_proj.weight", (f, d)),
                    B(t + "ffn.down_proj", s + "feed_forward.down_proj.weight", (d, f)),
                ]
        out.append(B("final_norm.weight", "model.norm.weight", (d,), init="ones"))
        if not c.tie_word_embeddings:
            out.append(B("head.weight", "lm_head.weight", (c.vocab_size, d)))
        return out

    #: tensor-name prefixes under which a checkpoint may store the text decoder
    checkpoint_prefixes = ("", "language_model.")
    #: tensors of other towers of a multimodal checkpoint; never reported as unexpected
    ignored_prefixes = ("vision_model.", "multi_modal_projector.")
