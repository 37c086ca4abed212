"""The Qwen2 dense decoder: its configuration and its layout as parts.

Keys, defaults and refusals follow the reference's reading of ``config.json``
(``metadata``, src/safetensors.rs:609-727) and its ``check_supported``
(src/model.rs:1272-1420): biases on q, k and v, no q/k norm, no window, SwiGLU,
rotate-half RoPE over the whole head (src/model.rs:506-538).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, ClassVar, Dict, Mapping, Optional, Tuple

from .base import ConfigError, ModelConfig, real_number, register_architecture, whole_number
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    architecture: ClassVar[str] = "Qwen2ForCausalLM"
    model_types: ClassVar[Tuple[str, ...]] = ("qwen2",)

    num_hidden_layers: int = 0
    hidden_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    vocab_size: int = 0
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 0
    use_sliding_window: bool = False
    hidden_act: str = "silu"

    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "Qwen2Config":
        def need(key: str) -> int:
            v = whole_number(cfg, key)
            if v is None:
                raise ConfigError(f"config.json {key} is missing")
            return v

        act = cfg.get("hidden_act")
        if act is not None and act != "silu":
            # src/safetensors.rs:618-622
            raise ConfigError(f"hidden_act {act} is not supported (silu)")
        if cfg.get("use_sliding_window") is True:
            # src/safetensors.rs:623-625
            raise ConfigError("use_sliding_window true is not supported")
        if cfg.get("quantization_config") is not None:
            raise ConfigError("quantized checkpoints are not supported (bfloat16 or float32 weights)")

        layers = need("num_hidden_layers")
        dim = need("hidden_size")
        heads = need("num_attention_heads")
        kv_heads = whole_number(cfg, "num_key_value_heads", default=heads)
        head_dim = whole_number(cfg, "head_dim")
        if head_dim is None:
            if dim % heads:
                # src/model.rs:1297-1305
                raise ConfigError(f"hidden_size {dim} doesn't split into {heads} heads")
            head_dim = dim // heads
        if head_dim % 2:
            raise ConfigError(f"head size {head_dim} is odd")  # src/model.rs:1313
        if heads % kv_heads:
            raise ConfigError(  # src/model.rs:1316
                f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        if whole_number(cfg, "num_experts", minimum=0) or whole_number(cfg, "num_local_experts", minimum=0):
            raise ConfigError("mixture-of-experts models are not supported by Qwen2ForCausalLM")

        rope = _rope_parameters(cfg)
        ty = rope.get("rope_type", rope.get("type"))
        if ty is not None and str(ty).lower() != "default":
            # The reference maps linear / yarn / llama3 scaling for other uses; this
            # engine runs plain RoPE only and refuses the rest by name.
            raise ConfigError(f"RoPE scaling type {ty} is not supported")
        theta = real_number(rope, "rope_theta", 10000.0)  # src/model.rs:639
        if theta <= 0:
            raise ConfigError(f"config.json rope_theta = {theta} must be positive")
        eps = real_number(cfg, "rms_norm_eps", 1e-6)  # src/model.rs:1784
        if eps < 0:
            raise ConfigError(f"config.json rms_norm_eps = {eps} must not be negative")
        tie = cfg.get("tie_word_embeddings", False)
        if not isinstance(tie, bool):
            raise ConfigError(f"config.json tie_word_embeddings = {tie!r} is not true or false")

        return cls(
            num_hidden_layers=layers,
            hidden_size=dim,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=need("intermediate_size"),
            vocab_size=need("vocab_size"),
            rope_theta=theta,
            rms_norm_eps=eps,
            tie_word_embeddings=tie,
            max_position_embeddings=need("max_position_embeddings"),
            use_sliding_window=False,
            hidden_act="silu",
        )


def _rope_parameters(cfg: Mapping[str, Any]) -> Dict[str, Any]:
    """One dictionary of RoPE parameters: ``rope_scaling``, the top-level
    ``rope_theta``, then ``rope_parameters`` (its ``full_attention`` entry when it
    has one), later ones winning (reference: ``rope_params``, src/safetensors.rs:488-504)."""
    p: Dict[str, Any] = {}
    if isinstance(cfg.get("rope_scaling"), Mapping):
        p.update(cfg["rope_scaling"])
    if cfg.get("rope_theta") is not None:
        p["rope_theta"] = cfg["rope_theta"]
    rp = cfg.get("rope_parameters")
    if isinstance(rp, Mapping):
        if isinstance(rp.get("full_attention"), Mapping):
            rp = rp["full_attention"]
        p.update(rp)
    return p


def qwen2_spec(c: Qwen2Config) -> ModelSpec:
    """The Qwen2 decoder as parts, with Hugging Face tensor names
    (reference name map: src/safetensors.rs:1137-1178)."""
    rope = PartSpec("rope", {"head_dim": c.head_dim, "theta": c.rope_theta, "pairing": "half"})

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": c.hidden_size, "eps": c.rms_norm_eps}, {"gain": name})

    layers = []
    for i in range(c.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = PartSpec(
            "attention",
            {"hidden_size": c.hidden_size, "heads": c.num_attention_heads,
             "kv_heads": c.num_key_value_heads, "head_dim": c.head_dim,
             "qkv_bias": True, "out_bias": False, "window": None,
             "scale": None},
            {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
             "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight",
             "q_bias": p + "self_attn.q_proj.bias", "k_bias": p + "self_attn.k_proj.bias",
             "v_bias": p + "self_attn.v_proj.bias"},
            {"position": rope})
        ffn = PartSpec(
            "swiglu",
            {"hidden_size": c.hidden_size, "intermediate_size": c.intermediate_size},
            {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
             "down": p + "mlp.down_proj.weight"})
        layers.append(LayerSpec("prenorm", {
            "norm_mixer": norm(p + "input_layernorm.weight"),
            "mixer": mixer,
            "norm_ffn": norm(p + "post_attention_layernorm.weight"),
            "ffn": ffn,
        }))
    embedding = PartSpec("embedding", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size},
                         {"table": "model.embed_tokens.weight"})
    head = PartSpec(
        "linear_head", {"vocab_size": c.vocab_size, "hidden_size": c.hidden_size},
        # a tied head reads the embedding table (src/model.rs:1799-1803)
        {"weight": "model.embed_tokens.weight" if c.tie_word_embeddings else "lm_head.weight"})
    spec = ModelSpec(
        architecture=c.architecture,
        hidden_size=c.hidden_size,
        vocab_size=c.vocab_size,
        max_positions=c.max_position_embeddings,
        embedding=embedding,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(c.num_hidden_layers)),
        final_norm=norm("model.norm.weight"),
        head=head,
        # ``rotary_emb.inv_freq`` is skipped (src/safetensors.rs:1157-1159); a tied
        # model that still stores a head does not use it
        ignored_suffixes=("self_attn.rotary_emb.inv_freq",)
        + (("lm_head.weight",) if c.tie_word_embeddings else ()),
    )
    spec.validate()
    return spec


register_architecture(Qwen2Config, qwen2_spec)
