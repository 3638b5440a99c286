"""Typed configuration of the Llama dense GQA decoder, read from config.json keys.

Keys, meanings and defaults follow the reference's Llama path
(crates/spissa-runtime/src/models/llama/api.rs:126-171): ``num_key_value_heads``
defaults to the head count, ``rms_norm_eps`` to 1e-5, ``rope_theta`` to 10000,
``max_position_embeddings`` to 2048, ``head_dim`` to hidden / heads; hidden must be
divisible by heads and heads by kv heads (api.rs:39-65).

Beyond the reference: ``head_dim`` is honoured as its own number, ``rope_scaling``
of type ``llama3`` is applied (the reference drops it,
crates/spissa-import/src/safetensors.rs:163-175), ``tie_word_embeddings`` decides
whether ``lm_head.weight`` is expected, and ``num_hidden_layers`` is required
instead of probing tensor names (api.rs:185-196).
"""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Optional

from .spec import LayerSpec, ModelSpec, PartSpec, default_schedule
from .registry import register_architecture


class ConfigError(ValueError):
    pass


def _require(d: dict, key: str, kind=int):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json is missing required field {key!r}")
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json field {key!r} must be an integer, got {v!r}")
    return v


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of config.json. ``rope_type`` is "llama3" or "linear"."""
    rope_type: str
    factor: float
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @staticmethod
    def from_dict(d: Optional[dict]) -> Optional["RopeScaling"]:
        if not d:
            return None
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind == "llama3":
            for k in ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings"):
                if k not in d:
                    raise ConfigError(f"rope_scaling of type llama3 is missing {k!r}")
            if d["high_freq_factor"] == d["low_freq_factor"]:
                raise ConfigError("rope_scaling: high_freq_factor must differ from low_freq_factor")
            return RopeScaling("llama3", float(d["factor"]), float(d["low_freq_factor"]),
                               float(d["high_freq_factor"]), int(d["original_max_position_embeddings"]))
        if kind == "linear":
            if "factor" not in d:
                raise ConfigError("rope_scaling of type linear is missing 'factor'")
            return RopeScaling("linear", float(d["factor"]))
        raise ConfigError(f"unsupported rope_scaling type {kind!r} (supported: llama3, linear, default)")

    def to_dict(self) -> dict:
        if self.rope_type == "linear":
            return {"rope_type": "linear", "factor": self.factor}
        return {"rope_type": self.rope_type, "factor": self.factor,
                "low_freq_factor": self.low_freq_factor, "high_freq_factor": self.high_freq_factor,
                "original_max_position_embeddings": self.original_max_position_embeddings}


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    max_position_embeddings: int
    tie_word_embeddings: bool
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[object] = None      # an int or a list of ints, as config.json has it

    architecture = "LlamaForCausalLM"
    model_type = "llama"

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        H = _require(d, "hidden_size")
        nh = _require(d, "num_attention_heads")
        nkv = d.get("num_key_value_heads")
        if nkv is None:
            nkv = nh
        head_dim = d.get("head_dim")
        if head_dim is None:
            if nh <= 0 or H % nh:
                raise ConfigError(f"hidden_size {H} must be divisible by num_attention_heads {nh}")
            head_dim = H // nh
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key):
                raise ConfigError(f"{key}=true is not supported by this architecture's parts")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported (silu only)")
        cfg = cls(
            vocab_size=_require(d, "vocab_size"),
            hidden_size=H,
            intermediate_size=_require(d, "intermediate_size"),
            num_hidden_layers=_require(d, "num_hidden_layers"),
            num_attention_heads=nh,
            num_key_value_heads=int(nkv),
            head_dim=int(head_dim),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5)),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=RopeScaling.from_dict(d.get("rope_scaling")),
            max_position_embeddings=int(d.get("max_position_embeddings", 2048)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            bos_token_id=d.get("bos_token_id"),
            eos_token_id=d.get("eos_token_id"),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        pos = dict(vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                   intermediate_size=self.intermediate_size, num_hidden_layers=self.num_hidden_layers,
                   num_attention_heads=self.num_attention_heads,
                   num_key_value_heads=self.num_key_value_heads, head_dim=self.head_dim,
                   max_position_embeddings=self.max_position_embeddings)
        for k, v in pos.items():
            if v <= 0:
                raise ConfigError(f"{k} must be positive, got {v}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"num_attention_heads {self.num_attention_heads} must be a multiple of "
                              f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary pairs")
        if not (self.rms_norm_eps >= 0.0):
            raise ConfigError(f"rms_norm_eps must be non-negative, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0.0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")

    def to_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": self.model_type,
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "mlp_bias": False,
            "torch_dtype": "bfloat16",
        }
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    def stop_token_ids(self) -> list:
        e = self.eos_token_id
        if e is None:
            return []
        return [int(x) for x in e] if isinstance(e, (list, tuple)) else [int(e)]

    # ------------------------------------------------------------------ model
    def to_spec(self) -> ModelSpec:
        """Every layer: pre-norm block of GQA attention with rotary positions and SwiGLU."""
        rope = PartSpec("rotary", dict(
            theta=self.rope_theta, rotary_dim=self.head_dim,
            scaling=self.rope_scaling.to_dict() if self.rope_scaling else None))
        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            norm = lambda name: PartSpec("rmsnorm", dict(size=self.hidden_size, eps=self.rms_norm_eps),
                                         prefix=p + name + ".")
            layers.append(LayerSpec(
                block="prenorm",
                mixer=PartSpec("attention", dict(
                    hidden_size=self.hidden_size, num_heads=self.num_attention_heads,
                    num_kv_heads=self.num_key_value_heads, head_dim=self.head_dim,
                    position=rope, window=None), prefix=p + "self_attn."),
                ffn=PartSpec("swiglu", dict(hidden_size=self.hidden_size,
                                            intermediate_size=self.intermediate_size), prefix=p + "mlp."),
                norms={"mixer": norm("input_layernorm"), "ffn": norm("post_attention_layernorm")},
            ))
        spec = ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            embedding=PartSpec("embedding", dict(vocab_size=self.vocab_size, hidden_size=self.hidden_size),
                               prefix="model.embed_tokens."),
            layers=tuple(layers),
            schedule=default_schedule(self.num_hidden_layers),
            final_norm=PartSpec("rmsnorm", dict(size=self.hidden_size, eps=self.rms_norm_eps),
                                prefix="model.norm."),
            head=PartSpec("lm_head", dict(vocab_size=self.vocab_size, hidden_size=self.hidden_size,
                                          tied_to="model.embed_tokens.weight" if self.tie_word_embeddings else None),
                          prefix="lm_head."),
            max_position=self.max_position_embeddings,
        )
        spec.validate()
        return spec


register_architecture(LlamaConfig.architecture, LlamaConfig, model_type=LlamaConfig.model_type)
