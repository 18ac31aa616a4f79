"""LlamaConfig: the typed configuration of a Llama 3 dense model.

Keys and defaults follow crates/ai-engine-runtime/src/config.rs:22-47,160-184
(hidden_size, intermediate_size, num_hidden_layers, num_attention_heads,
num_key_value_heads = heads, head_dim = hidden/heads, vocab_size,
max_position_embeddings = 8192, rope_theta = 10000, rms_norm_eps = 1e-6,
tie_word_embeddings = false).  Beyond the reference: `rope_scaling` of type
llama3 (the reference reads none), `rope_parameters` as a second home of
rope_theta / scaling (the reference's own fixture keeps theta only there,
crates/ai-engine-runtime/fixtures/toy-llama-3/config.json:36-39), and
`eos_token_id` as an int or a list (crates/ai-engine-rustyllm/src/provider.rs:297-303).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple

from .base import ConfigError, get_bool, get_float, get_int, read_json


@dataclass(frozen=True)
class RopeScaling:
    """llama3 frequency scaling: wavelengths above original/low_freq_factor are
    stretched by `factor`, those below original/high_freq_factor are kept, the
    band between is blended."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_dict(self) -> dict:
        return dict(rope_type=self.rope_type, factor=self.factor,
                    low_freq_factor=self.low_freq_factor,
                    high_freq_factor=self.high_freq_factor,
                    original_max_position_embeddings=self.original_max_position_embeddings)


def _parse_scaling(d) -> Optional[RopeScaling]:
    if d is None:
        return None
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: `rope_scaling` must be an object, got {d!r}")
    kind = d.get("rope_type", d.get("type", "default"))
    if kind in (None, "default"):
        return None
    if kind != "llama3":
        raise ConfigError(
            f"config.json: rope_scaling type `{kind}` is not supported (supported: default, llama3)")
    orig = get_int(d, "original_max_position_embeddings")
    sc = RopeScaling("llama3", get_float(d, "factor"), get_float(d, "low_freq_factor"),
                     get_float(d, "high_freq_factor"), orig)
    if sc.factor <= 0 or sc.high_freq_factor <= sc.low_freq_factor or sc.low_freq_factor <= 0:
        raise ConfigError(
            "config.json: rope_scaling needs factor > 0 and high_freq_factor > low_freq_factor > 0")
    return sc


@dataclass(frozen=True)
class LlamaConfig:
    architecture: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool
    rope_scaling: Optional[RopeScaling] = None
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)
    bos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None

    ARCHITECTURE = "LlamaForCausalLM"

    @classmethod
    def from_dict(cls, raw: dict) -> "LlamaConfig":
        archs = raw.get("architectures")
        if not isinstance(archs, list) or not archs or not all(isinstance(a, str) for a in archs):
            raise ConfigError("config.json: required key `architectures` must be a list of names")
        hidden = get_int(raw, "hidden_size")
        heads = get_int(raw, "num_attention_heads")
        kv_heads = get_int(raw, "num_key_value_heads", heads)
        if "head_dim" not in raw or raw["head_dim"] is None:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads "
                    f"{heads} and no head_dim is given")
        head_dim = get_int(raw, "head_dim", hidden // heads)
        inter = get_int(raw, "intermediate_size", 0, minimum=0)
        if inter == 0:
            raise ConfigError("config.json: required key `intermediate_size` is missing or 0")
        if heads % kv_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {heads} must be a multiple of "
                f"num_key_value_heads {kv_heads}")
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim {head_dim} must be even for rotary encoding")
        act = raw.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act `{act}` is not supported (supported: silu)")
        for k in ("attention_bias", "mlp_bias"):
            if get_bool(raw, k, False):
                raise ConfigError(f"config.json: `{k}` = true is not supported")
        rp = raw.get("rope_parameters")
        if rp is not None and not isinstance(rp, dict):
            raise ConfigError("config.json: `rope_parameters` must be an object")
        rp = rp or {}
        if raw.get("rope_theta") is not None:
            theta = get_float(raw, "rope_theta")
        else:
            theta = get_float(rp, "rope_theta", 10000.0)
        if theta <= 0:
            raise ConfigError(f"config.json: rope_theta must be positive, got {theta}")
        scaling = _parse_scaling(raw.get("rope_scaling"))
        if scaling is None and rp:
            scaling = _parse_scaling(rp)
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"config.json: `eos_token_id` must be an integer or a list, got {eos!r}")
        bos = raw.get("bos_token_id")
        eps = get_float(raw, "rms_norm_eps", 1e-6)
        if eps <= 0:
            raise ConfigError(f"config.json: rms_norm_eps must be positive, got {eps}")
        return cls(
            architecture=archs[0],
            hidden_size=hidden,
            intermediate_size=inter,
            num_hidden_layers=get_int(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=get_int(raw, "vocab_size"),
            max_position_embeddings=get_int(raw, "max_position_embeddings", 8192),
            rope_theta=theta,
            rms_norm_eps=eps,
            tie_word_embeddings=get_bool(raw, "tie_word_embeddings", False),
            rope_scaling=scaling,
            eos_token_ids=eos_ids,
            bos_token_id=bos if isinstance(bos, int) and not isinstance(bos, bool) else None,
            torch_dtype=raw.get("torch_dtype", raw.get("dtype")),
        )

    @classmethod
    def from_file(cls, path: str) -> "LlamaConfig":
        return cls.from_dict(read_json(path))

    def to_dict(self) -> dict:
        """The config.json that `from_dict` reads back to an equal object."""
        d = dict(
            architectures=[self.architecture], model_type="llama",
            hidden_size=self.hidden_size, intermediate_size=self.intermediate_size,
            num_hidden_layers=self.num_hidden_layers,
            num_attention_heads=self.num_attention_heads,
            num_key_value_heads=self.num_key_value_heads, head_dim=self.head_dim,
            vocab_size=self.vocab_size, max_position_embeddings=self.max_position_embeddings,
            rope_theta=self.rope_theta, rms_norm_eps=self.rms_norm_eps,
            tie_word_embeddings=self.tie_word_embeddings, hidden_act="silu",
            attention_bias=False, mlp_bias=False,
        )
        if self.rope_scaling is not None:
            d["rope_scaling"] = self.rope_scaling.to_dict()
        if self.eos_token_ids:
            d["eos_token_id"] = (self.eos_token_ids[0] if len(self.eos_token_ids) == 1
                                 else list(self.eos_token_ids))
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        if self.torch_dtype is not None:
            d["torch_dtype"] = self.torch_dtype
        return d
