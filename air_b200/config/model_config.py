"""Typed configuration of the Qwen2 dense decoder, read from config.json's own keys.

The checks follow AIR's architecture contract (src/model/qwen2_contract.cpp:33-67) and its
generic model validation (src/model/model.cpp:89-118): a geometry that is missing or
inconsistent is a *data error*; a feature that the engine does not compute is
*unsupported*.  No size has a default in code, except where AIR's own reader has one
(kv heads default to heads, src/formats/gguf/gguf_format.cpp:120).
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import Any, Mapping, Optional


class ConfigError(ValueError):
    """A configuration that cannot be used.  ``kind`` is "data_error" or "unsupported",
    AIR's two classes of refusal (include/air/status.hpp:8-17)."""

    def __init__(self, kind: str, message: str):
        super().__init__(f"{kind}: {message}")
        self.kind = kind
        self.message = message


def _require(d: Mapping[str, Any], key: str, typ):
    if key not in d or d[key] is None:
        raise ConfigError("data_error", f"config.json lacks '{key}'")
    v = d[key]
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError("data_error", f"config.json '{key}' must be an integer, got {v!r}")
    elif typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError("data_error", f"config.json '{key}' must be a number, got {v!r}")
        v = float(v)
    return v


@dataclass(frozen=True)
class Qwen2Config:
    """Hyper-parameters of Qwen2ForCausalLM (AIR: ModelConfig, include/air/model.hpp:17-33)."""
    architecture: str
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    tie_word_embeddings: bool = False
    attention_bias: bool = True
    hidden_act: str = "silu"
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @property
    def head_dim(self) -> int:
        # AIR fixes the head size as hidden/heads (src/model/qwen2_contract.cpp:47).
        return self.hidden_size // self.num_attention_heads

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen2Config":
        archs = d.get("architectures") or []
        arch = archs[0] if archs else None
        if arch is None:
            raise ConfigError("data_error", "config.json lacks 'architectures'")
        if d.get("model_type", "qwen2") != "qwen2":
            raise ConfigError("unsupported", f"model_type {d.get('model_type')!r} is not qwen2")
        heads = _require(d, "num_attention_heads", int)
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        known = {f for f in cls.__dataclass_fields__}
        cfg = cls(
            architecture=arch,
            num_hidden_layers=_require(d, "num_hidden_layers", int),
            hidden_size=_require(d, "hidden_size", int),
            num_attention_heads=heads,
            num_key_value_heads=d["num_key_value_heads"] if d.get("num_key_value_heads") is not None else heads,
            intermediate_size=_require(d, "intermediate_size", int),
            vocab_size=_require(d, "vocab_size", int),
            max_position_embeddings=_require(d, "max_position_embeddings", int),
            rope_theta=_require(d, "rope_theta", float),
            rms_norm_eps=_require(d, "rms_norm_eps", float),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            attention_bias=bool(d.get("attention_bias", True)),
            hidden_act=d.get("hidden_act", "silu"),
            use_sliding_window=bool(d.get("use_sliding_window", False)),
            sliding_window=d.get("sliding_window"),
            max_window_layers=d.get("max_window_layers"),
            eos_token_id=eos,
            bos_token_id=d.get("bos_token_id"),
            torch_dtype=d.get("torch_dtype", d.get("dtype")),
            extra={k: v for k, v in d.items() if k not in known and k not in ("architectures", "model_type")},
        )
        cfg.validate(raw=d)
        return cfg

    def to_dict(self) -> dict:
        d = asdict(self)
        d.pop("extra")
        arch = d.pop("architecture")
        d = {k: v for k, v in d.items() if v is not None}
        return {"architectures": [arch], "model_type": "qwen2", **d}

    # ------------------------------------------------------------------ checking
    def validate(self, raw: Optional[Mapping[str, Any]] = None) -> None:
        for name in ("num_hidden_layers", "hidden_size", "num_attention_heads", "num_key_value_heads",
                     "max_position_embeddings", "vocab_size"):
            if getattr(self, name) <= 0:
                raise ConfigError("data_error", f"Qwen2 model geometry is incomplete: {name} = {getattr(self, name)}")
        if self.hidden_size % self.num_attention_heads != 0:
            raise ConfigError("data_error", "Qwen2 hidden size is not divisible by attention head count")
        if self.num_key_value_heads > self.num_attention_heads or \
                self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError("data_error", "Qwen2 attention head count must be divisible by KV head count")
        if self.intermediate_size <= 0:
            raise ConfigError("data_error", "Qwen2 feed-forward size is missing")
        if not (self.rms_norm_eps > 0.0):
            raise ConfigError("data_error", "Qwen2 RMS norm epsilon is missing or invalid")
        if not (self.rope_theta > 0.0):
            raise ConfigError("data_error", "Qwen2 RoPE base is missing or invalid")
        if self.head_dim % 2 != 0:
            raise ConfigError("unsupported", "Qwen2 execution requires full, even head-dimension RoPE")
        if self.hidden_act != "silu":
            raise ConfigError("unsupported", f"hidden_act {self.hidden_act!r}: only silu is implemented")
        if raw is not None:
            scaling = raw.get("rope_scaling")
            if scaling not in (None, {}):
                kind = scaling.get("rope_type", scaling.get("type")) if isinstance(scaling, dict) else scaling
                if kind not in (None, "none", "default"):
                    raise ConfigError("unsupported", f"Qwen2 execution does not implement RoPE scaling type: {kind}")
                if isinstance(scaling, dict) and abs(float(scaling.get("factor", 1.0)) - 1.0) > 1e-12:
                    raise ConfigError("unsupported", "Qwen2 execution does not implement scaled RoPE")
            if raw.get("head_dim") is not None and raw["head_dim"] != self.head_dim:
                raise ConfigError("unsupported", "head_dim must equal hidden_size / num_attention_heads")
            if raw.get("partial_rotary_factor") not in (None, 1, 1.0):
                raise ConfigError("unsupported", "Qwen2 execution requires full, even head-dimension RoPE")
        if self.use_sliding_window:
            if self.sliding_window is None or self.sliding_window <= 0:
                raise ConfigError("data_error", "use_sliding_window is set but sliding_window is missing")
        for name in ("eos_token_id", "bos_token_id"):
            v = getattr(self, name)
            if v is not None and not (0 <= v < self.vocab_size):
                raise ConfigError("data_error", f"{name} is outside the vocabulary")

    def layer_window(self, layer: int) -> Optional[int]:
        """The window of a layer, or None when it sees all keys.  AIR rejects every window
        (src/model/qwen2_contract.cpp:62-64); this engine follows config.json's three keys:
        with use_sliding_window, layers from max_window_layers on see sliding_window keys."""
        if not self.use_sliding_window:
            return None
        first = self.max_window_layers if self.max_window_layers is not None else self.num_hidden_layers
        return int(self.sliding_window) if layer >= first else None
