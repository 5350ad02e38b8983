"""Qwen2Config: the Qwen2.5 dense decoder's config.json, typed.

Keys and defaults follow the reference's reading of the same hyper-parameters from
GGUF metadata (model_config.cpp:35-54): kv heads default to the head count (:43), the
head size to hidden/heads (:50), the norm's eps is required (:46), the rotary base
defaults to 10000 (:47).  Its checks (model_config.cpp:56-63) are kept, except the
restriction to a head size of 128.
"""
from dataclasses import dataclass

from .base import ConfigError, Key, positive, read_keys

ARCHITECTURE = "Qwen2ForCausalLM"

_KEYS = (
    Key("vocab_size", int, check=positive, rule="must be positive"),
    Key("hidden_size", int, check=positive, rule="must be positive"),
    Key("intermediate_size", int, check=positive, rule="must be positive"),
    Key("num_hidden_layers", int, check=positive, rule="must be positive"),
    Key("num_attention_heads", int, check=positive, rule="must be positive"),
    Key("num_key_value_heads", int, default=lambda v: v["num_attention_heads"], check=positive,
        rule="must be positive"),
    Key("head_dim", int, default=lambda v: v["hidden_size"] // v["num_attention_heads"], check=positive,
        rule="must be positive"),
    Key("max_position_embeddings", int, check=positive, rule="must be positive"),
    Key("rms_norm_eps", float, check=positive, rule="must be positive"),
    Key("rope_theta", float, default=10000.0, check=lambda v: v > 1.0, rule="must be greater than 1"),
    Key("tie_word_embeddings", bool, default=False),
    Key("use_sliding_window", bool, default=False),
    Key("sliding_window", int, default=None, check=positive, rule="must be positive"),
    Key("max_window_layers", int, default=0, check=lambda v: v >= 0, rule="must not be negative"),
    Key("torch_dtype", str, default="bfloat16"),
    Key("hidden_act", str, default="silu", check=lambda v: v == "silu", rule="this architecture has silu only"),
)


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    max_position_embeddings: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    use_sliding_window: bool
    sliding_window: object          # int or None
    max_window_layers: int
    torch_dtype: str
    hidden_act: str
    architecture: str = ARCHITECTURE

    @classmethod
    def from_dict(cls, d: dict) -> "Qwen2Config":
        v = read_keys(d, _KEYS)
        if v["num_attention_heads"] % v["num_key_value_heads"] != 0:
            raise ConfigError("config.json: 'num_attention_heads' (%d) must be a multiple of "
                              "'num_key_value_heads' (%d)" % (v["num_attention_heads"], v["num_key_value_heads"]))
        if v["head_dim"] % 2 != 0:
            raise ConfigError("config.json: 'head_dim' (%d) must be even: the rotary encoding pairs its halves"
                              % v["head_dim"])
        if v["use_sliding_window"] and v["sliding_window"] is None:
            raise ConfigError("config.json: 'use_sliding_window' is true but 'sliding_window' is missing")
        archs = d.get("architectures")
        if isinstance(archs, list) and archs and isinstance(archs[0], str):
            v["architecture"] = archs[0]          # another registered name may reuse these keys
        return cls(**v)

    def to_dict(self) -> dict:
        d = {k.name: getattr(self, k.name) for k in _KEYS}
        d["architectures"] = [self.architecture]
        d["model_type"] = "qwen2"
        return d

    def window_of(self, layer: int):
        """Keys that a query of `layer` may see (itself included), or None for all.

        The reference has no window.  A layer is windowed iff use_sliding_window and
        layer >= max_window_layers; a query at position p then sees max(0, p-W+1) .. p.
        """
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None
