"""Typed configuration of the LFM2 architecture, read from its own config.json keys.

The reference reads the same quantities from file metadata: embedding length, block count,
head counts, per-layer KV heads with 0 meaning a short-convolution layer, key length, rope base,
norm epsilon, short-conv window, optional sliding window (src/model.zig:395-490, 492-529).
No size is a constant in code: everything the model builder needs comes from here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError, ModelConfig, as_float, as_int, need

LAYER_CONV = "conv"
LAYER_FULL = "full_attention"
LAYER_WINDOW = "sliding_attention"
_LAYER_KINDS = (LAYER_CONV, LAYER_FULL, LAYER_WINDOW)


@dataclass
class Lfm2Config(ModelConfig):
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    layer_types: tuple[str, ...] = ()
    # short convolution
    conv_L_cache: int = 3
    conv_bias: bool = False
    # feed-forward width and its adjustment rule
    block_ff_dim: int = 0
    block_auto_adjust_ff_dim: bool = False
    block_ffn_dim_multiplier: float | None = None
    block_multiple_of: int = 256
    # numerics
    norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    sliding_window: int = 0
    tie_word_embeddings: bool = True

    # ------------------------------------------------------------------ derived sizes
    @property
    def ffn_dim(self) -> int:
        """Effective SwiGLU width: 2/3, then the multiplier, then rounded up to a multiple.

        The reference's file already carries the effective width (src/model.zig:423-440); a
        config.json carries `block_ff_dim` and this rule.  12288 -> 8192 (multiple of 256),
        288 -> 192 (multiple of 64); unchanged when auto-adjust is off.
        """
        f = self.block_ff_dim
        if self.block_auto_adjust_ff_dim:
            f = int(2 * f / 3)
            if self.block_ffn_dim_multiplier is not None:
                f = int(self.block_ffn_dim_multiplier * f)
            m = self.block_multiple_of
            f = m * ((f + m - 1) // m)
        return f

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_key_value_heads * self.head_dim

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_json_dict(cls, d: dict[str, Any]) -> "Lfm2Config":
        arch = (d.get("architectures") or ["Lfm2ForCausalLM"])[0]
        vocab = as_int(d, "vocab_size", need(d, "vocab_size"), 1)
        hidden = as_int(d, "hidden_size", need(d, "hidden_size"), 1)
        n_layers = as_int(d, "num_hidden_layers", need(d, "num_hidden_layers"), 1)
        heads = as_int(d, "num_attention_heads", need(d, "num_attention_heads"), 1)
        kv_heads = as_int(d, "num_key_value_heads", need(d, "num_key_value_heads"), 1)
        max_pos = as_int(d, "max_position_embeddings", need(d, "max_position_embeddings"), 1)
        ff = as_int(d, "block_ff_dim", need(d, "block_ff_dim", "intermediate_size"), 1)

        if d.get("head_dim") is not None:
            head_dim = as_int(d, "head_dim", d["head_dim"], 1)
        else:
            if hidden % heads:
                raise ConfigError(
                    f"config.json: hidden_size {hidden} is not a multiple of num_attention_heads {heads} "
                    "and no 'head_dim' is given")
            head_dim = hidden // heads                                # src/model.zig:441

        if d.get("layer_types") is not None:
            kinds = tuple(d["layer_types"])
        elif d.get("full_attn_idxs") is not None:
            idx = set(int(i) for i in d["full_attn_idxs"])
            bad = [i for i in idx if not 0 <= i < n_layers]
            if bad:
                raise ConfigError(f"config.json: full_attn_idxs {sorted(bad)} outside [0, {n_layers})")
            kinds = tuple(LAYER_FULL if i in idx else LAYER_CONV for i in range(n_layers))
        else:
            raise ConfigError("config.json: required key 'layer_types' is missing (or 'full_attn_idxs')")

        rope = d.get("rope_theta")
        if rope is None and isinstance(d.get("rope_parameters"), dict):
            rope = d["rope_parameters"].get("rope_theta")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        mult = d.get("block_ffn_dim_multiplier")
        tie = d.get("tie_word_embeddings", d.get("tie_embedding", True))

        cfg = cls(
            architecture=arch,
            vocab_size=vocab,
            hidden_size=hidden,
            max_position_embeddings=max_pos,
            eos_token_ids=eos_ids,
            bos_token_id=d.get("bos_token_id"),
            pad_token_id=d.get("pad_token_id"),
            raw=dict(d),
            num_hidden_layers=n_layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            layer_types=kinds,
            conv_L_cache=as_int(d, "conv_L_cache", d.get("conv_L_cache", 3)),
            conv_bias=bool(d.get("conv_bias", False)),
            block_ff_dim=ff,
            block_auto_adjust_ff_dim=bool(d.get("block_auto_adjust_ff_dim", False)),
            block_ffn_dim_multiplier=None if mult is None else as_float("block_ffn_dim_multiplier", mult),
            block_multiple_of=as_int(d, "block_multiple_of", d.get("block_multiple_of", 256), 1),
            norm_eps=as_float("norm_eps", d.get("norm_eps", 1e-5)),                 # src/model.zig:445
            rope_theta=as_float("rope_theta", 10000.0 if rope is None else rope),   # src/model.zig:446
            sliding_window=as_int(d, "sliding_window", d.get("sliding_window") or 0, 0),
            tie_word_embeddings=bool(tie),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        """The reference's checks (src/model.zig:484-489, 610, 1469) and those of the list of kinds."""
        if len(self.layer_types) != self.num_hidden_layers:
            raise ConfigError(
                f"config.json: layer_types has {len(self.layer_types)} entries for "
                f"num_hidden_layers {self.num_hidden_layers}")
        for i, k in enumerate(self.layer_types):
            if k not in _LAYER_KINDS:
                raise ConfigError(f"config.json: layer_types[{i}] = {k!r}; known kinds are {list(_LAYER_KINDS)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary pairs")
        if LAYER_CONV in self.layer_types and self.conv_L_cache < 2:
            raise ConfigError(f"config.json: conv_L_cache {self.conv_L_cache} must be >= 2 when a conv layer exists")
        if self.conv_L_cache > 64:
            raise ConfigError(f"config.json: conv_L_cache {self.conv_L_cache} exceeds the supported 64 taps")
        if LAYER_WINDOW in self.layer_types and self.sliding_window <= 0:
            raise ConfigError("config.json: a 'sliding_attention' layer needs 'sliding_window' > 0")
        if self.norm_eps <= 0:
            raise ConfigError(f"config.json: norm_eps must be positive, found {self.norm_eps}")
        if self.rope_theta <= 0:
            raise ConfigError(f"config.json: rope_theta must be positive, found {self.rope_theta}")
        if self.ffn_dim < 1:
            raise ConfigError(f"config.json: effective feed-forward width is {self.ffn_dim}")

    def to_json_dict(self) -> dict[str, Any]:
        eos: Any = list(self.eos_token_ids)
        if len(eos) == 1:
            eos = eos[0]
        elif not eos:
            eos = None
        d = {
            "architectures": [self.architecture],
            "model_type": "lfm2",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "max_position_embeddings": self.max_position_embeddings,
            "layer_types": list(self.layer_types),
            "conv_L_cache": self.conv_L_cache,
            "conv_bias": self.conv_bias,
            "block_ff_dim": self.block_ff_dim,
            "block_auto_adjust_ff_dim": self.block_auto_adjust_ff_dim,
            "block_ffn_dim_multiplier": self.block_ffn_dim_multiplier,
            "block_multiple_of": self.block_multiple_of,
            "norm_eps": self.norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "eos_token_id": eos,
            "bos_token_id": self.bos_token_id,
            "pad_token_id": self.pad_token_id,
        }
        if self.sliding_window:
            d["sliding_window"] = self.sliding_window
        return d
