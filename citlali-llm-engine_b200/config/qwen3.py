"""Typed configuration of the Qwen3 dense decoder, read from its own config.json keys.

The reference reads the same quantities from GGUF metadata
(include/citlali/model/qwen_config.h:10-25, src/model/qwen_config.cpp:32-124);
the fallbacks kept here are the reference's: ``num_key_value_heads`` defaults to the
number of query heads (qwen_config.cpp:56,95) and ``head_dim`` to hidden/heads
(qwen_config.cpp:112-115).  Options the reference's forward pass does not have
(attention bias, another activation, rope scaling, a sliding window) are refused by
name rather than ignored.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, asdict
from typing import Any, Dict, Optional, Tuple

from ..errors import CitlaliError, require
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleStep

ARCHITECTURE = "Qwen3ForCausalLM"


def _positive_int(d, key):
    require(key in d, f"config.json: required key '{key}' is missing")
    v = d[key]
    require(isinstance(v, int) and not isinstance(v, bool) and v > 0,
            f"config.json: '{key}' must be a positive integer, got {v!r}")
    return v


def _positive_float(d, key):
    require(key in d, f"config.json: required key '{key}' is missing")
    v = d[key]
    require(isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0,
            f"config.json: '{key}' must be a positive number, got {v!r}")
    return float(v)


def _rope_theta(d) -> float:
    """``rope_theta``, or the same number inside a ``rope_parameters`` object (how newer writers of
    config.json store it); a ``rope_type`` other than the plain one there is a scaling, which is refused."""
    params = d.get("rope_parameters")
    if params is not None:
        require(isinstance(params, dict), "config.json: 'rope_parameters' must be an object")
        kind = params.get("rope_type", params.get("type", "default"))
        require(kind in (None, "default"),
                f"config.json: rope_parameters.rope_type '{kind}' is not supported (plain rotary positions only)")
        if "rope_theta" not in d:
            require("rope_theta" in params, "config.json: required key 'rope_theta' is missing (also from 'rope_parameters')")
            return _positive_float(params, "rope_theta")
    return _positive_float(d, "rope_theta")


@dataclass(frozen=True)
class QwenConfig:
    architecture: str
    vocab_size: int
    max_position_embeddings: int
    hidden_size: int
    num_hidden_layers: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: Optional[bool]
    eos_token_ids: Tuple[int, ...] = ()

    # ---- reading -------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "QwenConfig":
        archs = d.get("architectures")
        require(isinstance(archs, list) and len(archs) >= 1 and isinstance(archs[0], str),
                "config.json: 'architectures' must be a non-empty list of names")
        hidden = _positive_int(d, "hidden_size")
        heads = _positive_int(d, "num_attention_heads")
        kv_heads = d.get("num_key_value_heads")
        if kv_heads is None:
            kv_heads = heads
        else:
            kv_heads = _positive_int(d, "num_key_value_heads")
        if d.get("head_dim") is None:
            require(hidden % heads == 0,
                    f"config.json: no 'head_dim' and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads}")
            head_dim = hidden // heads
        else:
            head_dim = _positive_int(d, "head_dim")
        require(heads % kv_heads == 0,
                f"config.json: num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}")
        require(head_dim % 2 == 0, f"config.json: head_dim {head_dim} must be even for rotary pairs")
        require(not d.get("attention_bias", False),
                "config.json: attention_bias=true is not supported (the Qwen3 dense path has no biases)")
        act = d.get("hidden_act", "silu")
        require(act == "silu", f"config.json: hidden_act '{act}' is not supported (SiLU gate only)")
        require(d.get("rope_scaling") is None,
                "config.json: rope_scaling is not supported (plain rotary positions only)")
        require(not d.get("use_sliding_window", False),
                "config.json: use_sliding_window=true is not supported (full causal attention only)")
        tie = d.get("tie_word_embeddings")
        require(tie is None or isinstance(tie, bool), "config.json: 'tie_word_embeddings' must be true or false")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        else:
            require(isinstance(eos, list) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos),
                    "config.json: 'eos_token_id' must be an integer or a list of integers")
            eos_ids = tuple(eos)
        vocab = _positive_int(d, "vocab_size")
        for e in eos_ids:
            require(0 <= e < vocab, f"config.json: eos_token_id {e} lies outside the vocabulary of {vocab}")
        return cls(
            architecture=archs[0],
            vocab_size=vocab,
            max_position_embeddings=_positive_int(d, "max_position_embeddings"),
            hidden_size=hidden,
            num_hidden_layers=_positive_int(d, "num_hidden_layers"),
            intermediate_size=_positive_int(d, "intermediate_size"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=_positive_float(d, "rms_norm_eps"),
            rope_theta=_rope_theta(d),
            tie_word_embeddings=tie,
            eos_token_ids=eos_ids,
        )

    @classmethod
    def from_model_dir(cls, model_dir: str) -> "QwenConfig":
        return cls.from_dict(read_config_json(model_dir))

    def to_dict(self) -> Dict[str, Any]:
        """The config.json this configuration is read back from."""
        d = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "max_position_embeddings": self.max_position_embeddings,
            "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_hidden_layers,
            "intermediate_size": self.intermediate_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "hidden_act": "silu",
            "attention_bias": False,
        }
        if self.tie_word_embeddings is not None:
            d["tie_word_embeddings"] = self.tie_word_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        return d

    def describe(self) -> Dict[str, Any]:
        return asdict(self)

    # ---- the architecture as data --------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        """Qwen3 dense: every layer is a pre-norm block of causal grouped-query attention
        (per-head q/k RMSNorm, half-split rotary positions) and a SiLU-gated feed-forward;
        layers run once each, in order (src/model/qwen_model.cpp:306-374)."""
        layers = []
        for i in range(self.num_hidden_layers):
            base = f"model.layers.{i}"
            norm = {"size": self.hidden_size, "eps": self.rms_norm_eps}
            layers.append(LayerSpec(block="pre_norm_residual", parts={
                "mixer_norm": PartSpec("rms_norm", dict(norm), f"{base}.input_layernorm"),
                "mixer": PartSpec("gqa_attention", {
                    "hidden_size": self.hidden_size,
                    "num_heads": self.num_attention_heads,
                    "num_kv_heads": self.num_key_value_heads,
                    "head_dim": self.head_dim,
                    "qk_norm_eps": self.rms_norm_eps,
                    "position": {"kind": "rotary_half_split", "theta": self.rope_theta,
                                 "rotary_dim": self.head_dim},
                    "window": None,
                }, f"{base}.self_attn"),
                "feed_forward_norm": PartSpec("rms_norm", dict(norm), f"{base}.post_attention_layernorm"),
                "feed_forward": PartSpec("gated_silu", {
                    "hidden_size": self.hidden_size,
                    "intermediate_size": self.intermediate_size,
                }, f"{base}.mlp"),
            }))
        spec = ModelSpec(
            architecture=self.architecture,
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            max_positions=self.max_position_embeddings,
            embedding_name="model.embed_tokens.weight",
            layers=tuple(layers),
            schedule=tuple(ScheduleStep(i) for i in range(self.num_hidden_layers)),
            final_norm=PartSpec("rms_norm", {"size": self.hidden_size, "eps": self.rms_norm_eps}, "model.norm"),
            head_name="lm_head.weight",
            tie_head_to_embedding=self.tie_word_embeddings,
            stop_token_ids=self.eos_token_ids,
        )
        spec.validate()
        return spec


def read_config_json(model_dir: str) -> Dict[str, Any]:
    path = os.path.join(model_dir, "config.json")
    require(os.path.isfile(path), f"no config.json in model folder '{model_dir}'")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except json.JSONDecodeError as e:
        raise CitlaliError(f"{path}: not valid JSON ({e})") from None
    require(isinstance(d, dict), f"{path}: the top level must be an object")
    return d
