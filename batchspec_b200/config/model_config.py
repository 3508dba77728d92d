"""Typed model configurations read from an architecture's own ``config.json`` keys.

The reference keeps its numbers in a by-name table of keyword dicts
(batchspec/models/configs/registry.py:7-131) feeding a ``ModelArgs`` dataclass
(batchspec/models/configs/model_config.py:9-66) and never reads ``config.json``.
Here ``config.json`` is the source of every size and constant; the by-name table
only holds ready-made ``config.json`` dicts for random-weight runs.

A configuration class is registered per architecture name (``architectures[0]``).
It must provide ``from_json_dict(d)``, ``to_json_dict()`` and the attribute
``architecture``; nothing else in the framework looks inside it except that
architecture's own model builder.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any, Callable, Dict, Optional, Tuple


class ConfigError(ValueError):
    """A config.json that this architecture cannot run: names the key and the value."""


_MISSING = object()


def _take(d: Dict[str, Any], key: str, kind, default=_MISSING):
    if key not in d or d[key] is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and float(v).is_integer():
                return int(v)
            raise ConfigError(f"config.json: '{key}' must be an integer, got {v!r}")
        return v
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {v!r}")
        return float(v)
    if kind is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: '{key}' must be true or false, got {v!r}")
        return v
    return v


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of config.json.  ``llama3``: the reference forwards
    factor / low_freq_factor / high_freq_factor / original_max_position_embeddings
    (batchspec/models/modules/rope.py:33-44).  ``linear``: every frequency divided
    by ``factor`` (rope.py:27-31, ``rope_scale``)."""
    rope_type: str
    factor: float
    low_freq_factor: Optional[float] = None
    high_freq_factor: Optional[float] = None
    original_max_position_embeddings: Optional[int] = None

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "RopeScaling":
        kind = d.get("rope_type", d.get("type"))
        read = {"rope_type", "type", "factor"} | ({"low_freq_factor", "high_freq_factor",
                                                   "original_max_position_embeddings"} if kind == "llama3" else set())
        unread = sorted(k for k, v in d.items() if k not in read and v is not None)
        if unread:
            raise ConfigError(f"config.json: rope_scaling of type {kind!r} has fields this engine does not apply: "
                              f"{', '.join(unread)}")
        if kind == "linear":
            return cls("linear", _take(d, "factor", float))
        if kind != "llama3":
            raise ConfigError(f"config.json: rope_scaling type {kind!r} is not supported "
                              f"(supported: 'llama3', 'linear', or null)")
        rs = cls("llama3", _take(d, "factor", float), _take(d, "low_freq_factor", float),
                 _take(d, "high_freq_factor", float),
                 _take(d, "original_max_position_embeddings", int))
        if rs.high_freq_factor == rs.low_freq_factor:
            raise ConfigError("config.json: rope_scaling high_freq_factor must differ from low_freq_factor")
        return rs

    def to_json_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"rope_type": self.rope_type, "factor": self.factor}
        if self.rope_type == "llama3":
            d.update(low_freq_factor=self.low_freq_factor, high_freq_factor=self.high_freq_factor,
                     original_max_position_embeddings=self.original_max_position_embeddings)
        return d


@dataclass(frozen=True)
class LlamaConfig:
    """The Llama-3 dense decoder as ``config.json`` describes it.

    Field -> reference name (model_config.py:14-37): hidden_size=dim,
    num_hidden_layers=n_layer, num_attention_heads=n_head,
    num_key_value_heads=n_local_heads, rms_norm_eps=norm_eps, rope_theta=rope_base,
    max_position_embeddings=block_size.
    """
    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    rope_scaling: Optional[RopeScaling] = None
    tie_word_embeddings: bool = False
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    torch_dtype: Optional[str] = None
    unread_keys: Tuple[str, ...] = ()      # keys of config.json that nothing here reads or knows to be harmless

    # keys whose only allowed value is the one that leaves the Llama-3 formulas as they are
    _NEUTRAL = {"sliding_window": (None, 0), "attention_dropout": (None, 0, 0.0), "partial_rotary_factor": (None, 1, 1.0),
                "attention_multiplier": (None,), "logits_scaling": (None, 1, 1.0), "residual_multiplier": (None, 1, 1.0),
                "embedding_multiplier": (None, 1, 1.0), "final_logit_softcapping": (None,),
                "attn_logit_softcapping": (None,), "use_qk_norm": (None, False), "qk_norm": (None, False),
                "num_local_experts": (None, 0), "num_experts": (None, 0), "layer_types": (None,),
                "no_rope_layers": (None,), "pretraining_tp": (None, 1)}
    _READ = {"architectures", "vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
             "num_key_value_heads", "head_dim", "intermediate_size", "rms_norm_eps", "rope_theta", "rope_scaling",
             "max_position_embeddings", "tie_word_embeddings", "bos_token_id", "eos_token_id", "torch_dtype", "dtype",
             "attention_bias", "mlp_bias", "hidden_act", "model_type"}
    _HARMLESS = {"transformers_version", "use_cache", "pad_token_id", "initializer_range", "_name_or_path",
                 "unread_keys"}

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "LlamaConfig":
        arch = (d.get("architectures") or [None])[0]
        if arch is None:
            raise ConfigError("config.json: 'architectures' is missing or empty")
        if d.get("model_type", "llama") != "llama":
            raise ConfigError(f"config.json: model_type {d['model_type']!r} is not 'llama'")
        changed = sorted(k for k, ok in cls._NEUTRAL.items() if k in d and d[k] not in ok)
        if changed:
            raise ConfigError("config.json: " + ", ".join(f"{k}={d[k]!r}" for k in changed)
                              + " would change the model's arithmetic and this engine does not apply it")
        unread = tuple(sorted(k for k in d if k not in cls._READ and k not in cls._NEUTRAL and k not in cls._HARMLESS))
        n_head = _take(d, "num_attention_heads", int)
        hidden = _take(d, "hidden_size", int)
        if _take(d, "attention_bias", bool, False) or _take(d, "mlp_bias", bool, False):
            raise ConfigError("config.json: attention_bias / mlp_bias = true is not supported by this architecture")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported (only 'silu')")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos]))
        rs = d.get("rope_scaling")
        cfg = cls(
            architecture=arch,
            vocab_size=_take(d, "vocab_size", int),
            hidden_size=hidden,
            num_hidden_layers=_take(d, "num_hidden_layers", int),
            num_attention_heads=n_head,
            num_key_value_heads=_take(d, "num_key_value_heads", int, n_head),
            head_dim=_take(d, "head_dim", int, hidden // n_head),
            intermediate_size=_take(d, "intermediate_size", int),
            rms_norm_eps=_take(d, "rms_norm_eps", float),
            rope_theta=_take(d, "rope_theta", float),
            max_position_embeddings=_take(d, "max_position_embeddings", int),
            rope_scaling=RopeScaling.from_json_dict(rs) if rs else None,
            tie_word_embeddings=_take(d, "tie_word_embeddings", bool, False),
            bos_token_id=d.get("bos_token_id"),
            eos_token_ids=eos_ids,
            torch_dtype=d.get("torch_dtype", d.get("dtype")),
            unread_keys=unread,
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for f in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "intermediate_size", "max_position_embeddings"):
            if getattr(self, f) <= 0:
                raise ConfigError(f"config.json: '{f}' must be positive, got {getattr(self, f)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"config.json: num_attention_heads ({self.num_attention_heads}) must be a "
                              f"multiple of num_key_value_heads ({self.num_key_value_heads})")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim ({self.head_dim}) must be even for rotary pairs")
        if not self.rms_norm_eps > 0:
            raise ConfigError("config.json: rms_norm_eps must be > 0")

    def to_json_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {
            "architectures": [self.architecture], "model_type": "llama", "hidden_act": "silu",
            "attention_bias": False, "mlp_bias": False,
        }
        for f in fields(self):
            if f.name in ("architecture", "rope_scaling", "eos_token_ids", "unread_keys"):
                continue
            d[f.name] = getattr(self, f.name)
        d["rope_scaling"] = self.rope_scaling.to_json_dict() if self.rope_scaling else None
        d["eos_token_id"] = (list(self.eos_token_ids) if len(self.eos_token_ids) != 1
                             else self.eos_token_ids[0]) if self.eos_token_ids else None
        return d


# --------------------------------------------------------------------------- registry

_CONFIG_CLASSES: Dict[str, type] = {}


def register_config_class(architecture: str, cls: type) -> None:
    """Make ``architectures[0] == architecture`` parse with ``cls.from_json_dict``."""
    _CONFIG_CLASSES[architecture] = cls


def known_architectures():
    return sorted(_CONFIG_CLASSES)


def config_from_json_dict(d: Dict[str, Any]):
    arch = (d.get("architectures") or [None])[0]
    if arch not in _CONFIG_CLASSES:
        raise ConfigError(f"config.json: architecture {arch!r} is not registered "
                          f"(known: {', '.join(known_architectures()) or 'none'})")
    return _CONFIG_CLASSES[arch].from_json_dict(d)


def load_config(model_dir) -> Any:
    path = Path(model_dir) / "config.json"
    if not path.is_file():
        raise FileNotFoundError(f"no config.json in {model_dir}")
    return config_from_json_dict(json.loads(path.read_text()))


def save_config(cfg, model_dir) -> None:
    Path(model_dir).mkdir(parents=True, exist_ok=True)
    (Path(model_dir) / "config.json").write_text(json.dumps(cfg.to_json_dict(), indent=2) + "\n")


register_config_class("LlamaForCausalLM", LlamaConfig)
