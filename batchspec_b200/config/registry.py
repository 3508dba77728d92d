"""By-name table of ready-made configurations, for runs with random weights.

Keeps the reference's lookup rule (batchspec/models/configs/registry.py:144-179):
an exact key wins; otherwise every key that is a case-insensitive substring of the
asked name is a candidate, the longest wins, a tie is an error, none is an error.
The entries are ``config.json`` files under ``presets/`` beside this module, so the
table holds data, not code.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Dict

from .model_config import config_from_json_dict

_PRESET_DIR = Path(__file__).parent / "presets"
MODEL_CONFIGS: Dict[str, Dict[str, Any]] = {
    p.stem: json.loads(p.read_text()) for p in sorted(_PRESET_DIR.glob("*.json"))
}


def register_config(name: str, config_json: Dict[str, Any]) -> None:
    """Add or replace a named ``config.json`` dict (registry.py:134-141)."""
    MODEL_CONFIGS[name] = dict(config_json)


def get_config(name: str):
    if name in MODEL_CONFIGS:
        return config_from_json_dict(MODEL_CONFIGS[name])
    low = name.lower()
    hits = [k for k in MODEL_CONFIGS if k.lower() in low]
    if not hits:
        raise ValueError(f"No configuration found for '{name}'. Known: {', '.join(sorted(MODEL_CONFIGS))}")
    hits.sort(key=len, reverse=True)
    if len(hits) > 1 and len(hits[0]) == len(hits[1]):
        raise ValueError(f"Ambiguous configuration name '{name}': matches {hits[0]!r} and {hits[1]!r}")
    return config_from_json_dict(MODEL_CONFIGS[hits[0]])
