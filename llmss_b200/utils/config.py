"""Model configuration loading.

Hugging Face checkpoints carry ``model_type`` in config.json and are read through ``transformers.AutoConfig``
(reference: `AutoConfig.from_pretrained`, generate.py:57-60).  Architectures that no library knows describe
themselves with an ``architecture`` key instead; their config.json is read as plain JSON into a
:class:`NativeConfig`, whose ``model_type`` (the lower-cased architecture name) selects the class in
``MODEL_REGISTRY`` the same way.
"""
from __future__ import annotations

import json
from pathlib import Path


class NativeConfig:
    """config.json of a native architecture: the parsed JSON (``raw``) plus the registry key."""

    def __init__(self, raw: dict):
        self.raw = raw
        self.model_type = str(raw["architecture"]).lower()

    def __repr__(self):
        return f"NativeConfig({self.model_type})"


def load_config(path):
    f = Path(path) / "config.json"
    if f.is_file():
        raw = json.loads(f.read_text())
        if "model_type" not in raw and "architecture" in raw:
            return NativeConfig(raw)
    from transformers import AutoConfig

    return AutoConfig.from_pretrained(path)
