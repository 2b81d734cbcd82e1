"""Model registry: `model_type` of a ModelConfig -> the class ModelRunner.load_model builds — the
role of the reference's ModelRegistry (python/sglang/srt/models/registry.py), without the import
scan: one line per model family of this package."""
from __future__ import annotations

import importlib
from typing import Dict, Tuple

_MODELS: Dict[str, Tuple[str, str]] = {
    "llama": ("llama", "LlamaForCausalLM"),
    "opt": ("opt", "OPTForCausalLM"),
    "deepseek_v2": ("deepseek_v2", "DeepseekV2ForCausalLM"),
    "rimidra": ("rimidra", "RimidraForCausalLM"),
    "nupovik": ("nupovik", "NupovikForCausalLM"),
    "matepel": ("matepel", "MatepelForCausalLM"),
    "sugelix": ("sugelix", "SugelixForCausalLM"),
}


def register_model(model_type: str, module: str, cls: str) -> None:
    _MODELS[model_type] = (module, cls)


def get_model_class(model_type: str):
    try:
        module, cls = _MODELS[model_type]
    except KeyError:
        raise ValueError(f"unknown model_type {model_type!r}; known: {sorted(_MODELS)}") from None
    return getattr(importlib.import_module(f"{__package__}.{module}"), cls)
