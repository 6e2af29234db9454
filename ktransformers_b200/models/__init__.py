"""Model registry: which class serves a checkpoint directory, chosen by its `config.json` (the role of `custom_models` in the
reference's local_chat.py:36-43, where `config.architectures[0]` picks the modeling class)."""
from __future__ import annotations

import json
import os

MODEL_REGISTRY = {
    # architecture name -> (module, class)
    "Lekapel": ("ktransformers_b200.models.modeling_lekapel", "LekapelForCausalLM"),
    "Mabidra": ("ktransformers_b200.models.modeling_mabidra", "MabidraForCausalLM"),
    "Zivulix": ("ktransformers_b200.models.modeling_zivulix", "ZivulixForCausalLM"),
    "Bilurax": ("ktransformers_b200.models.modeling_bilurax", "BiluraxForCausalLM"),
    "DeepseekV3ForCausalLM": ("ktransformers_b200.models.modeling_deepseek_v3", "DeepseekV3MoEOnlyForCausalLM"),
    "DeepseekV2ForCausalLM": ("ktransformers_b200.models.modeling_deepseek", "DeepseekV2MoE"),
}


def architecture_of(config: dict) -> str:
    if "architecture" in config:
        return config["architecture"]
    if config.get("architectures"):
        return config["architectures"][0]
    raise ValueError("config.json names no architecture")


def model_class(arch: str):
    import importlib
    if arch not in MODEL_REGISTRY:
        raise ValueError(f"no model class registered for architecture {arch!r} (known: {sorted(MODEL_REGISTRY)})")
    mod, cls = MODEL_REGISTRY[arch]
    return getattr(importlib.import_module(mod), cls)


def load_model(path: str, dtype="bfloat16", device: str = "cuda"):
    """Build the registered class for `path/config.json` and load `path`'s safetensors through the framework's loader.
    Only step-function models (those with a `config_class.from_dict` and `load(loader)`) are served this way."""
    import torch

    from ..util.custom_loader import ModelLoaderFactory
    with open(os.path.join(path, "config.json")) as f:
        raw = json.load(f)
    cls = model_class(architecture_of(raw))
    if not hasattr(cls, "config_class") or not hasattr(cls.config_class, "from_dict"):
        raise NotImplementedError(f"{cls.__name__} is an injection target, not a step-function model; use optimize_and_load_gguf")
    if isinstance(dtype, str):
        dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    model = cls(cls.config_class.from_dict(raw), dtype=dtype, device=device)
    model.load(ModelLoaderFactory.create_loader(path))
    return model.eval()
