"""Model dispatch (``/root/reference/src/tiny_llm/models.py:8-18``)."""

from __future__ import annotations

from .qwen3_week2 import Qwen3ModelWeek2
from .qwen3_week3 import Qwen3ModelWeek3

# /root/reference/model_names.py:1-8
MODEL_SHORTCUTS = {
    "qwen3-0.6b": "Qwen/Qwen3-0.6B-MLX-4bit",
    "qwen3-1.7b": "Qwen/Qwen3-1.7B-MLX-4bit",
    "qwen3-4b": "Qwen/Qwen3-4B-MLX-4bit",
}


# Designs that describe themselves in config.json (key "architecture"): name -> class with
# ``from_checkpoint(config, tensors, dtype=, device=, **kwargs)``.  Imported on demand: a process that runs one design
# loads (and, for the native libraries, builds) only what that design uses.
ARCHITECTURES = {
    "Voluzen": ("tiny_llm_b200.voluzen", "VoluzenModel"),
    "Bapovik": ("tiny_llm_b200.bapovik", "BapovikModel"),
    "Senurax": ("tiny_llm_b200.senurax", "SenuraxModel"),
    "Norusun": ("tiny_llm_b200.norusun", "NorusunModel"),
}


def model_class(architecture: str):
    import importlib

    if architecture not in ARCHITECTURES:
        raise ValueError(f"architecture {architecture!r} is not supported (known: {sorted(ARCHITECTURES)})")
    module, name = ARCHITECTURES[architecture]
    return getattr(importlib.import_module(module), name)


def load_model(path, device="cuda", dtype=None, **kwargs):
    """Model object for a checkpoint DIRECTORY, chosen by its config.json: a self-describing design
    (``architecture``) is built by its class from the plain tensors; an MLX 4-bit Qwen3 checkpoint goes through
    ``load_checkpoint`` + ``dispatch_model`` (week 3)."""
    import json
    from pathlib import Path

    import torch

    config = json.loads((Path(path) / "config.json").read_text())
    if "architecture" in config:
        from .checkpoint import read_tensors

        cls = model_class(config["architecture"])
        return cls.from_checkpoint(config, read_tensors(path), device=device, dtype=dtype or torch.bfloat16, **kwargs)
    from .checkpoint import load_checkpoint

    return dispatch_model("Qwen/Qwen3-" + str(path), load_checkpoint(path, device=device), week=3, **kwargs)


def shortcut_name_to_full_name(name: str) -> str:
    return MODEL_SHORTCUTS.get(name.lower(), name)


def dispatch_model(model_name: str, mlx_model, week: int, **kwargs):
    """Week 2 -> dense-cache model, week 3 -> paged model.  Week 1 (uncached,
    readable-only) is not part of the B200 hot path; its CPU restatement lives
    in ``oracle/model.py``."""
    full = shortcut_name_to_full_name(model_name)
    if full.startswith("Qwen/Qwen3"):
        if week == 2:
            return Qwen3ModelWeek2(mlx_model, **kwargs)
        if week == 3:
            return Qwen3ModelWeek3(mlx_model, **kwargs)
    raise ValueError(f"{full} for week {week} not supported")
