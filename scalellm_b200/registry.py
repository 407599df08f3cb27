"""Model registry: config.json -> model class (the counterpart of the reference's REGISTER_CAUSAL_MODEL
table, src/models/model_registry.h, keyed by the checkpoint's architecture name).

A registered class provides
    from_config(config: dict, dtype, device, max_seqs: int) -> model       (weights unset)
    load_weights(tensors: dict) / init_random(seed)
    alloc_cache(n_blocks, block_size)
    forward(tokens, positions, params, last_token_idxes=None) -> logits [rows, vocab]
    n_vocab: int ; needs_state_slots: bool ; CSRC: the kernel sources it runs on
"""
from __future__ import annotations

import os
from typing import Callable, Dict

import torch

from . import checkpoint

_MODELS: Dict[str, Callable] = {}


def register_model(*names: str):
    def deco(cls):
        for n in names:
            _MODELS[n.lower()] = cls
        return cls
    return deco


def architecture_of(config: dict) -> str:
    if "architecture" in config:
        return str(config["architecture"])
    if config.get("architectures"):
        return str(config["architectures"][0])
    if "model_type" in config:
        return str(config["model_type"])
    raise ValueError("config.json names no architecture")


def model_class(config: dict):
    _import_builtin()
    name = architecture_of(config).lower()
    if name not in _MODELS:
        raise ValueError(f"no model registered for architecture {architecture_of(config)!r}; known: {sorted(_MODELS)}")
    return _MODELS[name]


def create_model(config: dict, dtype: torch.dtype, device, max_seqs: int = 4):
    return model_class(config).from_config(config, dtype, device, max_seqs)


def load_model(model_dir: str, dtype: torch.dtype, device, max_seqs: int = 4):
    """Model of a folder with config.json + model.safetensors, weights on the device in `dtype`."""
    config = checkpoint.read_config(model_dir)
    model = create_model(config, dtype, device, max_seqs)
    model.load_weights(checkpoint.read_safetensors(os.path.join(model_dir, "model.safetensors"), device))
    return model


def _import_builtin() -> None:
    from . import decode_step, fesupel, kigalix, pokadra, zomurax  # noqa: F401  (their classes register themselves)
