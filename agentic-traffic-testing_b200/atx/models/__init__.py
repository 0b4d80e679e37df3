"""Model registry: which configuration class, weight container and layer program serve an architecture.

`architecture` (config.json) or HF's `model_type` picks the entry. The Llama family is the runner's built-in layer
schedule (ModelRunner._forward, tensor-parallel paths included); every other family brings a program object that the
runner calls for buffers, per-step staging and the kernel sequence, so that scheduler, paged cache, state slots,
staging, CUDA graphs, sampling and the engine loop are shared by all of them."""
from __future__ import annotations

from typing import Optional


def _entries():
    from . import gopopel, napuzen, safisun, zonidra

    return {"safisun": safisun, "gopopel": gopopel, "zonidra": zonidra, "napuzen": napuzen}


def _module(arch: str):
    mod = _entries().get(str(arch).lower())
    if mod is None:
        raise ValueError(f"unknown architecture {arch!r}; known: llama, {', '.join(sorted(_entries()))}")
    return mod


def config_class_for(arch: str):
    return _module(arch).Config


def load_weights(mcfg, path, device, dtype):
    return _module(mcfg.architecture).Weights.from_dir(mcfg, path, device, dtype)


def random_weights(mcfg, seed: int, device, dtype):
    return _module(mcfg.architecture).Weights.random(mcfg, seed, device, dtype)


def make_program(runner):
    """The layer program of a non-Llama family (None: the runner's own Llama schedule)."""
    arch = getattr(runner.m, "architecture", "llama")
    if arch == "llama":
        return None
    return _module(arch).Program(runner)


def random_shape(name: str) -> Optional[object]:
    """A named random-init shape of a non-Llama family (`random:<name>`), or None."""
    for mod in _entries().values():
        cfg = mod.named_shape(name)
        if cfg is not None:
            return cfg
    return None
