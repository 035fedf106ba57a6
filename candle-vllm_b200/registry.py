"""Model registry: ``config.json`` -> model class, the way the reference picks a pipeline from the ``architectures`` entry of a
checkpoint (src/openai/pipelines/pipeline.rs, ``get_arch_cfg``).  A model class offers
``from_pretrained(path, dtype=..., block_size=..., max_pos=...)``, ``cache_plan()`` and ``forward(batch, kv_cache, state_cache)``."""
from __future__ import annotations

import json
import os
from typing import Callable, Dict

from ._lib import BackendError

_REGISTRY: Dict[str, Callable] = {}


def register_model(architecture: str, loader: Callable) -> None:
    _REGISTRY[architecture] = loader


def architecture_of(config: dict) -> str:
    if "architecture" in config:
        return str(config["architecture"])
    archs = config.get("architectures")
    if archs:
        return str(archs[0])
    raise BackendError("config.json names no architecture")


# the source group (build.GROUPS) whose library alone serves an architecture, for a first start from a source-only checkout
_BUILD_GROUP = {"Gobesun": "ragged", "Guvusun": "latent", "Panarax": "hybrid", "Dofevik": "window"}


def build_group_of(path: str) -> str:
    with open(os.path.join(path, "config.json")) as f:
        return _BUILD_GROUP.get(architecture_of(json.load(f)), "ragged")


def registered() -> list:
    return sorted(_REGISTRY)


def load_model(path: str, **kw):
    with open(os.path.join(path, "config.json")) as f:
        arch = architecture_of(json.load(f))
    if arch not in _REGISTRY:
        raise BackendError(f"no model registered for architecture {arch!r} (have: {', '.join(registered())})")
    return _REGISTRY[arch](path, **kw)


def _gobesun(path, **kw):
    from .gobesun import GobesunModel
    return GobesunModel.from_pretrained(path, **kw)


def _guvusun(path, **kw):
    from .guvusun import GuvusunModel
    return GuvusunModel.from_pretrained(path, **kw)


def _panarax(path, **kw):
    from .panarax import PanaraxModel
    return PanaraxModel.from_pretrained(path, **kw)


def _dofevik(path, **kw):
    from .dofevik import DofevikModel
    return DofevikModel.from_pretrained(path, **kw)


def _llama(path, **kw):
    from .llama import load_dense_checkpoint
    return load_dense_checkpoint(path, **kw)


register_model("Gobesun", _gobesun)
register_model("Guvusun", _guvusun)
register_model("Panarax", _panarax)
register_model("Dofevik", _dofevik)
register_model("LlamaForCausalLM", _llama)
