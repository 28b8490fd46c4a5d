"""Model registry: ``config.json`` → configuration class and model class.

A checkpoint names its design with ``"architecture"`` (or the HF-style ``"model_type"`` / ``"architectures"``); a
directory without any of them is a LLaMA checkpoint, as every directory was before the registry existed.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Optional, Tuple

from ..config import CONFIG_NAME, BazulornConfig, DatozenConfig, FoliraxConfig, LLaMAConfig, NikonexConfig

_REGISTRY: Dict[str, Tuple[Any, Callable[[], Any]]] = {}
_KERNEL_SUBSET: Dict[str, Optional[str]] = {}
_DTYPES: Dict[str, Tuple[str, ...]] = {}


def register(name: str, config_class: Any, model_class_loader: Callable[[], Any], kernel_subset: Optional[str] = None,
             dtypes: Tuple[str, ...] = ("bfloat16",)) -> None:
    """`model_class_loader` returns the class when called, so registering a design imports nothing heavy.
    `kernel_subset`: the part of the native library this design needs (`ops/build.py` SUBSETS; None = all of it);
    `dtypes`: compute types its GPU engine runs in."""
    _REGISTRY[name.lower()] = (config_class, model_class_loader)
    _KERNEL_SUBSET[name.lower()] = kernel_subset
    _DTYPES[name.lower()] = tuple(dtypes)


def kernel_subset(name: str) -> Optional[str]:
    return _KERNEL_SUBSET[name.lower()]


def gpu_dtypes(name: str) -> Tuple[str, ...]:
    return _DTYPES[name.lower()]


def _llama() -> Any:
    from .llama import LLaMAForCausalLM
    return LLaMAForCausalLM


def _folirax() -> Any:
    from .folirax import FoliraxForCausalLM
    return FoliraxForCausalLM


def _nikonex() -> Any:
    from .nikonex import NikonexForCausalLM
    return NikonexForCausalLM


def _bazulorn() -> Any:
    from .bazulorn import BazulornForCausalLM
    return BazulornForCausalLM


def _datozen() -> Any:
    from .datozen import DatozenForCausalLM
    return DatozenForCausalLM


register("llama", LLaMAConfig, _llama)
register("folirax", FoliraxConfig, _folirax, kernel_subset="hybrid", dtypes=("bfloat16", "float32"))
register("nikonex", NikonexConfig, _nikonex, kernel_subset="hybrid", dtypes=("bfloat16", "float32"))
register("bazulorn", BazulornConfig, _bazulorn, kernel_subset="hybrid", dtypes=("bfloat16", "float32"))
register("datozen", DatozenConfig, _datozen, kernel_subset="hybrid_attention", dtypes=("bfloat16", "float32"))


def architecture_of(config: Dict[str, Any]) -> str:
    name = config.get("architecture") or config.get("model_type")
    if not name and config.get("architectures"):
        name = str(config["architectures"][0]).replace("ForCausalLM", "")
    name = str(name or "llama").lower()
    if name not in _REGISTRY:
        raise KeyError(f"unknown architecture {name!r}; registered: {sorted(_REGISTRY)}")
    return name


def resolve(path: str) -> Tuple[str, Any, Any]:
    """(architecture, config class, model class) of a checkpoint directory."""
    with open(os.path.join(path, CONFIG_NAME) if os.path.isdir(path) else path) as f:
        name = architecture_of(json.load(f))
    cfg_cls, loader = _REGISTRY[name]
    return name, cfg_cls, loader()


def load_pretrained(path: str, dtype: Optional[Any] = None, device: Any = "cpu", **kwargs: Any) -> Any:
    """The model of whatever design the directory holds, with its parameters on `device`."""
    _, _, model_cls = resolve(path)
    return model_cls.from_pretrained(path, dtype=dtype, device=device, **kwargs)
