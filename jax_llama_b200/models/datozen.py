"""Datozen causal LM: the model class the registry hands out for ``"architecture": "Datozen"`` (parallel blocks of one norm with
chunked, gated sink attention over rotated values, dense or mixture-of-experts feed-forwards with identity experts, a per-layer
token input, learned positions, a looped stretch of layers, tied logits; `config.DatozenConfig`)."""
from __future__ import annotations

from ..config import DatozenConfig
from .hybrid import HybridForCausalLM


class DatozenForCausalLM(HybridForCausalLM):
    config_class = DatozenConfig
