"""Bazulorn causal LM: the model class the registry hands out for ``"architecture": "Bazulorn"`` (blocks of one norm whose
mixers are attention beside a state space layer, or a gated delta rule; hashed token-pair embedding; tied logits;
`config.BazulornConfig`)."""
from __future__ import annotations

from ..config import BazulornConfig
from .hybrid import HybridForCausalLM


class BazulornForCausalLM(HybridForCausalLM):
    config_class = BazulornConfig
