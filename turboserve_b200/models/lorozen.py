"""Lorozen: its configuration class and its builder, registered by name.

The architecture is a translation of its ``config.json`` into parts
(:meth:`LorozenConfig.to_model_spec`): per layer one of three mixers (windowed attention with biases and a learned sink,
latent attention with a gate per head, wkv time mixing) and a dense or routed feed-forward, each between two RMS norms
of its own; a stretch of layers that runs several times with the embedding's output added before each further pass; a
head whose logits are capped.
"""

from __future__ import annotations

import torch

from ..config.lorozen import ARCHITECTURE, LorozenConfig
from ..config.registry import register_architecture
from .decoder import DecoderModel


def build_lorozen(config: LorozenConfig, dtype: torch.dtype, device: torch.device | str) -> DecoderModel:
    return DecoderModel(config.to_model_spec(), dtype, device)


register_architecture(ARCHITECTURE, LorozenConfig, build_lorozen)
