"""Begovik: its configuration class and its builder, registered by name.

The architecture is a translation of its ``config.json`` into parts
(:meth:`BegovikConfig.to_model_spec`): per layer one of three mixers (attention with a sink beside lightning
attention, wkv time mixing, the selective scan) and a clamped gated feed-forward, both reading the stream through
RMS norms and entering it together times a factor; a scaled embedding and a head of its own.
"""

from __future__ import annotations

import torch

from ..config.begovik import ARCHITECTURE, BegovikConfig
from ..config.registry import register_architecture
from .decoder import DecoderModel


def build_begovik(config: BegovikConfig, dtype: torch.dtype, device: torch.device | str) -> DecoderModel:
    return DecoderModel(config.to_model_spec(), dtype, device)


register_architecture(ARCHITECTURE, BegovikConfig, build_begovik)
