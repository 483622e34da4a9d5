"""Models: the generic decoder and the architectures registered on top of it."""

from .decoder import DecoderModel, NamedParam
from . import baporax, begovik, filezen, lorozen, qwen2  # noqa: F401  (register Baporax, Begovik, Filezen, Lorozen and Qwen2ForCausalLM)

__all__ = ["DecoderModel", "NamedParam"]
