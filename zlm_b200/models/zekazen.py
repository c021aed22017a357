"""Registers the Zekazen architecture: ``Zekazen`` -> ``ZekazenConfig``.  As for every architecture the model
is the generic ``DecoderModel`` built from the specification the configuration lowers to: retention and
convolved windowed attention mixers, routed gated experts with identity experts, all of them registered parts
that another design may name too."""
from ..config.zekazen import ARCHITECTURE, ZekazenConfig
from ..registry import register_architecture

register_architecture(ARCHITECTURE)(ZekazenConfig)
