"""Registers the Nuvilorn architecture: ``Nuvilorn`` -> ``NuvilornConfig``.  As for every
architecture the model is the generic ``DecoderModel`` built from the specification the
configuration lowers to: latent-attention mixers, dense or routed feed-forwards, norms with a
single gain, all of them registered parts that another design may name too."""
from ..config.nuvilorn import ARCHITECTURE, NuvilornConfig
from ..registry import register_architecture

register_architecture(ARCHITECTURE)(NuvilornConfig)
