"""Registers the Lodevik architecture: ``Lodevik`` -> ``LodevikConfig``.  As for every architecture the model is the
generic ``DecoderModel`` built from the specification the configuration lowers to: latent attention with a sink and a
gate per head, differential attention, the arrangement that norms a sublayer's output, the embedding with a scale and
a table looked up by pairs of tokens, all of them registered parts that another design may name too."""
from ..config.lodevik import ARCHITECTURE, LodevikConfig
from ..registry import register_architecture

register_architecture(ARCHITECTURE)(LodevikConfig)
