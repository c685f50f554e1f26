"""Registers the Sudupel architecture: ``Sudupel`` -> ``SudupelConfig``.  As for every architecture the model is the
generic ``DecoderModel`` built from the specification the configuration lowers to: pairs of mixers side by side
(attention beside a recurrent block or beside gated linear attention), linear attention with fixed decays, norms on
both ends of every sublayer, a clamped gated feed-forward and routed experts, all of them registered parts that
another design may name too."""
from ..config.sudupel import ARCHITECTURE, SudupelConfig
from ..registry import register_architecture

register_architecture(ARCHITECTURE)(SudupelConfig)
