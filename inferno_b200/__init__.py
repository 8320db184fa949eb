"""B200-native causal attention (forward + backward) behind Inferno's operator conventions."""
from .synth import CONFIGS, AttnConfig, make_config_inputs, make_inputs  # noqa: F401

__all__ = ["CONFIGS", "AttnConfig", "make_config_inputs", "make_inputs"]
