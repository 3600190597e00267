"""The Zasudra decoder: layers of three kinds (attention over blocks of positions
whose values are its keys; causal attention with a gate per head that may read
another layer's keys and values; the wkv recurrence), feed-forwards of routed
experts, a hashed token-pair table beside the token embedding and a norm on
every sublayer's output.  Its configuration checks and its plan are the host
core's (csrc/host/zasudra.hpp); this module registers the configuration class on
the Python side.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zasudra import ZasudraConfig
from .spec import ModelSpec


def build_zasudra(config: ZasudraConfig) -> ModelSpec:
    return ModelSpec.from_library(config)


register_architecture("Zasudra", ZasudraConfig, build_zasudra)
