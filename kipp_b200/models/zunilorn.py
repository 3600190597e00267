"""The Zunilorn decoder: layers of two kinds (the selective state space layer in
its matrix-state form; grouped-query attention with a stretched rotation, capped
scores, a learned sink and a gate per head), feed-forwards that are gated with
limits (dense, or experts chosen by softmax scores with identity experts and a
shared expert), a residual stream of several copies joined by hyper-connections,
a span of layers that may run several times, and capped logits from the
embedding table.  Its configuration checks and its plan are the host core's
(csrc/host/zunilorn.hpp); this module registers the configuration class on the
Python side.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zunilorn import ZunilornConfig
from .spec import ModelSpec


def build_zunilorn(config: ZunilornConfig) -> ModelSpec:
    return ModelSpec.from_library(config)


register_architecture("Zunilorn", ZunilornConfig, build_zunilorn)
