"""Configuration of the Zasudra decoder, from its ``config.json`` keys.

The file is nested: ``layers`` lists the layers one by one (``type``
``attention``, ``attention_2`` or ``wkv``, the mixer's sizes and constants under
``mixer``, the routed feed-forward under ``mlp`` or null), ``embedding.bigram``
gives the hashed token-pair table, ``norm.eps`` is the eps of every norm,
``residual_mult`` scales what a sublayer adds to the stream, ``logit_scale``
the logits, and ``vocab`` / ``width`` are the two global sizes.  The model
class is named by the key ``architecture``.  The checks are the host core's
(csrc/host/zasudra.hpp); this class keeps the keys as they are.
"""
from __future__ import annotations

import copy
import dataclasses
import json
from typing import Any

from .base import ConfigError, ModelConfig, architecture_name


@dataclasses.dataclass(frozen=True)
class ZasudraConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm: dict = dataclasses.field(default_factory=dict)
    layers: tuple = ()
    embedding: dict | None = None
    residual_mult: float | None = None
    logit_scale: float | None = None

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "ZasudraConfig":
        if not isinstance(data, dict):
            raise ConfigError("config.json must hold a JSON object")
        for key in ("vocab", "width", "norm", "layers"):
            if key not in data:
                raise ConfigError(f"config.json lacks required key {key!r}")
        if not isinstance(data["layers"], (list, tuple)):
            raise ConfigError("config key 'layers' must be a list of layers")
        config = cls(architecture=architecture_name(data), vocab=data["vocab"], width=data["width"],
                     norm=copy.deepcopy(data["norm"]), layers=tuple(copy.deepcopy(list(data["layers"]))),
                     embedding=copy.deepcopy(data.get("embedding")), residual_mult=data.get("residual_mult"),
                     logit_scale=data.get("logit_scale"))
        config.validate()
        return config

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": copy.deepcopy(self.norm), "layers": copy.deepcopy(list(self.layers))}
        if self.embedding is not None:
            out["embedding"] = copy.deepcopy(self.embedding)
        if self.residual_mult is not None:
            out["residual_mult"] = self.residual_mult
        if self.logit_scale is not None:
            out["logit_scale"] = self.logit_scale
        return out

    # what code that sizes a run asks of any configuration
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def initializer_range(self) -> float:
        return 0.02

    def normalized(self) -> dict:
        """The keys after the host core's checks and defaults."""
        from .. import native as N
        return json.loads(N.text_result(N.lib().kipp_config_normalize, json.dumps(self.to_dict()).encode()))

    def validate(self) -> None:
        self.normalized()
