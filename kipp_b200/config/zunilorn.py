"""Configuration of the Zunilorn decoder, from its ``config.json`` keys.

The file is nested: ``layers`` lists the layers one by one (``type`` ``mamba2``
or ``attention``, the mixer's sizes and constants under ``mixer``, the
feed-forward under ``mlp``: ``kind`` ``dense`` or ``moe``, or null), ``loop``
names a span of layers that runs several times in a row, ``streams`` is the
number of copies of the residual stream that the hyper-connections join (absent:
one stream and a plain residual sum), ``residual_mult`` scales what a sublayer
adds, ``logit_softcap`` caps the logits, ``norm.eps`` is the eps of every norm,
and ``vocab`` / ``width`` are the two global sizes.  The model class is named by
the key ``architecture``.  The checks are the host core's
(csrc/host/zunilorn.hpp); this class keeps the keys as they are.
"""
from __future__ import annotations

import copy
import dataclasses
import json
from typing import Any

from .base import ConfigError, ModelConfig, architecture_name


@dataclasses.dataclass(frozen=True)
class ZunilornConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm: dict = dataclasses.field(default_factory=dict)
    layers: tuple = ()
    loop: dict | None = None
    streams: int | None = None
    residual_mult: float | None = None
    logit_softcap: float | None = None

    @classmethod
    def from_dict(cls, data: dict[str, Any]) -> "ZunilornConfig":
        if not isinstance(data, dict):
            raise ConfigError("config.json must hold a JSON object")
        for key in ("vocab", "width", "norm", "layers"):
            if key not in data:
                raise ConfigError(f"config.json lacks required key {key!r}")
        if not isinstance(data["layers"], (list, tuple)):
            raise ConfigError("config key 'layers' must be a list of layers")
        config = cls(architecture=architecture_name(data), vocab=data["vocab"], width=data["width"],
                     norm=copy.deepcopy(data["norm"]), layers=tuple(copy.deepcopy(list(data["layers"]))),
                     loop=copy.deepcopy(data.get("loop")), streams=data.get("streams"),
                     residual_mult=data.get("residual_mult"), logit_softcap=data.get("logit_softcap"))
        config.validate()
        return config

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": copy.deepcopy(self.norm), "layers": copy.deepcopy(list(self.layers))}
        for key in ("loop", "streams", "residual_mult", "logit_softcap"):
            if getattr(self, key) is not None:
                out[key] = copy.deepcopy(getattr(self, key))
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
