"""Causal grouped-query attention over the paged cache, with optional per-head
q/k RMSNorm and a position encoding applied to q and k.

Order of operations as the reference's block (docs/ARCHITECTURE.md:77-92,
src/kipp.c:2950-2993): q/k/v projections (no bias) -> per-head norm of q and k
-> rotation -> keys and values into the cache -> attention -> output
projection added to the residual stream.  The part itself: csrc/host/parts.hpp.

Options (each off by default): ``value_dim`` value heads of a size of their
own; ``keep_first`` a window keeps the first positions of the sequence visible;
``head_mix`` a tensor [heads, heads] mixes the heads' scores before the softmax;
``output_scale`` a factor on the mixer's output; ``bias`` biases of the q, k and
v projections; ``score_maps`` several score maps per head over the head's values
(q and k hold the maps of a head side by side); ``combine_maps`` with two maps
o = a1 - lambda a2, lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + ``lambda_init``,
then o / sqrt(mean(o^2) + ``combine_eps``) times (1 - lambda_init); ``names`` the
checkpoint names of its tensors by role (q, k, v, o, q_norm, k_norm, head_mix,
q_bias, k_bias, v_bias, lq1, lk1, lq2, lk2).
"""
from __future__ import annotations

from typing import Optional

from .base import Mixer, PagedKVSpec, PositionEncoding


class AttentionMixer(Mixer):
    kind = "attention"

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: PositionEncoding, qk_norm_eps: Optional[float] = None,
                 window: Optional[int] = None, scale: Optional[float] = None, *,
                 value_dim: Optional[int] = None, keep_first: int = 0, head_mix: bool = False,
                 output_scale: float = 1.0, bias: bool = False, score_maps: int = 1, combine_maps: bool = False,
                 lambda_init: float = 0.0, combine_eps: float = 1e-5, names: Optional[dict] = None,
                 sink: str = "none", head_gate: bool = False, softcap: float = 0.0, **more):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.position = position
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = scale
        self.q_dim = num_heads * score_maps * head_dim
        self.kv_dim = num_kv_heads * score_maps * head_dim
        self.value_dim, self.keep_first, self.head_mix = value_dim, keep_first, head_mix
        self.output_scale, self.names = output_scale, dict(names or {})
        self.bias, self.score_maps, self.combine_maps = bias, score_maps, combine_maps
        self.lambda_init, self.combine_eps = lambda_init, combine_eps
        # sink: none, learned (a number per head in the softmax's denominator) or unit; head_gate: a sigmoid gate
        # per head from the mixer's input; softcap c > 0: scores c tanh(s / c); `more`: further options of the
        # part by their plan names (norm_whole, interleaved, chunk, values_are_keys, shared_kv)
        self.sink, self.head_gate, self.softcap, self.more = sink, bool(head_gate), float(softcap), dict(more)

    def cache_spec(self) -> PagedKVSpec:
        # (the maps of a key head lie side by side in one row of the key pages)
        return PagedKVSpec(self.num_kv_heads, self.score_maps * self.head_dim, self.window,
                           self.value_dim or (self.head_dim if self.score_maps > 1 else None),
                           self.keep_first if self.window else 0)

    def params(self, prefix, ctx) -> dict:
        return {"hidden_size": self.hidden_size, "num_heads": self.num_heads, "num_kv_heads": self.num_kv_heads,
                "head_dim": self.head_dim, "position": self.position.describe(prefix, ctx),
                "qk_norm_eps": self.qk_norm_eps, "window": int(self.window or 0), "scale": self.scale,
                "value_dim": int(self.value_dim or 0), "keep_first": int(self.keep_first),
                "head_mix": bool(self.head_mix), "output_scale": float(self.output_scale), "bias": bool(self.bias),
                "score_maps": int(self.score_maps), "combine_maps": bool(self.combine_maps),
                "lambda_init": float(self.lambda_init), "combine_eps": float(self.combine_eps), "names": self.names,
                "sink": self.sink, "head_gate": self.head_gate, "softcap": self.softcap, **self.more}
