"""Arrangement of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from .base import Block, FeedForward, Mixer, Norm


class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x)): the un-normed x is the
    residual stream (src/kipp.c:2948, 2994).  ``post_norm`` and ``ffn`` None: a
    block with the first sublayer only.  The part itself: csrc/host/parts.hpp."""
    kind = "pre_norm_block"

    def __init__(self, input_norm: Norm, mixer: Mixer, post_norm: Norm, ffn: FeedForward,
                 names: tuple[str, str, str, str] = ("input_layernorm.", "self_attn.",
                                                     "post_attention_layernorm.", "mlp.")):
        self.input_norm, self.mixer, self.post_norm, self.ffn = input_norm, mixer, post_norm, ffn
        self.names = tuple(names)

    def params(self, prefix, ctx) -> dict:
        parts = (self.input_norm, self.mixer, self.post_norm, self.ffn)
        described = [None if p is None else p.describe(prefix + n, ctx) for p, n in zip(parts, self.names)]
        return {"names": list(self.names), "input_norm": described[0], "mixer": described[1],
                "post_norm": described[2], "ffn": described[3]}


class ParallelBlock(Block):
    """x += mixer(n) + ffn(n) with n = norm(x): ONE norm whose output both
    sublayers read.  ``ffn`` None: the mixer only.  The part itself:
    csrc/host/parts.hpp."""
    kind = "parallel_block"

    def __init__(self, norm: Norm, mixer: Mixer, ffn: FeedForward, names: tuple[str, str, str] = ("norm.", "mix.", "mlp.")):
        self.norm, self.mixer, self.ffn = norm, mixer, ffn
        self.names = tuple(names)

    def params(self, prefix, ctx) -> dict:
        parts = (self.norm, self.mixer, self.ffn)
        described = [None if p is None else p.describe(prefix + n, ctx) for p, n in zip(parts, self.names)]
        return {"names": list(self.names), "norm": described[0], "mixer": described[1], "ffn": described[2]}


class HyperConnectionBlock(Block):
    """The residual stream as ``streams`` copies: sublayer q reads
    u = sum_s in_q[s] x_s through its RMS norm and its output y joins every copy,
    x_t <- sum_s mix_q[s, t] x_s + residual_mult * out_q[t] * y.  ``connections``
    False: one stream and the plain x <- x + residual_mult * sublayer(norm(x)).
    ``names``: prefixes of the two norms, the mixer, the feed-forward and the two
    sets of connection tensors.  The part itself: csrc/host/parts.hpp."""
    kind = "hyper_connection_block"

    def __init__(self, input_norm: Norm, mixer: Mixer, post_norm: Norm, ffn: FeedForward, *, streams: int = 1,
                 connections: bool = True, residual_mult: float = 1.0,
                 names: tuple = ("", "mix.", "", "mlp.", "hc1.", "hc2.")):
        self.input_norm, self.mixer, self.post_norm, self.ffn = input_norm, mixer, post_norm, ffn
        self.streams, self.connections, self.residual_mult = int(streams), bool(connections), float(residual_mult)
        self.names = tuple(names)

    def params(self, prefix, ctx) -> dict:
        parts = (self.input_norm, self.mixer, self.post_norm, self.ffn)
        described = [None if p is None else p.describe(prefix + n, ctx) for p, n in zip(parts, self.names)]
        return {"names": list(self.names), "streams": self.streams, "connections": self.connections,
                "residual_mult": self.residual_mult, "input_norm": described[0], "mixer": described[1],
                "post_norm": described[2], "ffn": described[3]}
