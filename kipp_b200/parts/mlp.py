"""Dense SwiGLU feed-forward: x += W_down (silu(W_gate n) * (W_up n))
(src/kipp.c:2994-3010, silu src/kipp.c:2402-2404), and the dense feed-forward with
one up projection, x += W_down act(W_up n), and the gated feed-forward with
limits.  The parts themselves: csrc/host/parts.hpp."""
from __future__ import annotations

from .base import FeedForward


class SwiGLUFeedForward(FeedForward):
    kind = "swiglu"

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size

    def params(self, prefix, ctx) -> dict:
        return {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size}


class DenseFeedForward(FeedForward):
    """``activation``: relu, relu_squared, gelu_tanh or silu."""
    kind = "dense_mlp"

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu_squared",
                 names: dict | None = None):
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.names = dict(names or {})

    def params(self, prefix, ctx) -> dict:
        return {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
                "activation": self.activation, "names": self.names}


class GatedFeedForward(FeedForward):
    """x += W_down (g sigmoid(alpha g) (u + 1)) with g = min(W_gate n, limit) and
    u = clamp(W_up n, -limit, limit) (limit 0: none); ``bias``: biases on all three
    projections; ``row_gate``: the output is also multiplied by sigmoid(w . n), one
    number per token."""
    kind = "gated_mlp"

    def __init__(self, hidden_size: int, intermediate_size: int, *, limit: float = 0.0, alpha: float = 1.0,
                 bias: bool = False, row_gate: bool = False, names: dict | None = None):
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.limit, self.alpha, self.bias, self.row_gate = float(limit), float(alpha), bool(bias), bool(row_gate)
        self.names = dict(names or {})

    def params(self, prefix, ctx) -> dict:
        return {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size, "limit": self.limit,
                "alpha": self.alpha, "bias": self.bias, "row_gate": self.row_gate, "names": self.names}
