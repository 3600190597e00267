"""Mixers with a matrix state per request, a mixer made of several side by side,
and the feed-forward with a PolyNorm activation.  The parts themselves:
csrc/host/recurrent_parts.hpp; their kernels: csrc/recurrent.cu.

``RetentionMixer``      S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t per head (q, k rotated,
                        k scaled), each head's o divided by its root mean square, gated, projected.
``DeltaRuleMixer``      S_t = diag(w_t) S_{t-1} - (a_t u_t)(u_t^T S_{t-1}) + k_t v_t^T, o_t = S_t^T r_t.
``GatedMemoryMixer``    m_t = max(f_t + m_{t-1}, i_t), S_t = e^(f_t + m_{t-1} - m_t) S_{t-1} + e^(i_t - m_t) k_t v_t^T,
                        n_t alike, o_t = S_t^T q_t / (max(|n_t . q_t|, e^(-m_t)) + 1e-6): the matrix memory of the xLSTM.
``ParallelMixer``       the sum of its branches, each with its own cache or state and output_scale.
``PolyNormFeedForward`` W_down (c0 N(z) + c1 N(z^2) + c2 N(z^3) + c3), z = W_up h.
"""
from __future__ import annotations

from typing import Optional, Sequence

from .base import FeedForward, Mixer, PositionEncoding


class RetentionMixer(Mixer):
    kind = "retention"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, decay: Sequence[float],
                 position: PositionEncoding, eps: float, *, value_dim: Optional[int] = None,
                 gate: str = "silu", output_scale: float = 1.0, key_scale: Optional[float] = None,
                 names: Optional[dict] = None):
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, head_dim
        self.decay, self.position, self.eps = [float(d) for d in decay], position, eps
        self.value_dim, self.gate, self.output_scale = value_dim or head_dim, gate, output_scale
        self.key_scale, self.names = key_scale, dict(names or {})

    def params(self, prefix, ctx) -> dict:
        out = {"hidden_size": self.hidden_size, "num_heads": self.num_heads, "head_dim": self.head_dim,
               "value_dim": self.value_dim, "decay": self.decay, "position": self.position.describe(prefix, ctx),
               "eps": self.eps, "gate": self.gate, "output_scale": float(self.output_scale), "names": self.names}
        if self.key_scale is not None:
            out["key_scale"] = float(self.key_scale)
        return out


class DeltaRuleMixer(Mixer):
    kind = "delta_rule"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, decay_rank: int, eps: float, *,
                 gate: str = "sigmoid", output_scale: float = 1.0, names: Optional[dict] = None):
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, head_dim
        self.decay_rank, self.eps, self.gate, self.output_scale = decay_rank, eps, gate, output_scale
        self.names = dict(names or {})

    def params(self, prefix, ctx) -> dict:
        return {"hidden_size": self.hidden_size, "num_heads": self.num_heads, "head_dim": self.head_dim,
                "decay_rank": self.decay_rank, "eps": self.eps, "gate": self.gate,
                "output_scale": float(self.output_scale), "names": self.names}


class ParallelMixer(Mixer):
    kind = "parallel"

    def __init__(self, branches: Sequence[tuple]):
        """``branches``: (prefix, mixer) pairs; each mixer brings its own output_scale."""
        self.branches = list(branches)

    def params(self, prefix, ctx) -> dict:
        return {"branches": [{"prefix": p, "part": m.describe(prefix + p, ctx)} for p, m in self.branches]}


class PolyNormFeedForward(FeedForward):
    kind = "polynorm_mlp"

    def __init__(self, hidden_size: int, intermediate_size: int, eps: float, names: Optional[dict] = None):
        self.hidden_size, self.intermediate_size, self.eps = hidden_size, intermediate_size, eps
        self.names = dict(names or {})

    def params(self, prefix, ctx) -> dict:
        return {"hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size, "eps": self.eps,
                "names": self.names}


class GatedMemoryMixer(Mixer):
    kind = "gated_memory"

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, gate_cap: float, eps: float, *,
                 value_dim: Optional[int] = None, gate: str = "sigmoid", output_scale: float = 1.0,
                 query_scale: Optional[float] = None, names: Optional[dict] = None):
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, head_dim
        self.gate_cap, self.eps, self.value_dim = float(gate_cap), eps, value_dim or head_dim
        self.gate, self.output_scale, self.query_scale, self.names = gate, output_scale, query_scale, dict(names or {})

    def params(self, prefix, ctx) -> dict:
        out = {"hidden_size": self.hidden_size, "num_heads": self.num_heads, "head_dim": self.head_dim,
               "value_dim": self.value_dim, "gate_cap": self.gate_cap, "eps": self.eps, "gate": self.gate,
               "output_scale": float(self.output_scale), "names": self.names}
        if self.query_scale is not None:
            out["query_scale"] = float(self.query_scale)
        return out


class StateSpaceMixer(Mixer):
    """The selective state space layer in its matrix-state form: one projection
    [z | x | B | C | dt], a causal convolution of ``conv`` taps over x, B and C,
    S_t = exp(-exp(A) dt) S_(t-1) + dt B_t x_t^T per head (the heads of a group share
    B and C), y = S^T C + D x, the gate silu(z), a root-mean-square division in
    ``norm_groups`` parts.  Per request: S and the convolution's last inputs."""
    kind = "state_space"

    def __init__(self, hidden_size: int, num_heads: int, value_dim: int, state_dim: int, conv: int, eps: float, *,
                 groups: int = 1, norm_groups: int = 1, names: Optional[dict] = None):
        self.hidden_size, self.num_heads, self.value_dim, self.state_dim = hidden_size, num_heads, value_dim, state_dim
        self.conv, self.eps, self.groups, self.norm_groups, self.names = conv, eps, groups, norm_groups, dict(names or {})

    def params(self, prefix, ctx) -> dict:
        return {"hidden_size": self.hidden_size, "num_heads": self.num_heads, "value_dim": self.value_dim,
                "state_dim": self.state_dim, "conv": self.conv, "eps": self.eps, "groups": self.groups,
                "norm_groups": self.norm_groups, "names": self.names}
