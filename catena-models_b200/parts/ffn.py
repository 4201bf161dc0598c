"""Gated feed-forward: a = act(g) * u with g = x Wgate^T, u = x Wup^T, then Wdown; act is silu (SwiGLU) or tanh-gelu
(src/catena/lfm3.hex:833-845; fused epilogue src/catena/lfm3_wmma.hex:10790-10815).  Gate and up
are packed into one matrix at bind time so that one product reads x once
(src/lfm3.rs:1062-1075 fuses them in its kernel the same way).
"""
from __future__ import annotations

from .base import FeedForward, register_part
from .linear import Linear


class SwiGLU(FeedForward):
    prompt_capturable = True
    fused_decode_ok = True
    supports_append = True

    def __init__(self, prefix, hidden, intermediate, names=None, out_dtype=None, activation="silu", limit=0.0):
        """out_dtype "float32": the down projection's result stays in float (for a float residual stream).
        activation: what the gate passes through, "silu" or "gelu_tanh" (the tanh form of gelu), or "clamped_swish" with
        `limit` L: a = g' sigmoid(1.702 g') (u' + 1) with g' = min(g, L), u' = clamp(u, -L, L)."""
        import torch

        if activation not in ("silu", "gelu_tanh", "clamped_swish"):
            raise ValueError("SwiGLU: activation silu|gelu_tanh|clamped_swish")
        if activation == "clamped_swish" and not limit > 0.0:
            raise ValueError("SwiGLU: the clamped gate needs its limit")
        self.gelu = activation == "gelu_tanh"
        self.clamped, self.limit = activation == "clamped_swish", float(limit)
        if self.gelu or self.clamped:
            self.fused_decode_ok = False         # the persistent decode kernel's gated product has silu only
        self.out_dtype = {None: None, "float32": torch.float32}[out_dtype]
        names = names or {}
        n = lambda key, default: prefix + names.get(key, default)
        self.hidden, self.intermediate = hidden, intermediate
        self.gate_up = Linear([n("gate", "ffn_gate.weight"), n("up", "ffn_up.weight")],
                              [intermediate, intermediate], hidden)
        self.down = Linear(n("down", "ffn_down.weight"), hidden, intermediate)

    def children(self):
        return [self.gate_up, self.down]

    def forward(self, rt, batch, x):
        a = rt.gate_up_swiglu(x, self.gate_up.weight, self.intermediate, gelu=self.gelu,
                              limit=self.limit if self.clamped else None)
        return self.down.apply(rt, a, out_dtype=self.out_dtype, partial_ok=batch.partial_sums_ok and self.out_dtype is None)


class ReluSquared(FeedForward):
    """Plain two-matrix feed-forward with a squared ReLU between: W_down max(W_up x, 0)^2."""
    prompt_capturable = True
    supports_append = True

    def __init__(self, prefix, hidden, intermediate, names=None, out_dtype=None):
        import torch

        self.out_dtype = {None: None, "float32": torch.float32}[out_dtype]
        names = names or {}
        self.hidden, self.intermediate = hidden, intermediate
        self.up = Linear(prefix + names.get("up", "up"), intermediate, hidden)
        self.down = Linear(prefix + names.get("down", "down"), hidden, intermediate)

    def children(self):
        return [self.up, self.down]

    def forward(self, rt, batch, x):
        from .. import kernels

        a = self.up.apply(rt, x)
        kernels.relu2_inplace(a)
        return self.down.apply(rt, a, out_dtype=self.out_dtype, partial_ok=batch.partial_sums_ok and self.out_dtype is None)


class SumOfFeedForwards(FeedForward):
    """Several feed-forwards that read the same input; the result is the sum of theirs (a routed feed-forward and an
    expert that every token runs, say).  Each member hands over a tensor or `kernels.Terms`; the block's residual sum
    adds all pieces in the members' order."""
    prompt_capturable = True
    supports_append = True

    def __init__(self, members):
        self.members = list(members)
        if not self.members:
            raise ValueError("SumOfFeedForwards: no members")

    def children(self):
        return self.members

    def forward(self, rt, batch, x):
        from .. import kernels

        out = kernels.Terms()
        for member in self.members:
            y = member.forward(rt, batch, x)
            out += y if isinstance(y, kernels.Terms) else [(y, 1.0, 1)]
        return out


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "sum", SumOfFeedForwards)
register_part("feed_forward", "relu_squared", ReluSquared)
