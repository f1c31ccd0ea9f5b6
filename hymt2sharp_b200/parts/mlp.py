"""Dense feed-forward with one up and one down projection: residual += W_down act(W_up x).

Activations: "xielu", with two learned numbers (p, q) stored as a tensor of two values:
act(z) = softplus(p) z^2 + z/2 for z > 0, and (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2 for z <= 0;
"relu2", the square of relu, act(z) = max(z, 0)^2, which has no tensor of its own.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import register_part
from .linear import Linear, compute_form

ACTIVATIONS = ("xielu", "relu2")


class DenseMLP:
    graph_safe = True
    can_store = True   # forward(..., store=True) overwrites `residual` with its output instead of adding to it

    def __init__(self, hidden: int, intermediate: int, activation: str, up_proj: str, down_proj: str, act_params: str | None = None):
        if activation not in ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not known (known: {', '.join(ACTIVATIONS)})")
        self.hidden, self.intermediate, self.activation = int(hidden), int(intermediate), activation
        self.names = dict(u=up_proj, d=down_proj, a=act_params)
        self.up = self.down = self.pq = None

    def tensors(self):
        n = self.names
        t = {n["u"]: TensorSpec((self.intermediate, self.hidden)), n["d"]: TensorSpec((self.hidden, self.intermediate))}
        if self.activation == "xielu":
            t[n["a"]] = TensorSpec((2,))
        return t

    def load(self, weights, device, dtype):
        n = self.names
        self.up = Linear(compute_form(weights[n["u"]], device, dtype), role="up")
        self.down = Linear(compute_form(weights[n["d"]], device, dtype), ops.EPILOGUE_ACCUMULATE, role="down")
        self.down_store = Linear(self.down.weight, ops.EPILOGUE_STORE, role="down")
        if self.activation == "xielu":
            self.pq = weights[n["a"]].to(device).float().contiguous()

    def first_weights(self):
        return self.up.weight if self.up is not None else None

    def forward(self, x, residual: torch.Tensor, ctx, store: bool = False) -> None:
        z = self.up(x, ctx=ctx)
        if self.activation == "xielu":
            ops.xielu(z, z, self.pq)
        else:
            ops.relu_squared(z, z)
        if store:
            self.down_store(z, out=residual)
        else:
            self.down.add_then_norm(z, residual, getattr(ctx, "norm_ahead", None), ctx)


register_part("feed_forward", "dense_mlp", DenseMLP)
