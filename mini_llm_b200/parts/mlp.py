"""Dense feed-forward: x += act(h @ W_fc^T + b_fc) @ W_proj^T + b_proj.

As in the reference the bias and the activation ride in the first product's
epilogue (src/kernels/linear.cu:48-66) and the bias and the residual sum in
the second's (src/kernels/linear.cu:28-46; src/model/gpt2_model.cu:345-363).
Activations: "gelu_tanh" (src/kernels/gemm.cu:17-20) and "gelu_erf".
"""
from __future__ import annotations

from .base import FeedForward, ParamSpec, register_part

ACTIVATIONS = ("gelu_tanh", "gelu_erf")


class MLP(FeedForward):
    accepts_lazy_norm = True

    def __init__(self, hidden_size: int, inner_size: int, activation: str, bias: bool = True):
        if activation not in ACTIVATIONS:
            raise ValueError(f"MLP activation must be one of {ACTIVATIONS}, got {activation!r}")
        self.hidden_size = int(hidden_size)
        self.inner_size = int(inner_size)
        self.activation = activation
        self.has_bias = bool(bias)
        self.fc_bias = None
        self.proj_bias = None

    def param_specs(self):
        p = {"fc_weight": ParamSpec((self.inner_size, self.hidden_size), "matrix"),
             "proj_weight": ParamSpec((self.hidden_size, self.inner_size), "matrix")}
        if self.has_bias:
            p["fc_bias"] = ParamSpec((self.inner_size,), "vector")
            p["proj_bias"] = ParamSpec((self.hidden_size,), "vector")
        return p

    def forward(self, h, ctx, out_accum):
        ops = self.rt.ops
        mid = ctx.ws.buf("ff_mid", h.shape[0], self.inner_size, self.rt.act_dtype)
        ops.linear(h, self.fc_weight, self.fc_bias, out=mid, act=self.activation)
        ops.linear(mid, self.proj_weight, self.proj_bias, out=out_accum, accumulate=True)


register_part("feed_forward", "mlp", MLP)
