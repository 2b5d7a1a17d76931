"""LayerNorm with its eps as a parameter.

Formula as the reference computes it (src/kernels/layernorm.cu:32-49): mean,
biased variance of the centred values, (x-mean)*rsqrt(var+eps)*gamma+beta, all
in 32-bit; the reference kernel is fixed to 768 columns (:12), this one takes
any width.
"""
from __future__ import annotations

from .base import Norm, ParamSpec, register_part


class LayerNorm(Norm):
    supports_lazy = True

    def __init__(self, hidden_size: int, eps: float):
        self.hidden_size = int(hidden_size)
        self.eps = float(eps)

    def param_specs(self):
        return {"weight": ParamSpec((self.hidden_size,), "vector"),
                "bias": ParamSpec((self.hidden_size,), "vector")}

    def forward(self, x, ctx, rows=None, lazy=False):
        """``lazy``: the consumer is a product that can fuse the norm into its loads; it gets
        a NormedInput instead of a tensor (and may still ask for the tensor)."""
        if lazy:
            return self.rt.ops.NormedInput(x, self.weight, self.bias, self.eps, rows, ctx.ws, self.rt.act_dtype)
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.buf("norm_out", n, self.hidden_size, self.rt.act_dtype)
        self.rt.ops.layernorm(x, self.weight, self.bias, self.eps, out, rows=rows)
        return out


register_part("norm", "layernorm", LayerNorm)
