"""Causal multi-head attention over the paged cache.

One fused projection gives Q | K | V (column thirds, head h = columns
h*dh..h*dh+dh-1 of its third: src/kernels/prefill/flashattention.cu:60-64,
100-111); keys and values of the step's tokens go to their page slots before
attention (src/kernels/prefill/append_kv.cu:28-46); every query at absolute
position p attends to cached positions <= p of its own request with
score = (q.k)*scale and a 32-bit softmax (src/kernels/prefill/flashattention.cu:
129-168, src/kernels/decode/paged_attention.cu:60-120, without the latter's
+1e-6 on the denominator); the output projection adds its bias and the
residual in its epilogue (src/model/gpt2_model.cu:326-334).

Unlike the reference's prefill kernel, which reads the step's own QKV buffer
and therefore needs the whole prompt at once (src/model/gpt2_model.cu:307-324),
every query here reads the cache, so a prompt can be cut anywhere.
"""
from __future__ import annotations

from typing import Optional

from ..cache.manager import PagedNeed
from .base import Mixer, ParamSpec, register_part


class Attention(Mixer):
    accepts_lazy_norm = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, scale: float,
                 num_kv_heads: Optional[int] = None, window: Optional[int] = None, bias: bool = True):
        self.hidden_size = int(hidden_size)
        self.num_heads = int(num_heads)
        self.num_kv_heads = int(num_kv_heads if num_kv_heads is not None else num_heads)
        self.head_dim = int(head_dim)
        self.scale = float(scale)
        self.window = None if window is None else int(window)
        self.has_bias = bool(bias)
        if self.num_heads % self.num_kv_heads != 0:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.qkv_bias = None
        self.out_bias = None
        self.positions = None

    def param_specs(self):
        p = {"qkv_weight": ParamSpec((self.q_size + 2 * self.kv_size, self.hidden_size), "matrix"),
             "out_weight": ParamSpec((self.hidden_size, self.q_size), "matrix")}
        if self.has_bias:
            p["qkv_bias"] = ParamSpec((self.q_size + 2 * self.kv_size,), "vector")
            p["out_bias"] = ParamSpec((self.hidden_size,), "vector")
        return p

    def kernel_limits(self, dtype: str):
        # every attention kernel of the library works on head sizes that are multiples of 16 from 16 to 256
        # (16-byte pieces of a key row per lane; mma tiles of 16): anything else has no kernel
        if self.head_dim % 16 != 0 or not (16 <= self.head_dim <= 256):
            return [f"attention: head size {self.head_dim} (hidden size {self.hidden_size} over {self.num_heads} heads) "
                    f"is not a multiple of 16 between 16 and 256, the sizes the attention kernels take"]
        return []

    def cache_need(self):
        return PagedNeed(kv_heads=self.num_kv_heads, head_dim=self.head_dim, window=self.window)

    def forward(self, h, ctx, cache, out_accum):
        ops = self.rt.ops
        T = h.shape[0]
        gv = ctx.groups[cache.group]
        rotates = self.positions is not None and getattr(self.positions, "acts_on_qk", False)
        if cache.write and not rotates:
            # keys and values go to their page slots from the projection itself
            q = ops.linear_qkv_cache(h, self.qkv_weight, self.qkv_bias,
                                     ctx.ws.buf("q", T, self.q_size, self.rt.act_dtype), cache.k_pages,
                                     cache.v_pages, gv.slot_mapping, ctx.ws)
        else:
            qkv = ctx.ws.buf("qkv", T, self.q_size + 2 * self.kv_size, self.rt.act_dtype)
            ops.linear(h, self.qkv_weight, self.qkv_bias, out=qkv)
            q = qkv[:, :self.q_size]
            k = qkv[:, self.q_size:self.q_size + self.kv_size]
            v = qkv[:, self.q_size + self.kv_size:]
            if rotates:
                self.positions.apply_qk(q, k, ctx)
            if cache.write:
                ops.kv_write(k, v, cache.k_pages, cache.v_pages, gv.slot_mapping)
        att = ctx.ws.buf("attn_out", T, self.q_size, self.rt.act_dtype)
        ops.paged_attention(q, cache.k_pages, cache.v_pages, gv.block_table, ctx, att,
                            num_heads=self.num_heads, num_kv_heads=self.num_kv_heads,
                            head_dim=self.head_dim, scale=self.scale, window=self.window)
        ops.linear(att, self.out_weight, self.out_bias, out=out_accum, accumulate=True)


register_part("mixer", "attention", Attention)
