"""Causal grouped-query attention whose weights are not a softmax.

h -> one stacked product gives q (heads x head_dim), k (kv heads x head_dim) and v (kv heads x value_dim) as float32 sums
-> every query and key head is RMS-normed over head_dim (one gain shared by the query heads, one by the key heads), then
the first rotary_dim channels of each are rotated in neighbouring pairs (2i, 2i+1) at the row's position; k (normed and
rotated) and v go into the paged cache at the row's slot (all rows of the step before any attention) -> per (row, head)
out = sum over the row's visible keys j of sigmoid(q.k_j * scale + b_head) * v_j: every key weighs on its own, nothing is
normalised over the keys -> residual += out Wo^T. A window w lets position p see keys p-w+1 .. p; pages behind the window
of every future query go back to the pool, as for any windowed paged group. Norms, angles, scores, weights and the sums
over keys are float32 whatever the activation dtype; the cache holds the activation dtype.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.binding import ParamSpec
from .base import Mixer, PagedKvSpec, build_part, register_part
from .linear import linear


class SigmoidAttention(Mixer):
    launches_through_kernels_only = True
    can_overwrite_output = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        s = spec
        if s.num_heads <= 0 or s.num_kv_heads <= 0 or s.num_heads % s.num_kv_heads:
            raise ValueError(f"num_heads {s.num_heads} is not a multiple of num_kv_heads {s.num_kv_heads}")
        if not 0 < s.head_dim <= 256 or not 0 < s.value_dim <= 256:
            raise ValueError(f"head_dim {s.head_dim} and value_dim {s.value_dim} must lie in 1..256")
        if s.window is not None and s.window <= 0:
            raise ValueError(f"window {s.window} must be positive")
        self.hidden_size = hidden_size
        self.H, self.G, self.D, self.V = s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim
        self.position = build_part("position", s.position)
        self.rot = int(getattr(self.position, "rotary_dim", 0))
        if self.rot and getattr(self.position, "pairing", None) != "interleaved":
            raise ValueError("sigmoid attention rotates channel 2i with channel 2i + 1 only (pairing 'interleaved')")
        if self.rot > self.D:
            raise ValueError(f"rotary_dim {self.rot} exceeds head_dim {self.D}")
        self.in_cols = (self.H + self.G) * self.D + self.G * self.V

    def sub_parts(self):
        return {"position": self.position}

    def param_specs(self):
        d, s = self.hidden_size, self.spec
        specs = {"w_in": ParamSpec((self.in_cols, d), pieces=(self.H * self.D, self.G * self.D, self.G * self.V)),
                 "wo": ParamSpec((d, self.H * self.V))}
        if s.qk_norm_eps is not None:
            specs["q_norm"] = ParamSpec((self.D,), role="gain")
            specs["k_norm"] = ParamSpec((self.D,), role="gain")
        if s.head_bias:
            specs["head_bias"] = ParamSpec((self.H,), role="gain", init=(-2.0, 0.3))
        return specs

    def cache_spec(self):
        return PagedKvSpec(self.G, self.D, self.spec.window, value_dim=self.V)

    def forward(self, ctx, h, residual, cache, writes_cache: bool) -> None:
        n, s = h.shape[0], self.spec
        ld = -(-self.in_cols // 4) * 4                      # rows of the float32 buffer start 16-byte aligned
        qkv = ctx.scratch("sa_qkv", (n, ld), torch.float32)[:, :self.in_cols]
        linear(ctx, h, self.params["w_in"], qkv)
        q = ctx.scratch("sa_q", (n, self.H * self.D))
        inv_freq = self.position.inv_freq(q.device) if self.rot else None
        kernels.qk_norm_rope_write(qkv, self.params.get("q_norm"), self.params.get("k_norm"), inv_freq, ctx.positions, cache.slots, q,
                                   cache.k, cache.v, self.H, self.G, self.D, self.V, self.rot, s.qk_norm_eps or 0.0, cache.page_size,
                                   writes_cache, ctx.status)
        att = ctx.scratch("att", (n, self.H * self.V))
        self.attend(ctx, q, att, cache)
        linear(ctx, att, self.params["wo"], residual, accumulate=not getattr(ctx, "overwrite_output", False))

    def attend(self, ctx, q, att, cache) -> None:
        """Single decoded tokens take the kernel that shares a row's keys between the warps of a block; prompt portions in
        bfloat16 at head sizes the tile kernel is built for run on the tensor cores; everything else (float32 portions,
        other sizes) takes the one-warp-per-(row, head) kernel."""
        if ctx.decode_only and kernels.sigmoid_attention_decode_supported(q.dtype, self.V):
            kernels.sigmoid_attention_decode(q, att, cache.k, cache.v, cache.block_tables, ctx.row_seq, ctx.positions,
                                             self.params.get("head_bias"), self.H, self.G, self.D, self.V, cache.page_size,
                                             self.spec.scale, self.spec.window, ctx.status)
            return
        if not ctx.decode_only and kernels.sigmoid_attention_tiles_supported(q.dtype, self.D, self.V):
            kernels.sigmoid_attention_tiles(q, att, cache.k, cache.v, cache.block_tables, ctx.seq_first_row, ctx.seq_start_pos,
                                            ctx.max_rows_per_seq, self.params.get("head_bias"), self.H, self.G, self.D, self.V,
                                            cache.page_size, self.spec.scale, self.spec.window, ctx.status)
            return
        kernels.sigmoid_attention_rows(q, att, cache.k, cache.v, cache.block_tables, ctx.row_seq, ctx.positions,
                                       self.params.get("head_bias"), self.H, self.G, self.D, self.V, cache.page_size,
                                       self.spec.scale, self.spec.window, ctx.status)


register_part("mixer", "sigmoid_attention", SigmoidAttention, replace=True)
