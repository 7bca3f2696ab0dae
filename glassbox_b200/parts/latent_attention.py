"""Causal attention over a compressed (latent) cache.

h -> q = h Wq^T, per head [nope_dim unrotated | rope_dim rotated]; [latent | shared key part] = h Wdkv^T. The latent is
RMS-normed (plain gain), the shared key part and every head's rotated query part are rotated at the row's position
(interleaved pairs), and latent + rotated key part are what the cache keeps per token: one row of latent_dim + rope_dim
numbers, for all heads. A head's unrotated key is W_uk_h latent and its value W_uv_h latent, so

    score_h(row, j) = scale * ((W_uk_h^T q_nope_h) . latent_j + q_rope_h . key_rope_j)
    out_h(row)      = W_uv_h (sum_j p_j latent_j)

and the attention kernel never sees a per-head key or value: the up-projections are applied to the query before it and
to the weighted sum of latents after it (one small product per head each). The softmax may carry a sink logit per
head in its denominator. A layer with ``kv_source`` has no Wdkv: it reads the cache layer another layer wrote (the
schedule's ``writes_cache`` False) with its own queries, W_uk, W_uv and sink.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.binding import ParamSpec
from .base import Mixer, PagedKvSpec, build_part, register_part
from .linear import linear


class LatentAttention(Mixer):
    accepts_deferred_input = True
    launches_through_kernels_only = True
    can_overwrite_output = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        s = spec
        for name in ("num_heads", "latent_dim", "value_dim"):
            if getattr(s, name) <= 0:
                raise ValueError(f"latent attention: {name} must be positive, got {getattr(s, name)}")
        if s.nope_dim < 0 or s.rope_dim < 0 or s.nope_dim + s.rope_dim == 0:
            raise ValueError("latent attention: a head's query needs at least one number")
        if s.window is not None and s.window <= 0:
            raise ValueError(f"window {s.window} must be positive")
        self.hidden_size = hidden_size
        self.H, self.dq, self.r, self.dv, self.c = s.num_heads, s.nope_dim, s.rope_dim, s.value_dim, s.latent_dim
        self.owns_cache = s.kv_source is None
        self.position = build_part("position", s.position)
        if self.r and getattr(self.position, "pairing", None) != "interleaved":
            raise ValueError("latent attention rotates interleaved pairs: its position must be a rope with pairing 'interleaved'")
        if self.position.rotary_dim > self.r:
            raise ValueError(f"{self.position.rotary_dim} rotated numbers do not fit a rotated part of {self.r}")
        self.q_cols = self.H * (self.dq + self.r)

    def sub_parts(self):
        return {"position": self.position}

    def param_specs(self):
        d = self.hidden_size
        specs = {"w_uk": ParamSpec((self.H * self.dq, self.c)), "w_uv": ParamSpec((self.H * self.dv, self.c)),
                 "wo": ParamSpec((d, self.H * self.dv))}
        if self.owns_cache:
            specs["w_in"] = ParamSpec((self.q_cols + self.c + self.r, d), pieces=(self.q_cols, self.c + self.r))
            specs["latent_norm"] = ParamSpec((self.c,), role="gain")
        else:
            specs["w_in"] = ParamSpec((self.q_cols, d))
        if self.spec.sink:
            specs["sink"] = ParamSpec((self.H,), role="gain")
        return specs

    def bind(self, params) -> None:
        super().bind(params)
        # W_uk is applied to the query: per head the [latent_dim, nope_dim] transpose, contiguous, as a product's weight
        w_uk = self.params["w_uk"]
        self.w_uk_t = w_uk.view(self.H, self.dq, self.c).transpose(1, 2).contiguous() if self.dq else None
        self.w_uv = self.params["w_uv"].view(self.H, self.dv, self.c).contiguous()

    def cache_spec(self):
        return PagedKvSpec(1, self.c + self.r, self.spec.window, value_dim=0)

    def forward(self, ctx, h, residual, cache, writes_cache: bool) -> None:
        n = h.shape[0]
        H, dq, r, dv, c = self.H, self.dq, self.r, self.dv, self.c
        if writes_cache and not self.owns_cache:
            raise ValueError("a latent attention layer without a projection of its own cannot write a cache layer")
        width = self.q_cols + (c + r if self.owns_cache else 0)
        proj = ctx.scratch("latent_proj", (n, width))
        linear(ctx, h, self.params["w_in"], proj)
        qabs = ctx.scratch("latent_q", (n, H * (c + r)))
        kernels.latent_kv_write(proj, self.q_cols, qabs, cache.k, self.params.get("latent_norm"),
                                self.position.inv_freq(proj.device) if r else proj.new_zeros(1, dtype=torch.float32),
                                ctx.positions, cache.slots, H, dq, r, c, self.position.rotary_dim if r else 0,
                                self.spec.latent_eps, writes_cache and self.owns_cache, ctx.status)
        # the key up-projection, applied to the query: one launch for all heads where the sizes allow, else head by head
        if dq and kernels.head_linear_supported(proj, self.w_uk_t, qabs, dq + r, c + r):
            kernels.head_linear(proj, self.w_uk_t, qabs, dq + r, c + r)
        else:
            q3 = qabs.view(n, H, c + r)
            p3 = proj[:, :self.q_cols].unflatten(1, (H, dq + r))
            for head in range(H):
                if dq:
                    linear(ctx, p3[:, head, :dq], self.w_uk_t[head], q3[:, head, :c])
                else:
                    q3[:, head, :c].zero_()
        lat = ctx.scratch("latent_out", (n, H * c))
        self.attend(ctx, qabs, lat, cache)
        att = ctx.scratch("att", (n, H * dv))
        # the value up-projection, applied to the weighted sum of latents
        if kernels.head_linear_supported(lat, self.w_uv, att, c, dv):
            kernels.head_linear(lat, self.w_uv, att, c, dv)
        else:
            l3, a3 = lat.view(n, H, c), att.view(n, H, dv)
            for head in range(H):
                linear(ctx, l3[:, head, :], self.w_uv[head], a3[:, head, :])
        linear(ctx, att, self.params["wo"], residual, accumulate=not getattr(ctx, "overwrite_output", False))

    def attend(self, ctx, qabs, lat, cache) -> None:
        """lat[row, head, :] = the softmax-weighted sum of the latents the row sees. bfloat16 at the sizes the
        tensor-core kernel is built for: decode steps cut each row's keys into shares so that few requests still fill the
        GPU; steps with prompt portions run tiles of tokens x heads. Anything else: one warp per (row, head)."""
        n = qabs.shape[0]
        if kernels.latent_attention_mma_supported(qabs.dtype, self.c, self.r, cache.page_size):
            common = (qabs, lat, cache.k, cache.block_tables, ctx.seq_first_row, ctx.seq_start_pos, ctx.positions,
                      self.params.get("sink"), self.H, self.c, self.r, cache.page_size, self.spec.scale, self.spec.window,
                      ctx.status)
            if ctx.decode_only:
                window = self.spec.window or ctx.max_context
                splits = kernels.latent_decode_splits(n, self.H, min(ctx.max_context, window))
                part_o = part_ml = None
                if splits > 1:
                    part_o = ctx.scratch("latent_part_o", (n, self.H * splits * self.c), torch.float32, grow=True)
                    part_ml = ctx.scratch("latent_part_ml", (n, self.H * splits * 2), torch.float32, grow=True)
                kernels.latent_attention_mma(*common, decode=True, splits=splits, part_o=part_o, part_ml=part_ml)
            else:
                kernels.latent_attention_mma(*common, max_rows_per_seq=ctx.max_rows_per_seq)
            return
        kernels.latent_attention_rows(qabs, lat, cache.k, cache.block_tables, ctx.row_seq, ctx.positions,
                                      self.params.get("sink"), self.H, self.c, self.r, cache.page_size, self.spec.scale,
                                      self.spec.window, ctx.status)


register_part("mixer", "latent_attention", LatentAttention, replace=True)
