"""minGRU: a gated recurrence whose gate and candidate read only the current token.

h -> one stacked product gives, as float32 sums, the gate's logits (W_z h), the candidate's input (W_x h) and the output
gate's input (W_g h), `width` columns each. Per channel, along a request's tokens:

    z_t = sigmoid(W_z h_t + b_z)
    c_t = u_t + 1/2 where u_t >= 0, sigmoid(u_t) elsewhere,  u_t = W_x h_t + b_x     (a positive, continuous candidate)
    S_t = (1 - z_t) S_(t-1) + z_t c_t

and the mixer's output is W_o (S_t * silu(W_g h_t)). S is `width` float32 numbers in the request's state slot: zero when
the request starts, carried from step to step, copied on fork, given back at the end. Since z and c do not depend on S,
a portion of a prompt is a first-order linear recurrence that the kernel cuts into pieces and chains. Gate, candidate,
state and the product with the output gate are float32 whatever the activation dtype.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.binding import ParamSpec
from .base import Mixer, StateSpec, register_part
from .linear import linear


class MinGru(Mixer):
    launches_through_kernels_only = True
    can_overwrite_output = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        if spec.width <= 0:
            raise ValueError(f"width {spec.width} must be positive")
        self.hidden_size, self.width = hidden_size, spec.width

    def param_specs(self):
        d, w = self.hidden_size, self.width
        return {"w_in": ParamSpec((3 * w, d), pieces=(w, w, w)),
                "bias_z": ParamSpec((w,), role="gain", init=(-2.0, 1.0)),
                "bias_x": ParamSpec((w,), role="gain", init=(0.0, 0.2)),
                "wo": ParamSpec((d, w))}

    def cache_spec(self):
        """One float32 row per request: S [width]."""
        return StateSpec((self.width,), torch.float32)

    def forward(self, ctx, h, residual, cache, writes_cache: bool) -> None:
        n, w = h.shape[0], self.width
        ld = -(-3 * w // 4) * 4
        proj = ctx.scratch("mingru_proj", (n, ld), torch.float32)[:, :3 * w]
        linear(ctx, h, self.params["w_in"], proj)
        gated = ctx.scratch("att", (n, w))
        kernels.mingru_scan(proj, self.params["bias_z"], self.params["bias_x"], cache.state, 0, gated, ctx.seq_first_row,
                            ctx.seq_start_pos, ctx.seq_slots, w, writes_cache, ctx.status,
                            max_rows=1 if ctx.decode_only else ctx.max_rows_per_seq)
        linear(ctx, gated, self.params["wo"], residual, accumulate=not getattr(ctx, "overwrite_output", False))


register_part("mixer", "mingru", MinGru, replace=True)
