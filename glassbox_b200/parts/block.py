"""A layer: a mixer and a feed-forward wired around the float32 residual stream.

"pre_norm" is x += mixer(norm(x)); x += ffn(norm(x)), with no norms after the parts
(crates/glassbox-core/src/model.rs:251-348). "sandwich_norm" norms each branch on the way out as well:
x += post(mixer(norm(x))); x += post(ffn(norm(x))). The arrangement is looked up by name, so another
wiring (post-norm, parallel branches) is another registered class.
"""
from __future__ import annotations

import torch

from .base import DeferredNorm, Part, build_part, register_part


class PreNormBlock(Part):
    launches_through_kernels_only = True

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        self.hidden_size = hidden_size
        self.mixer_norm = build_part("norm", spec.mixer_norm, hidden_size=hidden_size)
        self.mixer = build_part("mixer", spec.mixer, hidden_size=hidden_size)
        self.ffn_norm = build_part("norm", spec.ffn_norm, hidden_size=hidden_size)
        self.ffn = build_part("ffn", spec.ffn, hidden_size=hidden_size)

    def sub_parts(self):
        return {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "ffn_norm": self.ffn_norm, "ffn": self.ffn}

    def entry_norm(self):
        """The norm that reads the residual first when this layer runs (whoever runs the layer before may tell
        its last product, through ``ctx.next_norm``, to prepare it)."""
        return self.mixer_norm

    def forward(self, ctx, x, cache, writes_cache: bool, after_mixer=None) -> None:
        """``after_mixer`` (optional) is called once the mixer's kernels are launched: the model uses it
        to let the next layer's mixer start its prefetch beside this layer's feed-forward.
        ``ctx.norm_after_layer`` (optional) is the norm that will read ``x`` after this layer."""
        after_layer = getattr(ctx, "norm_after_layer", None)
        h = DeferredNorm(ctx, self.mixer_norm, x)
        ctx.next_norm = self.ffn_norm          # a hint to the product that adds the mixer's output into x
        self.mixer.forward(ctx, h if self.mixer.accepts_deferred_input else h.tensor(), x, cache, writes_cache)
        if after_mixer is not None:
            after_mixer()
        h = DeferredNorm(ctx, self.ffn_norm, x)
        ctx.next_norm = after_layer
        self.ffn.forward(ctx, h if self.ffn.accepts_deferred_input else h.tensor(), x)
        ctx.next_norm = None


class SandwichNormBlock(Part):
    """x += post_norm(mixer(norm(x))), then x += post_norm(ffn(norm(x))) (the second half only if the layer has a
    feed-forward). A branch cannot add into the residual stream itself, because its output is normed first: it is given
    a float32 buffer of the residual's shape instead. Parts that say ``can_overwrite_output`` store their result there
    (``ctx.overwrite_output`` tells them so); for any other part the buffer is cleared and the part adds into it as it
    would into the residual. The post norm then adds the normed branch into x (``Norm.add_normed``)."""
    launches_through_kernels_only = False      # (clearing the buffer for a part that adds is a torch operation)

    def __init__(self, spec, *, hidden_size: int):
        super().__init__(spec)
        if spec.mixer_post_norm is None or (spec.ffn is not None and spec.ffn_post_norm is None):
            raise ValueError("a sandwich_norm layer needs a norm behind its mixer and behind its feed-forward")
        self.hidden_size = hidden_size
        self.mixer_norm = build_part("norm", spec.mixer_norm, hidden_size=hidden_size)
        self.mixer = build_part("mixer", spec.mixer, hidden_size=hidden_size)
        self.mixer_post_norm = build_part("norm", spec.mixer_post_norm, hidden_size=hidden_size)
        self.ffn = self.ffn_norm = self.ffn_post_norm = None
        if spec.ffn is not None:
            self.ffn_norm = build_part("norm", spec.ffn_norm, hidden_size=hidden_size)
            self.ffn = build_part("ffn", spec.ffn, hidden_size=hidden_size)
            self.ffn_post_norm = build_part("norm", spec.ffn_post_norm, hidden_size=hidden_size)

    def sub_parts(self):
        parts = {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "mixer_post_norm": self.mixer_post_norm}
        if self.ffn is not None:
            parts.update({"ffn_norm": self.ffn_norm, "ffn": self.ffn, "ffn_post_norm": self.ffn_post_norm})
        return parts

    def entry_norm(self):
        return self.mixer_norm

    def _branch(self, ctx, part, norm, post, x, run) -> None:
        branch = ctx.scratch("branch", tuple(x.shape), torch.float32)
        ctx.overwrite_output = bool(part.can_overwrite_output)
        if not ctx.overwrite_output:
            branch.zero_()
        h = DeferredNorm(ctx, norm, x)
        try:
            run(h if part.accepts_deferred_input else h.tensor(), branch)
        finally:
            ctx.overwrite_output = False
        post.add_normed(ctx, branch, x)
        ctx.prepared_norm = None         # x has changed behind the back of whatever was prepared from it

    def forward(self, ctx, x, cache, writes_cache: bool, after_mixer=None) -> None:
        ctx.next_norm = None             # no product of this layer completes residual rows: nothing to prepare
        self._branch(ctx, self.mixer, self.mixer_norm, self.mixer_post_norm, x,
                     lambda h, out: self.mixer.forward(ctx, h, out, cache, writes_cache))
        if after_mixer is not None:
            after_mixer()
        if self.ffn is not None:
            self._branch(ctx, self.ffn, self.ffn_norm, self.ffn_post_norm, x, lambda h, out: self.ffn.forward(ctx, h, out))


register_part("arrangement", "sandwich_norm",
              lambda kind, *, layer_spec, hidden_size: SandwichNormBlock(layer_spec, hidden_size=hidden_size), replace=True)
register_part("arrangement", "pre_norm", lambda kind, *, layer_spec, hidden_size: PreNormBlock(layer_spec, hidden_size=hidden_size),
              replace=True)


def build_block(layer_spec, *, hidden_size: int):
    """Build the layer that ``layer_spec.arrangement`` names."""
    return build_part("arrangement", layer_spec.arrangement, layer_spec=layer_spec, hidden_size=hidden_size)
