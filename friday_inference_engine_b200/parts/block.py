"""Pre-norm residual block: x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x)).

The two sums happen inside the mixer's and the feed-forward's last product (each gets
the residual stream and returns it with its own output added), as in the reference
(transformer.cpp:997-1074).  Which mixer, feed-forward and norms a block has is decided
by its specification, layer by layer.
"""
from .. import ops
from .base import Part, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Part):
    category = "block"

    def __init__(self, env, norm1, mixer, norm2, feed_forward):
        super().__init__(env)
        self.norm1 = self.adopt(norm1.prefix, build_part("norm", norm1, env))
        self.mixer = self.adopt(mixer.prefix, build_part("mixer", mixer, env))
        self.norm2 = self.adopt(norm2.prefix, build_part("norm", norm2, env))
        self.feed_forward = self.adopt(feed_forward.prefix, build_part("feed_forward", feed_forward, env))

    def cache_request(self):
        return self.mixer.cache_request()

    chains_norm = True

    @property
    def first_norm(self):
        return self.norm1

    @staticmethod
    def _call(part, norm, h, x, *rest):
        """part(h, x, ...) and `norm` of the result: by the part itself if it chains norms, else here."""
        if part.chains_norm:
            x, normed = part.forward(h, x, *rest, then=norm)
        else:
            x, normed = part.forward(ops.materialize(h), x, *rest), None
        if normed is None and norm is not None:
            normed = norm.forward(x)
        return x, normed

    def forward(self, x, ctx, cache, normed=None, then=None):
        """normed: norm1(x) if the caller has it already; then: the norm that follows this block, if any.
        Returns x and then(x) (None without `then`)."""
        h = normed if normed is not None else self.norm1.forward(x)
        x, h = self._call(self.mixer, self.norm2, h, x, ctx, cache)
        return self._call(self.feed_forward, then, h, x, ctx)
