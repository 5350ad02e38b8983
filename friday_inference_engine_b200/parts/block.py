"""Pre-norm residual block: x = x + mixer(norm1(x)); x = x + feed_forward(norm2(x)).

The two sums happen inside the mixer's and the feed-forward's last product (each gets
the residual stream and returns it with its own output added), as in the reference
(transformer.cpp:997-1074).  Which mixer, feed-forward and norms a block has is decided
by its specification, layer by layer.
"""
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

    def forward(self, x, ctx, cache):
        x = self.mixer.forward(self.norm1.forward(x), x, ctx, cache)
        return self.feed_forward.forward(self.norm2.forward(x), x, ctx)
