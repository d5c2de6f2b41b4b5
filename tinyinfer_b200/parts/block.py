"""Block arrangements. 'pre_norm' is the reference's decoder layer
(tinyinfer/models/qwen3.py:192-221): x += mixer(norm(x)); x += feed_forward(norm(x)).
The residual sums are left to the parts' last kernels where they can fuse them."""
from __future__ import annotations

from .base import Block, register_block


class PreNormBlock(Block):
    def forward(self, x, step, cache):
        return self.forward_linked(x, None, None, step, cache)[0]

    def forward_linked(self, x, link, next_norm, step, cache):
        # each part gets its input before the norm, with the norm and with the norm that comes after it:
        # parts whose products can share a norm between them do so (a decode step saves the norm kernels)
        x, link = self.mixer.forward_prenorm(x, self.mixer_norm, link, self.feed_forward_norm, step, cache)
        x, link = self.feed_forward.forward_prenorm(x, self.feed_forward_norm, link, next_norm, step)
        return x, link


class OutputNormBlock(Block):
    """x <- x + norm1(mixer(x)); x <- x + norm2(feed_forward(x)): both sublayers read x itself and the norm sits on
    a sublayer's OUTPUT. The stream is a pair (x32, copy): the residual sums are float32, ``copy`` is their
    rounding in the compute dtype, which the matrix products read (the same tensor in a float32 model).
    A block may have no feed-forward."""

    def forward(self, x, step, cache):
        return self.forward_linked(x, None, None, step, cache)[0]

    def forward_linked(self, x, link, next_norm, step, cache):
        from .. import ops
        x32, copy = x
        rms = self.mixer_norm.as_rms()
        if rms is None:
            raise ValueError("the output-norm arrangement needs RMSNorms")
        mixed = self.mixer.forward(copy, step, cache)
        x32, copy = ops.norm_add(x32, mixed, rms[0], rms[1], self.mixer.dtype)
        if self.feed_forward is not None:
            if hasattr(self.feed_forward, "forward_stream"):
                x32, copy = self.feed_forward.forward_stream(x32, copy, self.feed_forward_norm, step)
            else:
                rms = self.feed_forward_norm.as_rms()
                x32, copy = ops.norm_add(x32, self.feed_forward.forward(copy, step), rms[0], rms[1], self.mixer.dtype)
        return (x32, copy), None


register_block("pre_norm", PreNormBlock)
register_block("output_norm", OutputNormBlock)
