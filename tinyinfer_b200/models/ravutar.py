"""Ravutar: a decoder whose layers are either a softmax attention with short convolutions and a sink beside a gated
linear attention, or a selective state-space mixer, each with a dense feed-forward, around a residual of several
float32 streams with learned mixing; a stretch of layers may run several times with the same weights. The blocks,
cache and step function are the generic decoder's; this class only has the frame: the embedding copied into every
stream, and at the end the streams' sum through the final norm, the head and a constant factor on the logits."""
from __future__ import annotations

import torch

from .. import ops
from ..config.ravutar import NAME, RavutarConfig
from ..config.registry import register_architecture
from .decoder import DecoderModel


class RavutarForCausalLM(DecoderModel):
    def __init__(self, config: RavutarConfig, dtype, device):
        super().__init__(config.model_spec(), dtype, device)
        self.config = config
        self.streams = config.streams or 1
        self._ones = None

    def embed(self, step):
        """(streams float32 [S, T, width], the update still to be applied to them: none yet)."""
        return ops.streams_embed(step.token_ids, self.embedding, self.streams), None

    def logits(self, x, step):
        streams, pending = x
        if self._ones is None:
            self._ones = torch.ones(self.streams, dtype=torch.float32, device=self.device)
        rms = self.final_norm.as_rms()
        # the last sublayer's update, the sum of the streams and the final norm, for the wanted rows only
        h = ops.streams_step(streams, pending, self._ones, rms[0], rms[1], self.dtype, rows=step.logit_rows)
        return ops.scale_(ops.linear(h, self.head, out_float32=True), self.config.logit_scale)


def _layers(pattern: str, parallel: dict, mamba: dict, mlp: dict):
    """config.json layers from a pattern: 'p' a parallel layer, 'm' a state-space layer."""
    return [dict(type="parallel" if kind == "p" else "mamba2", mixer=dict(parallel if kind == "p" else mamba), mlp=mlp)
            for kind in pattern]


# Sizes worth running with random weights (config.json keys): a toy, and two with the layer sizes of models of about
# one and of a few billion parameters, eight layer runs each (a benchmark runs as many layers as it lists).
PRESETS = {
    "ravutar-tiny": dict(
        vocab=256, width=64, norm=dict(eps=1e-5), logit_scale=0.25, streams=2, loop=dict(start=1, stop=3, times=2),
        layers=_layers("pmp",
                       dict(left=dict(heads=4, kv_heads=2, dim=16, vdim=8, scale=0.25, conv=4,
                                      q_temp=dict(coef=0.3, every=16)),
                            right=dict(heads=2, dim=16, vdim=24, tau=8.0, gate_rank=8), left_scale=0.7, right_scale=1.1),
                       dict(heads=4, vdim=16, state=16, groups=2, conv=4, norm_groups=2),
                       dict(kind="dense", ff=96))),
    "ravutar-1b": dict(
        vocab=102400, width=1024, norm=dict(eps=1e-6), logit_scale=1.0, streams=2,
        layers=_layers("ppmp" * 2,
                       dict(left=dict(heads=8, kv_heads=4, dim=128, vdim=128, scale=128 ** -0.5, conv=4,
                                      q_temp=dict(coef=0.1, every=1024)),
                            right=dict(heads=8, dim=64, vdim=128, tau=16.0, gate_rank=16), left_scale=1.0, right_scale=1.0),
                       dict(heads=32, vdim=64, state=128, groups=1, conv=4, norm_groups=1),
                       dict(kind="dense", ff=4096))),
    "ravutar-2b": dict(
        vocab=102400, width=2048, norm=dict(eps=1e-6), logit_scale=1.0, streams=2,
        layers=_layers("ppmp" * 2,
                       dict(left=dict(heads=16, kv_heads=8, dim=128, vdim=128, scale=128 ** -0.5, conv=4,
                                      q_temp=dict(coef=0.1, every=1024)),
                            right=dict(heads=16, dim=64, vdim=128, tau=16.0, gate_rank=16), left_scale=1.0, right_scale=1.0),
                       dict(heads=64, vdim=64, state=128, groups=1, conv=4, norm_groups=1),
                       dict(kind="dense", ff=8192))),
}

register_architecture(NAME, RavutarConfig, RavutarForCausalLM, presets=PRESETS)
