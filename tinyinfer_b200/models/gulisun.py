"""Gulisun: a decoder whose layers mix attention over a cached latent (with or without a softmax sink, some
layers reading an earlier layer's cache), gated linear recurrences and mixtures of experts, each sublayer's norm
on its OUTPUT, around a float32 residual stream. The blocks, cache and step function are the generic decoder's;
this class only has the frame: an embedding that is scaled into the float32 stream, and the final norm read
from it. The head is the embedding table (without its scale)."""
from __future__ import annotations

from .. import ops
from ..config.gulisun import NAME, GulisunConfig
from ..config.registry import register_architecture
from .decoder import DecoderModel


class GulisunForCausalLM(DecoderModel):
    def __init__(self, config: GulisunConfig, dtype, device):
        super().__init__(config.model_spec(), dtype, device)
        self.config = config

    def embed(self, step):
        """(x32, copy): the float32 stream and its rounding in the compute dtype."""
        return ops.embedding_scaled(step.token_ids, self.embedding, self.config.embedding_scale)

    def logits(self, x, step):
        rms = self.final_norm.as_rms()
        h = ops.rmsnorm_rows32(x[0], rms[0], rms[1], step.logit_rows, self.dtype)
        return ops.linear(h, self.head, out_float32=True)


def _layers(pattern: str, latent: dict, recurrent: dict, mlp: dict):
    """config.json layers from a pattern: 's' attention with a sink, 'k' the same reading the cache of the last
    's' before it, 'p' attention with the plain softmax, 'r' a recurrent layer."""
    out = []
    for kind in pattern:
        if kind == "r":
            out.append(dict(type="rglru", mixer=dict(recurrent), mlp=mlp))
        elif kind == "s":
            out.append(dict(type="latent_attention", mixer=dict(latent), mlp=mlp))
        elif kind == "k":
            src = max(i for i, l in enumerate(out) if l["type"] == "latent_attention" and "kv_from" not in l["mixer"])
            out.append(dict(type="latent_attention", mixer=dict(latent, kv_from=src), mlp=mlp))
        else:
            out.append(dict(type="latent_attention_2", mixer=dict(latent), mlp=mlp))
    return out


# Sizes worth running with random weights (config.json keys): a toy, and two with the layer sizes of models of one and
# of a few billion parameters (the larger: width 2048, 16 heads over a latent of 512 + 64, 64 experts of 1408 of which 6 run),
# eight layers each: a benchmark runs as many layers as it lists.
PRESETS = {
    "gulisun-tiny": dict(
        vocab=256, width=64, embedding=dict(scale=8.0), norm=dict(eps=1e-5),
        layers=_layers("srkp",
                       dict(heads=2, dim=16, rot_dim=8, vdim=16, q_rank=24, kv_rank=32, scale=24 ** -0.5,
                            rot=dict(base=10000.0, dims=8)),
                       dict(width=64, blocks=2, conv=4),
                       dict(kind="moe", router=dict(experts=4, top=2), expert=dict(ff=32), shared=dict(ff=48)))),
    "gulisun-1b": dict(
        vocab=102400, width=1024, embedding=dict(scale=1.0), norm=dict(eps=1e-6),
        layers=_layers("srkp" * 2,
                       dict(heads=8, dim=64, rot_dim=32, vdim=64, q_rank=768, kv_rank=256, scale=96 ** -0.5,
                            rot=dict(base=10000.0, dims=32)),
                       dict(width=1280, blocks=5, conv=4),
                       dict(kind="moe", router=dict(experts=32, top=4), expert=dict(ff=704), shared=dict(ff=1408)))),
    "gulisun-2b": dict(
        vocab=102400, width=2048, embedding=dict(scale=1.0), norm=dict(eps=1e-6),
        layers=_layers("srkp" * 2,
                       dict(heads=16, dim=128, rot_dim=64, vdim=128, q_rank=1536, kv_rank=512, scale=192 ** -0.5,
                            rot=dict(base=10000.0, dims=64)),
                       dict(width=2560, blocks=10, conv=4),
                       dict(kind="moe", router=dict(experts=64, top=6), expert=dict(ff=1408), shared=dict(ff=2816)))),
}

register_architecture(NAME, GulisunConfig, GulisunForCausalLM, presets=PRESETS)
