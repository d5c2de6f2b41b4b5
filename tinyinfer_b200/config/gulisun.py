"""Typed configuration of the Gulisun decoder, read from the keys of its own config.json.

config.json: ``architecture`` (the name), ``vocab``, ``width``, ``embedding.scale``, ``norm.eps`` and ``layers``,
a list whose entries give ``type`` (which mixer), ``mixer`` (its sizes) and ``mlp`` (its feed-forward, or null).
Mixer types: ``latent_attention`` (softmax with a per-head sink) and ``latent_attention_2`` (ordinary softmax),
both with keys ``heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot.{base,dims}`` and optionally ``kv_from``
(the layer whose cached rows this one reads instead of making its own); ``rglru`` with ``width, blocks, conv``.
Feed-forward: ``kind`` "moe" with ``router.{experts,top}``, ``expert.ff`` and optionally ``shared.ff``.
Every size and constant comes from there; tensors are named ``embed``, ``final.norm`` and
``l<i>.{norm1,norm2,mix.*,mlp.*}``. The output head is the embedding table itself.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import List, Optional

from .specs import (ExecStep, ExpertsSpec, GatedRecurrenceSpec, LatentAttentionSpec, LayerSpec, ModelSpec, NormSpec,
                    PositionSpec, TensorNames)

NAME = "Gulisun"
_LATENT_TYPES = {"latent_attention": True, "latent_attention_2": False}      # type -> has a sink
MAX_POSITIONS = 1 << 20         # the design sets no limit; the engine's tables need one


@dataclass
class GulisunConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: List[dict]
    eos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None
    architectures: List[str] = field(default_factory=lambda: [NAME])

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, data: dict) -> "GulisunConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm", "embedding") if k not in data]
        if missing:
            raise ValueError(f"config.json lacks required keys: {missing}")
        cfg = cls(vocab=int(data["vocab"]), width=int(data["width"]),
                  embedding_scale=float(data["embedding"]["scale"]), norm_eps=float(data["norm"]["eps"]),
                  layers=copy.deepcopy(list(data["layers"])), eos_token_id=data.get("eos_token_id"),
                  torch_dtype=data.get("torch_dtype", data.get("dtype")))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": NAME, "embedding": {"scale": self.embedding_scale}, "layers": copy.deepcopy(self.layers),
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    # ------------------------------------------------------------------ checks
    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ValueError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            kind, m = layer.get("type"), layer.get("mixer")
            if not isinstance(m, dict):
                raise ValueError(f"layer {i} has no mixer sizes")
            if kind in _LATENT_TYPES:
                for key in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot"):
                    if key not in m:
                        raise ValueError(f"layer {i} ({kind}) lacks mixer.{key}")
                if int(m["rot"]["dims"]) % 2 or int(m["rot"]["dims"]) > int(m["rot_dim"]):
                    raise ValueError(f"layer {i}: rot.dims must be even and at most rot_dim")
                src = m.get("kv_from")
                if src is not None:
                    if (not 0 <= int(src) < i or self.layers[int(src)].get("type") not in _LATENT_TYPES
                            or self.layers[int(src)]["mixer"].get("kv_from") is not None):
                        raise ValueError(f"layer {i}: kv_from must name an earlier latent-attention layer that has "
                                         "a key/value down projection of its own")
                    other = self.layers[int(src)]["mixer"]
                    if (other["kv_rank"], other["rot_dim"], other["rot"]) != (m["kv_rank"], m["rot_dim"], m["rot"]):
                        raise ValueError(f"layer {i}: kv_rank, rot_dim and rot must equal those of layer {src}")
            elif kind == "rglru":
                for key in ("width", "blocks", "conv"):
                    if key not in m:
                        raise ValueError(f"layer {i} (rglru) lacks mixer.{key}")
                if int(m["width"]) % int(m["blocks"]):
                    raise ValueError(f"layer {i}: width must be a multiple of blocks")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            f = layer.get("mlp")
            if f is not None:
                if f.get("kind") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")
                if int(f["router"]["top"]) > int(f["router"]["experts"]):
                    raise ValueError(f"layer {i}: top exceeds the number of experts")

    # ------------------------------------------------------------------ layers
    def model_spec(self) -> ModelSpec:
        eps, width = float(self.norm_eps), self.width
        norm = NormSpec(width, eps, tensor="")
        layers, execution, entry_of = [], [], {}
        next_entry = 0
        for i, layer in enumerate(self.layers):
            kind, m, f = layer["type"], layer["mixer"], layer.get("mlp")
            if kind in _LATENT_TYPES:
                src = m.get("kv_from")
                mixer = LatentAttentionSpec(
                    hidden_size=width, num_heads=int(m["heads"]), head_dim=int(m["dim"]), rot_dim=int(m["rot_dim"]),
                    v_dim=int(m["vdim"]), q_rank=int(m["q_rank"]), kv_rank=int(m["kv_rank"]), scale=float(m["scale"]),
                    position=PositionSpec(kind="rope", theta=float(m["rot"]["base"]), rotary_dim=int(m["rot"]["dims"]),
                                          exact_frequencies=True),
                    norm_eps=eps, sink=_LATENT_TYPES[kind], shares_cache=src is not None)
            else:
                src = None
                mixer = GatedRecurrenceSpec(hidden_size=width, width=int(m["width"]), blocks=int(m["blocks"]),
                                            conv_taps=int(m["conv"]))
            if src is None:
                entry_of[i] = next_entry
                next_entry += 1
                execution.append(ExecStep(layer=i, cache=entry_of[i], writes_cache=True))
            else:
                execution.append(ExecStep(layer=i, cache=entry_of[int(src)], writes_cache=False))
            ffn = None
            if f is not None:
                shared = f.get("shared")
                ffn = ExpertsSpec(hidden_size=width, num_experts=int(f["router"]["experts"]), top=int(f["router"]["top"]),
                                  expert_size=int(f["expert"]["ff"]), shared_size=int(shared["ff"]) if shared else 0)
            layers.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                    feed_forward_norm=norm if ffn is not None else None, arrangement="output_norm"))
        names = TensorNames(embedding="embed", layer="l{i}.", mixer="mix.", feed_forward="mlp.", mixer_norm="norm1",
                            feed_forward_norm="norm2", final_norm="final.norm", head="")
        return ModelSpec(architecture=NAME, vocab_size=self.vocab, hidden_size=width, layers=tuple(layers),
                         execution=tuple(execution), final_norm=norm, tie_embeddings=True,
                         max_positions=MAX_POSITIONS, names=names)
