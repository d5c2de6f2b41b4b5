"""Typed configuration of the Ravutar decoder, read from the keys of its own config.json.

config.json: ``architecture`` (the name), ``vocab``, ``width``, ``norm.eps``, ``logit_scale``, optionally
``streams`` (the residual is that many float32 streams with learned mixing, "hyper-connections"; without the key
there is one plain residual) and ``loop`` = {start, stop, times} (layers start .. stop-1 run ``times`` times in a
row with the same weights, every pass with a cache and state of its own), and ``layers``, a list whose entries
give ``type`` (which mixer), ``mixer`` (its sizes) and ``mlp`` (its feed-forward, or null).
Mixer types: ``parallel``: an attention branch ``left`` (``heads, kv_heads, dim, vdim, scale, conv`` and optionally
``q_temp.{coef, every}``) beside a gated-linear-attention branch ``right`` (``heads, dim, vdim, tau``; the inner
size of its decay projections is the checkpoint's, or ``gate_rank`` for random weights), summed with
``left_scale`` and ``right_scale``; ``mamba2``: ``heads, vdim, state, groups, conv, norm_groups``.
Feed-forward: ``kind`` "dense" with ``ff``. Every size and constant comes from there; tensors are named ``embed``,
``head``, ``final.norm`` and ``l<i>.{norm1, norm2, mix.*, mlp.*, hc1.*, hc2.*}``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import List, Optional

from .specs import (ConvAttentionSpec, DenseMLPSpec, ExecStep, GatedLinearAttentionSpec, LayerSpec, ModelSpec, NormSpec,
                    ParallelMixerSpec, StateSpaceSpec, TensorNames)

NAME = "Ravutar"
MAX_POSITIONS = 1 << 20         # the design sets no limit; the engine's tables need one
SINK_LOGIT = 0.0                # the design's softmax adds exp(0) = 1 to its denominator


@dataclass
class RavutarConfig:
    vocab: int
    width: int
    norm_eps: float
    logit_scale: float
    layers: List[dict]
    streams: Optional[int] = None          # None: one plain residual
    loop: Optional[dict] = None
    eos_token_id: Optional[int] = None
    torch_dtype: Optional[str] = None
    architectures: List[str] = field(default_factory=lambda: [NAME])

    # ------------------------------------------------------------------ parsing
    @classmethod
    def from_dict(cls, data: dict) -> "RavutarConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if k not in data]
        if missing:
            raise ValueError(f"config.json lacks required keys: {missing}")
        loop = data.get("loop")
        cfg = cls(vocab=int(data["vocab"]), width=int(data["width"]), norm_eps=float(data["norm"]["eps"]),
                  logit_scale=float(data.get("logit_scale", 1.0)), layers=copy.deepcopy(list(data["layers"])),
                  streams=int(data["streams"]) if data.get("streams") is not None else None,
                  loop=dict(loop) if loop else None, eos_token_id=data.get("eos_token_id"),
                  torch_dtype=data.get("torch_dtype", data.get("dtype")))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": NAME, "layers": copy.deepcopy(self.layers), "logit_scale": self.logit_scale,
             "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.loop:
            d["loop"] = dict(self.loop)
        if self.eos_token_id is not None:
            d["eos_token_id"] = self.eos_token_id
        return d

    # ------------------------------------------------------------------ checks
    def validate(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ValueError("vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ValueError("norm.eps must be positive")
        if self.streams is not None and not 1 <= self.streams <= 8:
            raise ValueError("streams must be 1..8")
        if self.loop:
            for key in ("start", "stop", "times"):
                if key not in self.loop:
                    raise ValueError(f"loop lacks {key}")
            start, stop, times = (int(self.loop[k]) for k in ("start", "stop", "times"))
            if not (0 <= start <= stop <= len(self.layers)) or times < 1:
                raise ValueError("loop: need 0 <= start <= stop <= number of layers and times >= 1")
        for i, layer in enumerate(self.layers):
            kind, m = layer.get("type"), layer.get("mixer")
            if not isinstance(m, dict):
                raise ValueError(f"layer {i} has no mixer sizes")
            if kind == "parallel":
                for side, keys in (("left", ("heads", "kv_heads", "dim", "vdim", "scale")),
                                   ("right", ("heads", "dim", "vdim", "tau"))):
                    if not isinstance(m.get(side), dict):
                        raise ValueError(f"layer {i} (parallel) lacks mixer.{side}")
                    for key in keys:
                        if key not in m[side]:
                            raise ValueError(f"layer {i} (parallel) lacks mixer.{side}.{key}")
                if int(m["left"]["heads"]) % int(m["left"]["kv_heads"]):
                    raise ValueError(f"layer {i}: left.heads must be a multiple of left.kv_heads")
                qt = m["left"].get("q_temp")
                if qt and (int(qt["every"]) < 1):
                    raise ValueError(f"layer {i}: q_temp.every must be at least 1")
                if not float(m["right"]["tau"]) > 0:
                    raise ValueError(f"layer {i}: right.tau must be positive")
            elif kind == "mamba2":
                for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                    if key not in m:
                        raise ValueError(f"layer {i} (mamba2) lacks mixer.{key}")
                if int(m["heads"]) % int(m["groups"]):
                    raise ValueError(f"layer {i}: heads must be a multiple of groups")
                if (int(m["heads"]) * int(m["vdim"])) % int(m["norm_groups"]):
                    raise ValueError(f"layer {i}: heads * vdim must be a multiple of norm_groups")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
            f = layer.get("mlp")
            if f is not None and f.get("kind") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {f.get('kind')!r}")

    # ------------------------------------------------------------------ layers
    def run_order(self) -> List[int]:
        """Layer indices in the order they run."""
        n = len(self.layers)
        if not self.loop:
            return list(range(n))
        start, stop, times = (int(self.loop[k]) for k in ("start", "stop", "times"))
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))

    def model_spec(self) -> ModelSpec:
        eps, width = float(self.norm_eps), self.width
        norm = NormSpec(width, eps, tensor="")
        layers = []
        for layer in self.layers:
            kind, m, f = layer["type"], layer["mixer"], layer.get("mlp")
            if kind == "parallel":
                left, right = m["left"], m["right"]
                qt = left.get("q_temp")
                attention = ConvAttentionSpec(
                    hidden_size=width, num_heads=int(left["heads"]), num_kv_heads=int(left["kv_heads"]),
                    head_dim=int(left["dim"]), v_dim=int(left["vdim"]), scale=float(left["scale"]),
                    conv_taps=int(left.get("conv", 0)),
                    query_temperature=(float(qt["coef"]), int(qt["every"])) if qt else None, sink=SINK_LOGIT, bias=True)
                linear = GatedLinearAttentionSpec(
                    hidden_size=width, num_heads=int(right["heads"]), key_dim=int(right["dim"]),
                    value_dim=int(right["vdim"]), tau=float(right["tau"]), norm_eps=eps,
                    gate_rank=int(right.get("gate_rank", 0)))
                mixer = ParallelMixerSpec(branches=(attention, linear),
                                          scales=(float(m.get("left_scale", 1.0)), float(m.get("right_scale", 1.0))),
                                          prefixes=("left.", "right."))
            else:
                mixer = StateSpaceSpec(hidden_size=width, num_heads=int(m["heads"]), head_dim=int(m["vdim"]),
                                       state_dim=int(m["state"]), groups=int(m["groups"]), conv_taps=int(m["conv"]),
                                       norm_groups=int(m["norm_groups"]), norm_eps=eps)
            ffn = DenseMLPSpec(hidden_size=width, intermediate_size=int(f["ff"])) if f is not None else None
            layers.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm,
                                    feed_forward_norm=norm if ffn is not None else None, arrangement="multi_stream",
                                    streams=self.streams or 1, learned_mixing=self.streams is not None))
        # every run of a layer has a cache entry of its own: a layer that runs twice keeps two caches and two states
        execution = tuple(ExecStep(layer=i, cache=n, writes_cache=True) for n, i in enumerate(self.run_order()))
        names = TensorNames(embedding="embed", layer="l{i}.", mixer="mix.", feed_forward="mlp.", mixer_norm="norm1",
                            feed_forward_norm="norm2", final_norm="final.norm", head="head")
        return ModelSpec(architecture=NAME, vocab_size=self.vocab, hidden_size=width, layers=tuple(layers),
                         execution=execution, final_norm=norm, tie_embeddings=False,
                         max_positions=MAX_POSITIONS, names=names)
