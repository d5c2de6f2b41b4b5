"""Small Gulisun configurations and model folders for the tests. Tensor names and shapes are derived here from
the configuration, independently of the engine, so a folder written here also checks what the engine's loader
expects. Weights are drawn so that every mechanism carries weight in the logits: matrices of unit gain, sinks
and biases of order one, a router whose scores are well apart."""
from __future__ import annotations

import json
import random
from pathlib import Path
from typing import Dict, List, Sequence

import numpy as np
import torch
from safetensors.torch import save_file

import plain_gulisun as plain


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale=None, base=10000.0, **extra):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank,
             scale=(dim + rot_dim) ** -0.5 if scale is None else scale, rot=dict(base=base, dims=rot_dim))
    m.update(extra)
    return m


def moe(experts, top, ff, shared=None):
    f = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff))
    if shared:
        f["shared"] = dict(ff=shared)
    return f


def config(layers, vocab=300, width=72, scale=3.0, eps=1e-5):
    return dict(architecture="Gulisun", vocab=vocab, width=width, embedding=dict(scale=scale), norm=dict(eps=eps),
                layers=layers)


LAT_A = latent(3, 20, 12, 24, 28, 40)                      # nothing a power of two, K of the query up projection not / 8
LAT_B = latent(5, 8, 16, 8, 48, 64, base=500.0)
MOE_A = moe(5, 3, 24, shared=40)
MOE_B = moe(7, 1, 16)                                      # one expert a token, no shared expert

# every mixer, a layer that reads another's cache, differing sizes from layer to layer, a layer without feed-forward
MIX = config([
    dict(type="latent_attention", mixer=LAT_A, mlp=MOE_A),
    dict(type="rglru", mixer=dict(width=96, blocks=3, conv=3), mlp=MOE_B),
    dict(type="latent_attention_2", mixer=LAT_B, mlp=MOE_A),
    dict(type="latent_attention", mixer=dict(LAT_A, kv_from=0, heads=2, q_rank=16), mlp=None),
    dict(type="rglru", mixer=dict(width=40, blocks=1, conv=5), mlp=MOE_A),
])
# a recurrent layer first, a reader of a plain-softmax layer's rows, sizes that reach the tensor-core products
WIDE = config([
    dict(type="rglru", mixer=dict(width=128, blocks=4, conv=4), mlp=moe(8, 2, 64, shared=64)),
    dict(type="latent_attention_2", mixer=latent(4, 32, 16, 16, 64, 96), mlp=moe(8, 2, 64, shared=64)),
    dict(type="latent_attention", mixer=latent(8, 16, 16, 32, 32, 96, kv_from=1), mlp=moe(4, 4, 32)),
    dict(type="latent_attention", mixer=latent(4, 32, 32, 32, 64, 160, base=1e6), mlp=None),
], vocab=515, width=128, scale=1.0, eps=1e-6)


def single(kind, mlp=None, **kw):
    """One mechanism alone: a model of one layer (two for the reader of another layer's cache)."""
    if kind == "sink":
        return config([dict(type="latent_attention", mixer=LAT_A, mlp=mlp)], **kw)
    if kind == "plain":
        return config([dict(type="latent_attention_2", mixer=LAT_B, mlp=mlp)], **kw)
    if kind == "reader":
        return config([dict(type="latent_attention", mixer=LAT_A, mlp=None),
                       dict(type="latent_attention", mixer=dict(LAT_A, kv_from=0), mlp=mlp)], **kw)
    if kind == "recurrent":
        return config([dict(type="rglru", mixer=dict(width=96, blocks=3, conv=4), mlp=mlp)], **kw)
    raise ValueError(kind)


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W = cfg["width"]
    shapes = {"embed": (cfg["vocab"], W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (W,)
        if layer["type"].startswith("latent_attention"):
            H = m["heads"]
            shapes[p + "mix.dq"] = (m["q_rank"], W)
            shapes[p + "mix.dq.norm"] = (m["q_rank"],)
            shapes[p + "mix.uq"] = (H * (m["dim"] + m["rot_dim"]), m["q_rank"])
            if "kv_from" not in m:
                shapes[p + "mix.dkv"] = (m["kv_rank"] + m["rot_dim"], W)
                shapes[p + "mix.dkv.norm"] = (m["kv_rank"],)
            shapes[p + "mix.uk"] = (H * m["dim"], m["kv_rank"])
            shapes[p + "mix.uv"] = (H * m["vdim"], m["kv_rank"])
            if layer["type"] == "latent_attention":
                shapes[p + "mix.sink"] = (H,)
            shapes[p + "mix.o"] = (W, H * m["vdim"])
        else:
            R, B = m["width"], m["blocks"]
            shapes.update({p + "mix.y": (R, W), p + "mix.y.b": (R,), p + "mix.x": (R, W), p + "mix.x.b": (R,),
                           p + "mix.conv": (R, m["conv"]), p + "mix.conv.b": (R,),
                           p + "mix.ra": (B, R // B, R // B), p + "mix.ra.b": (B, R // B),
                           p + "mix.ri": (B, R // B, R // B), p + "mix.ri.b": (B, R // B),
                           p + "mix.lam": (R,), p + "mix.o": (W, R)})
        f = layer.get("mlp")
        if f is not None:
            shapes[p + "norm2"] = (W,)
            for e in range(f["router"]["experts"]):
                shapes[p + f"mlp.e{e}.up"] = (f["expert"]["ff"], W)
                shapes[p + f"mlp.e{e}.down"] = (W, f["expert"]["ff"])
            shapes[p + "mlp.router"] = (f["router"]["experts"], W)
            if f.get("shared"):
                shapes[p + "mlp.shared.up"] = (f["shared"]["ff"], W)
                shapes[p + "mlp.shared.down"] = (W, f["shared"]["ff"])
    return shapes


def draw_tensors(cfg: dict, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        t = torch.randn(shape, generator=gen, dtype=torch.float32)
        leaf = name.split(".", 1)[1] if name.startswith("l") else name
        if leaf in ("norm1", "norm2", "mix.dq.norm", "mix.dkv.norm") or name == "final.norm":
            t = 1.0 + 0.2 * t
        elif leaf == "mix.sink":
            t = 1.5 * t                                  # of the order of the scores: leaving it out shows
        elif leaf in ("mix.y.b", "mix.x.b", "mix.conv.b", "mix.ra.b", "mix.ri.b", "mix.lam"):
            t = 0.7 * t
        elif leaf == "mix.conv":
            t = 0.6 * t
        elif leaf == "mlp.router":
            t = 2.0 * t / shape[-1] ** 0.5               # scores well apart: no choice hangs on a rounding
        elif name == "embed":
            t = 0.3 * t
        else:
            t = t / shape[-1] ** 0.5                     # unit gain
        out[name] = t.to(dtype).contiguous()
    return out


def write_folder(folder, cfg: dict, seed: int, dtype: str = "float32", edit=None) -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    tensors = draw_tensors(cfg, seed, torch.float32 if dtype == "float32" else torch.bfloat16)
    if edit is not None:
        edit(tensors)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file(tensors, str(folder / "model.safetensors"))
    return folder


def read_folder(folder):
    from safetensors.torch import load_file
    cfg = json.loads((Path(folder) / "config.json").read_text())
    return cfg, {k: (v.to(torch.float64) if v.is_floating_point() else v)
                 for k, v in load_file(str(Path(folder) / "model.safetensors")).items()}


def random_requests(cfg: dict, lengths: Sequence[int], seed: int) -> Dict[str, List[int]]:
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg["vocab"]) for _ in range(n)] for i, n in enumerate(lengths)}


def plain_logits(folder, requests, edit=None) -> Dict[str, np.ndarray]:
    cfg, w = read_folder(folder)
    if edit is not None:
        edit(cfg, w)
    return {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in requests.items()}
