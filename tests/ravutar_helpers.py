"""Small Ravutar configurations and model folders for the tests. Tensor names and shapes are derived here from
the configuration, independently of the engine, so a folder written here also checks what the engine's loader
expects. Weights are drawn so that every mechanism carries weight in the logits: matrices of unit gain, biases,
convolution taps and mixing coefficients of order one, decays near one so that a state remembers far tokens."""
from __future__ import annotations

import json
import random
from pathlib import Path
from typing import Dict, List, Sequence

import numpy as np
import torch
from safetensors.torch import save_file

import plain_ravutar as plain


def left(heads, kv_heads, dim, vdim, scale=None, conv=3, q_temp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=dim ** -0.5 if scale is None else scale)
    if conv is not None:          # one tap is still a weight per channel; no key: no convolution
        m["conv"] = conv
    if q_temp is not None:
        m["q_temp"] = dict(coef=q_temp[0], every=q_temp[1])
    return m


def right(heads, dim, vdim, tau=8.0, gate_rank=10):
    return dict(heads=heads, dim=dim, vdim=vdim, tau=tau, gate_rank=gate_rank)


def parallel(l, r, left_scale=0.9, right_scale=1.2, mlp=None):
    return dict(type="parallel", mixer=dict(left=l, right=r, left_scale=left_scale, right_scale=right_scale), mlp=mlp)


def mamba(heads, vdim, state, groups, conv=4, norm_groups=1, mlp=None):
    return dict(type="mamba2", mixer=dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv,
                                          norm_groups=norm_groups), mlp=mlp)


def dense(ff):
    return dict(kind="dense", ff=ff)


def config(layers, vocab=300, width=72, eps=1e-5, logit_scale=0.7, streams=3, loop=None):
    cfg = dict(architecture="Ravutar", vocab=vocab, width=width, norm=dict(eps=eps), logit_scale=logit_scale, layers=layers)
    if streams is not None:
        cfg["streams"] = streams
    if loop is not None:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return cfg


# nothing a power of two; key and value sizes differ; grouped heads; a looped stretch; a layer without feed-forward;
# a layer without convolution and without query temperature
MIX = config([
    parallel(left(6, 2, 20, 12, scale=0.3, conv=4, q_temp=(0.4, 8)), right(3, 24, 20, tau=6.0), mlp=dense(88)),
    mamba(6, 12, 20, 3, conv=3, norm_groups=3, mlp=dense(56)),
    parallel(left(2, 1, 12, 28, conv=None), right(2, 12, 36, tau=11.0, gate_rank=7), left_scale=1.3, right_scale=0.6),
    mamba(2, 36, 28, 1, conv=5, norm_groups=1, mlp=dense(40)),
], loop=(1, 3, 2))
# sizes that reach the tensor-core products; one plain residual (no streams key); every layer runs three times
WIDE = config([
    mamba(8, 16, 32, 2, conv=4, norm_groups=4, mlp=dense(256)),
    parallel(left(4, 4, 32, 16, conv=2, q_temp=(0.25, 32)), right(4, 32, 32, tau=16.0, gate_rank=16), mlp=dense(128)),
], vocab=515, width=128, eps=1e-6, logit_scale=1.0, streams=None, loop=(0, 2, 3))
# one stream with learned coefficients
ONE = config([parallel(left(3, 3, 8, 8, q_temp=(0.5, 4)), right(1, 40, 8), mlp=dense(24)),
              mamba(3, 8, 8, 3, conv=2, norm_groups=1)], width=40, streams=1)


# keys and values of one size (64): the cache of two planes and, in bfloat16, the tensor-core attention kernels
SAME = config([parallel(left(4, 2, 64, 64, scale=0.2, conv=3, q_temp=(0.3, 16)), right(2, 32, 64, tau=9.0, gate_rank=8), mlp=dense(64)),
               parallel(left(2, 2, 64, 64, scale=0.2, conv=None), right(2, 64, 32, tau=9.0, gate_rank=8))],
              width=128, vocab=200, streams=2)


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    W = cfg["width"]
    shapes = {"embed": (cfg["vocab"], W), "head": (cfg["vocab"], W), "final.norm": (W,)}
    S = cfg.get("streams")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (W,)
        if layer["type"] == "parallel":
            a, b = m["left"], m["right"]
            nq, nk, nv = a["heads"] * a["dim"], a["kv_heads"] * a["dim"], a["kv_heads"] * a["vdim"]
            for name, n in (("q", nq), ("k", nk), ("v", nv)):
                shapes[p + f"mix.left.{name}"] = (n, W)
                shapes[p + f"mix.left.{name}.b"] = (n,)
                if "conv" in a:
                    shapes[p + f"mix.left.{name}.conv"] = (n, a["conv"])
            shapes[p + "mix.left.o"] = (W, a["heads"] * a["vdim"])
            shapes[p + "mix.left.o.b"] = (W,)
            rk, rv = b["heads"] * b["dim"], b["heads"] * b["vdim"]
            shapes.update({p + "mix.right.q": (rk, W), p + "mix.right.k": (rk, W), p + "mix.right.v": (rv, W),
                           p + "mix.right.g": (rv, W), p + "mix.right.o": (W, rv), p + "mix.right.norm": (b["vdim"],),
                           p + "mix.right.a1": (b["gate_rank"], W), p + "mix.right.a2": (rk, b["gate_rank"]),
                           p + "mix.right.a2.b": (rk,)})
        else:
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            shapes.update({p + "mix.in": (2 * inner + 2 * gn + m["heads"], W), p + "mix.conv": (inner + 2 * gn, m["conv"]),
                           p + "mix.conv.b": (inner + 2 * gn,), p + "mix.dt_bias": (m["heads"],),
                           p + "mix.A_log": (m["heads"],), p + "mix.D": (m["heads"],), p + "mix.norm": (inner,),
                           p + "mix.o": (W, inner)})
        subs = ["hc1"]
        f = layer.get("mlp")
        if f is not None:
            shapes.update({p + "norm2": (W,), p + "mlp.up": (f["ff"], W), p + "mlp.up.b": (f["ff"],),
                           p + "mlp.down": (W, f["ff"]), p + "mlp.down.b": (W,)})
            subs.append("hc2")
        if S is not None:
            for q in subs:
                shapes.update({p + f"{q}.in": (S,), p + f"{q}.out": (S,), p + f"{q}.mix": (S, S)})
    return shapes


def draw_tensors(cfg: dict, seed: int, dtype=torch.float32) -> Dict[str, torch.Tensor]:
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        t = torch.randn(shape, generator=gen, dtype=torch.float32)
        leaf = name.split(".", 1)[1] if name.startswith("l") else name
        if leaf in ("norm1", "norm2", "mix.norm", "mix.right.norm", "mix.D") or name == "final.norm":
            t = 1.0 + 0.2 * t
        elif leaf.endswith(".conv"):
            t = 0.6 * t
        elif leaf == "mix.right.a2.b":
            t = 2.0 + t                                  # decays near one: the state remembers far tokens
        elif leaf == "mix.A_log":
            t = -2.0 + 0.7 * t
        elif leaf.endswith(".b") or leaf == "mix.dt_bias":
            t = 0.5 * t
        elif leaf.endswith(".in") and leaf.startswith("hc") or leaf.endswith(".out"):
            t = 1.0 + 0.3 * t
        elif leaf.endswith(".mix"):
            t = torch.eye(shape[0]) + 0.3 * t
        elif name == "embed":
            t = 0.5 * t
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
