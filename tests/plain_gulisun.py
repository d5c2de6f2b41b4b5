"""A plain, slow statement of the Gulisun decoder in PyTorch on the CPU: one function per mechanism,
written from the design's equations, sharing no code with the engine. The tests compare the engine's
kernels, cache and step function with it.

Everything is computed in one dtype (float64 by default) from tensors held in a dict under their
checkpoint names; a whole sequence is run at once and nothing is cached, so whatever the engine does
with pages, slots, portions and batches has to come out equal to this.

Notation: h is a sublayer's input [T, width]; a layer is x <- x + norm1(mixer(x)),
x <- x + norm2(ff(x)) with both sublayers reading x itself.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_half_split(v: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """Turns the first ``dims`` features of the last axis: feature i pairs with i + dims/2,
    (u, v) -> (u cos a - v sin a, v cos a + u sin a), a = position * base^(-2i/dims)."""
    half = dims // 2
    i = torch.arange(half, dtype=torch.float64)
    freq = (base ** (-2.0 * i / dims)).to(v.dtype)
    angle = positions.to(v.dtype)[:, None] * freq[None, :]                 # [T, half]
    shape = [angle.shape[0]] + [1] * (v.dim() - 2) + [half]
    cos, sin = torch.cos(angle).reshape(shape), torch.sin(angle).reshape(shape)
    a, b, rest = v[..., :half], v[..., half:dims], v[..., dims:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, rest], dim=-1)


def latent_keys(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, positions: torch.Tensor):
    """What a latent-attention layer leaves for its keys: the normed latent c [T, kv_rank] and the one
    rotated key part [T, rot_dim] that all heads share."""
    rank, rot = m["kv_rank"], m["rot_dim"]
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :rank], w["dkv.norm"], eps)
    k_rot = rotate_half_split(down[:, rank:rank + rot], positions, m["rot"]["base"], m["rot"]["dims"])
    return c, k_rot


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float,
                     positions: torch.Tensor, c: torch.Tensor, k_rot: torch.Tensor, sink: bool) -> torch.Tensor:
    """Causal attention with queries through a latent and keys/values raised from the latent ``c``;
    ``sink``: every head's softmax denominator also holds exp(sink_h), a term with no key and no value."""
    H, d, rot, dv = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    T = h.shape[0]
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(T, H, d + rot)
    q_plain = q[..., :d]
    q_rot = rotate_half_split(q[..., d:], positions, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w["uk"].T).reshape(T, H, d)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain)
              + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    causal = torch.ones(T, T, dtype=torch.bool).tril()
    scores = scores.masked_fill(~causal, float("-inf"))
    if sink:
        top = torch.maximum(scores.max(dim=-1, keepdim=True).values, w["sink"].to(h.dtype)[:, None, None])
        e = torch.exp(scores - top)
        p = e / (e.sum(dim=-1, keepdim=True) + torch.exp(w["sink"].to(h.dtype)[:, None, None] - top))
    else:
        p = torch.softmax(scores, dim=-1)
    out = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    return out @ w["o"].T


def rglru(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict) -> torch.Tensor:
    """Recurrent block: a gelu branch y, and a branch through a causal per-channel convolution into
    a gated diagonal recurrence S_t = a_t S_(t-1) + sqrt(1 - a_t^2) i_t u_t from S = 0; out = W_o (S * y)."""
    T = h.shape[0]
    width, blocks, taps = m["width"], m["blocks"], m["conv"]
    y = gelu_tanh(h @ w["y"].T + w["y.b"])
    xb = h @ w["x"].T + w["x.b"]
    padded = torch.cat([torch.zeros(taps - 1, width, dtype=h.dtype), xb], dim=0)
    u = torch.zeros(T, width, dtype=h.dtype) + w["conv.b"]
    for k in range(taps):                                   # column taps-1 multiplies the current token
        u = u + padded[k:k + T] * w["conv"][:, k]
    bw = width // blocks
    ub = u.reshape(T, blocks, bw)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w["ra"]) + w["ra.b"]).reshape(T, width)
    g = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w["ri"]) + w["ri.b"]).reshape(T, width)
    log_a = -8.0 * r * torch.nn.functional.softplus(w["lam"])
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * g * u
    state = torch.zeros(width, dtype=h.dtype)
    out = []
    for t in range(T):
        state = a[t] * state + drive[t]
        out.append(state)
    return (torch.stack(out) * y) @ w["o"].T


def relu_squared_expert(h: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (torch.relu(h @ up.T) ** 2) @ down.T


def mixture_of_experts(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict) -> torch.Tensor:
    """Each token runs its ``top`` best experts by softmax score, weighted by those scores over their
    sum; a shared expert runs for every token."""
    experts, top = f["router"]["experts"], f["router"]["top"]
    scores = torch.softmax(h @ w["router"].T, dim=-1)
    best, chosen = torch.topk(scores, top, dim=-1)
    weight = best / (best.sum(dim=-1, keepdim=True) + 1e-20)
    out = torch.zeros_like(h)
    for e in range(experts):
        for k in range(top):
            rows = (chosen[:, k] == e).nonzero().flatten()
            if rows.numel():
                out[rows] += weight[rows, k, None] * relu_squared_expert(h[rows], w[f"e{e}.up"], w[f"e{e}.down"])
    if f.get("shared") is not None:
        out = out + relu_squared_expert(h, w["shared.up"], w["shared.down"])
    return out


def _part(tensors: Dict[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: (v.to(dtype) if v.is_floating_point() else v)
            for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: Dict[str, torch.Tensor], token_ids: List[int], dtype=torch.float64,
            layer_outputs: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence. ``layer_outputs``: a list that receives the residual
    stream after every layer."""
    eps = config["norm"]["eps"]
    T = len(token_ids)
    positions = torch.arange(T)
    embed = tensors["embed"].to(dtype)
    x = embed[torch.tensor(token_ids)] * config["embedding"]["scale"]
    kept = {}                                                # layer -> (c, k_rot) of latent layers
    for i, layer in enumerate(config["layers"]):
        m = layer["mixer"]
        w = _part(tensors, f"l{i}.mix.", dtype)
        if layer["type"] in ("latent_attention", "latent_attention_2"):
            src = m.get("kv_from")
            if src is None:
                kept[i] = latent_keys(x, w, m, eps, positions)
                c, k_rot = kept[i]
            else:
                c, k_rot = kept[src]
            mixed = latent_attention(x, w, m, eps, positions, c, k_rot, sink=layer["type"] == "latent_attention")
        elif layer["type"] == "rglru":
            mixed = rglru(x, w, m)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(mixed, tensors[f"l{i}.norm1"].to(dtype), eps)
        if layer.get("mlp") is not None:
            ff = mixture_of_experts(x, _part(tensors, f"l{i}.mlp.", dtype), layer["mlp"])
            x = x + rms_norm(ff, tensors[f"l{i}.norm2"].to(dtype), eps)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    x = rms_norm(x, tensors["final.norm"].to(dtype), eps)
    return x @ embed.T
