"""A plain, slow statement of the Ravutar decoder in PyTorch on the CPU: one function per mechanism,
written from the design's equations, sharing no code with the engine. The tests compare the engine's
kernels, cache, state slots and step function with it.

Everything is computed in one dtype (float64 by default) from tensors held in a dict under their
checkpoint names; a whole sequence is run at once, token by token where the design has a recurrence,
and nothing is cached, so whatever the engine does with pages, slots, portions and batches has to
come out equal to this.

Notation: h is a sublayer's input [T, width]; weights are stored [out, in]; positions count from 0.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * weight


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def gelu_erf(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def short_conv(u: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal per-channel convolution over time. u [T, C], w [C, taps]; the last column of w meets the
    current token, the one before it the token before, and so on; before the start there are zeros."""
    T, C = u.shape
    taps = w.shape[1]
    out = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                out[t] += w[:, j] * u[src]
    if bias is not None:
        out = out + bias
    return out


def query_temperature(positions: torch.Tensor, coef: float, every: int, dtype) -> torch.Tensor:
    """The factor a query at position p is multiplied with: 1 + coef * ln(floor((p + 1) / every) + 1)."""
    steps = torch.div(positions + 1, every, rounding_mode="floor").to(dtype)
    return 1.0 + coef * torch.log(steps + 1.0)


def sink_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, sink: bool = True) -> torch.Tensor:
    """Grouped-query causal softmax attention without a rotation: biased projections, a short convolution on
    q, k and v, a query temperature that grows with the position, and a softmax whose denominator holds one
    more term exp(0) that has no value (``sink`` False leaves that term out: what a test compares with)."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = (h @ w[n].T + w[n + ".b"] for n in ("q", "k", "v"))
    if "q.conv" in w:
        q, k, v = (short_conv(u, w[n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    pos = torch.arange(T)
    qt = m.get("q_temp")
    if qt:
        q = q * query_temperature(pos, float(qt["coef"]), int(qt["every"]), h.dtype)[:, None]
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    per = H // G
    for head in range(H):
        g = head // per
        s = (q[:, head] @ k[:, g].T) * float(m["scale"])                     # [T, T]
        s = s.masked_fill(pos[None, :] > pos[:, None], float("-inf"))
        top = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - top)
        p = e / ((torch.exp(-top) if sink else 0.0) + e.sum(dim=-1, keepdim=True))
        out[:, head] = p @ v[:, g]
    return out.reshape(T, H * dv) @ w["o"].T + w["o.b"]


def gated_linear_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Linear attention with a decay per key channel: S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t per head,
    a = sigmoid(z)^(1/tau); every head's o is brought to unit root mean square, weighted, gated and projected."""
    T = h.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ w["q"].T * d ** -0.5).reshape(T, H, d)
    k = (h @ w["k"].T).reshape(T, H, d)
    v = (h @ w["v"].T).reshape(T, H, dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    a = torch.exp(torch.nn.functional.logsigmoid(z) / tau).reshape(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = unit_rms(o, eps) * w["norm"]
    gate = silu(h @ w["g"].T)
    return (o.reshape(T, H * dv) * gate) @ w["o"].T


def parallel_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    left = sink_attention(h, _sub(w, "left."), m["left"], sink=not m.get("test_without_sink"))
    right = gated_linear_attention(h, _sub(w, "right."), m["right"], eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


def state_space_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Selective state-space mixer with a scalar decay per head: S <- exp(-exp(A_log) dt) S + dt B x^T,
    y = S^T C + D x; B and C are shared by the heads of a group."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + w["dt_bias"], threshold=1e9)          # [T, H]
    decay = torch.exp(-torch.exp(w["A_log"]) * dt)                               # [T, H]
    per = H // G
    S = torch.zeros(H, N, P, dtype=h.dtype)
    y = torch.zeros(T, H, P, dtype=h.dtype)
    for t in range(T):
        Bh = B[t].repeat_interleave(per, dim=0)                                  # [H, N]
        Ch = C[t].repeat_interleave(per, dim=0)
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * Bh[:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, Ch) + w["D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


def dense_feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    return gelu_erf(h @ w["up"].T + w["up.b"]) @ w["down"].T + w["down.b"]


def _sub(w: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in w.items() if k.startswith(prefix)}


def run_order(config: dict) -> List[int]:
    """Layer indices in the order they run: the layers start .. stop-1 are repeated ``times`` times in a row."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens, dtype=torch.float64, return_layers: bool = False):
    """Logits [T, vocab] of one sequence run whole (and, if asked, the stream after every layer run)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = float(config["norm"]["eps"])
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    hyper = "streams" in config
    streams = [x0.clone() for _ in range(int(config["streams"]))] if hyper else [x0]
    after = []
    for i in run_order(config):
        layer = config["layers"][i]
        lw = _sub(w, f"l{i}.")
        sublayers = [("1", "norm1", lambda h: _mixer(h, layer, _sub(lw, "mix."), eps))]
        if layer.get("mlp") is not None:
            sublayers.append(("2", "norm2", lambda h: dense_feed_forward(h, _sub(lw, "mlp."))))
        for q, norm, fn in sublayers:
            if hyper:
                c_in, c_out, c_mix = lw[f"hc{q}.in"], lw[f"hc{q}.out"], lw[f"hc{q}.mix"]
                u = sum(c_in[s] * streams[s] for s in range(len(streams)))
                y = fn(rms_norm(u, lw[norm], eps))
                streams = [sum(c_mix[s, t] * streams[s] for s in range(len(streams))) + c_out[t] * y
                           for t in range(len(streams))]
            else:
                streams = [streams[0] + fn(rms_norm(streams[0], lw[norm], eps))]
        after.append(sum(streams))
    x = sum(streams)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T * float(config["logit_scale"])
    return (logits, torch.stack(after)) if return_layers else logits


def _mixer(h, layer, mw, eps):
    if layer["type"] == "parallel":
        return parallel_mixer(h, mw, layer["mixer"], eps)
    if layer["type"] == "mamba2":
        return state_space_mixer(h, mw, layer["mixer"], eps)
    raise ValueError(f"unknown layer type {layer['type']!r}")
