"""Gated linear attention ("Gated Linear Attention Transformers with Hardware-Efficient Training", Yang et al.,
2024): per head a matrix state S (key_dim x value_dim) with a decay per key channel,
S <- diag(a) S + k v^T, o = S^T q, a = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau), q scaled by key_dim^-1/2.
Every head's o is divided by its root mean square and weighted (one weight of value_dim entries for all heads),
the heads side by side are multiplied by silu(W_g h) and projected.

The state is float32 and lives in the request's state slot (zero at the start); the decay's logits leave their
product as float32, and the decay, the recurrence, o and its norm are float32.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorSpec, register_mixer


class GatedLinearAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        self.w_in = self.w_a1 = self.w_a2 = self.b_a2 = self.norm_w = self.w_o = None

    def state_need(self):
        s = self.spec
        return StateNeed((s.num_heads * s.key_dim * s.value_dim,), torch.float32)

    def tensors(self):
        s = self.spec
        nk, nv = s.num_heads * s.key_dim, s.num_heads * s.value_dim
        rank = s.gate_rank if s.gate_rank > 0 else -1
        return {"q": TensorSpec((nk, s.hidden_size)), "k": TensorSpec((nk, s.hidden_size)),
                "v": TensorSpec((nv, s.hidden_size)), "g": TensorSpec((nv, s.hidden_size)),
                "o": TensorSpec((s.hidden_size, nv)),
                "norm": TensorSpec((s.value_dim,), role="vector32", init="ones_noise"),
                "a1": TensorSpec((rank, s.hidden_size)), "a2": TensorSpec((nk, rank)),
                "a2.b": TensorSpec((nk,), role="vector32")}

    def load(self, tensors):
        if tensors["a1"].shape[0] != tensors["a2"].shape[1]:
            raise ValueError("the two projections of the decay do not fit each other")
        self.w_in = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0).contiguous()
        self.w_a1, self.w_a2, self.b_a2 = tensors["a1"].contiguous(), tensors["a2"].contiguous(), tensors["a2.b"]
        self.norm_w, self.w_o = tensors["norm"], tensors["o"].contiguous()

    def input_rows(self):
        return self.w_in, None

    def drop_input_rows(self):
        self.w_in = None

    def forward_projected(self, projected, offset, x, scale, residual, step, cache):
        return ops.linear(self._features(x, step, cache, out_scale=scale, packed=projected, at=offset), self.w_o,
                          residual=residual)

    def _features(self, x, step, cache, out_scale=1.0, packed=None, at=0):
        s = self.spec
        nk, nv = s.num_heads * s.key_dim, s.num_heads * s.value_dim
        if packed is None:
            packed = ops.linear(x, self.w_in)                                        # [T, q | k | v | g]
        logits = ops.linear(ops.linear(x, self.w_a1), self.w_a2, bias=self.b_a2, out_float32=True)
        state = cache.state.unflatten(1, (s.num_heads, s.value_dim, s.key_dim))
        o = ops.linear_scan(packed, packed, packed, ops.ScanGate("sigmoid_power", logits, per_channel=True, tau=s.tau),
                            state=state, heads=s.num_heads, groups=s.num_heads, key_dim=s.key_dim, value_dim=s.value_dim,
                            q_offset=at, k_offset=at + nk, v_offset=at + 2 * nk, q_scale=s.key_dim ** -0.5,
                            cu_seqlens=step.cu_seqlens, state_slots=step.state_slots, num_seqs=step.num_seqs, max_q_len=step.max_q_len)
        return ops.gated_group_norm(o, packed, self.norm_w, group=s.value_dim, eps=s.norm_eps, gate_first=False,
                                    out_dtype=self.dtype, gate_offset=at + 2 * nk + nv, out_scale=out_scale)

    def forward(self, x, step, cache):
        return ops.linear(self._features(x, step, cache), self.w_o)

    def forward_residual(self, x, residual, step, cache):
        return ops.linear(self._features(x, step, cache), self.w_o, residual=residual)

    def forward_scaled(self, x, scale, residual, step, cache):
        return ops.linear(self._features(x, step, cache, out_scale=scale), self.w_o, residual=residual)


register_mixer("gated_linear_attention", GatedLinearAttention)
