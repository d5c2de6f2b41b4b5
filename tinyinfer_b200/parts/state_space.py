"""Selective state-space mixer with a scalar decay per head ("Transformers are SSMs", Dao and Gu, 2024): the input
projection gives [z | x | B | C | dt]; x, B and C pass a causal per-channel convolution with bias and silu;
dt = softplus(dt + dt_bias); per head S <- exp(-exp(A_log) dt) S + dt B x^T (state_dim x head_dim, B and C shared
by the heads of a group), y = S^T C + D x; y * silu(z) is divided by its root mean square in norm_groups equal
parts, weighted and projected.

Per request the mixer keeps, in its state slot, S (float32) and the convolution's last taps - 1 inputs. The step
sizes leave their product as float32; softplus, the decay, the recurrence, y and its norm are float32.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorSpec, register_mixer, state_slices


class StateSpace(Mixer):
    graph_safe = True

    def __init__(self, spec, dtype, device):
        super().__init__(spec, dtype, device)
        if spec.num_heads % spec.groups:
            raise ValueError(f"{spec.num_heads} heads do not split into {spec.groups} groups")
        if spec.inner_size % spec.norm_groups:
            raise ValueError(f"{spec.inner_size} features do not split into {spec.norm_groups} equal parts")
        self.w_main = self.w_dt = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.skip = None
        self.norm_w = self.w_o = None

    def _state_shapes(self):
        s = self.spec
        shapes = [(s.num_heads, s.head_dim, s.state_dim)]
        return shapes + [(s.conv_taps - 1, s.conv_size)] if s.conv_taps > 1 else shapes

    def state_need(self):
        s = self.spec
        return StateNeed((s.num_heads * s.head_dim * s.state_dim + (s.conv_taps - 1) * s.conv_size,), torch.float32)

    def tensors(self):
        s = self.spec
        return {"in": TensorSpec((s.inner_size + s.conv_size + s.num_heads, s.hidden_size)),
                "conv": TensorSpec((s.conv_size, s.conv_taps), role="vector32", init="ones_noise"),
                "conv.b": TensorSpec((s.conv_size,), role="vector32"),
                "dt_bias": TensorSpec((s.num_heads,), role="vector32"),
                "A_log": TensorSpec((s.num_heads,), role="vector32"),
                "D": TensorSpec((s.num_heads,), role="vector32", init="ones_noise"),
                "norm": TensorSpec((s.inner_size,), role="vector32", init="ones_noise"),
                "o": TensorSpec((s.hidden_size, s.inner_size))}

    def load(self, tensors):
        s = self.spec
        cut = s.inner_size + s.conv_size
        self.w_main = tensors["in"][:cut].contiguous()          # [z | x | B | C]
        self.w_dt = tensors["in"][cut:].contiguous()            # the step sizes: their product stays float32
        self.conv_w, self.conv_b = tensors["conv"].t().contiguous(), tensors["conv.b"]      # tap by tap, [taps, channels]
        self.dt_bias, self.a_log, self.skip = tensors["dt_bias"], tensors["A_log"], tensors["D"]
        self.norm_w, self.w_o = tensors["norm"], tensors["o"].contiguous()

    def _features(self, x, step, cache, out_scale=1.0):
        s = self.spec
        inner, gn = s.inner_size, s.groups * s.state_dim
        main = ops.linear(x, self.w_main)
        dt = ops.linear(x, self.w_dt, out_float32=True)                              # float32 [T, heads]
        state, history = (state_slices(cache.state, self._state_shapes()) + [None])[:2]
        single = step.num_tokens == step.num_seqs          # every request brings one token: the kernel keeps the history itself
        xbc = ops.short_conv(main, offset=inner, width=s.conv_size, history=history, weight=self.conv_w,
                             bias=self.conv_b, silu=True, token_seq=step.token_seq, cu_seqlens=step.cu_seqlens,
                             state_slots=step.state_slots, shift_history=single)
        if not single:
            ops.conv_state_update(history, main, offset=inner, width=s.conv_size, taps=s.conv_taps,
                                  cu_seqlens=step.cu_seqlens, state_slots=step.state_slots, num_seqs=step.num_seqs)
        gate = ops.ScanGate("step_size", dt, per_channel=False, a_log=self.a_log, dt_bias=self.dt_bias)
        y = ops.linear_scan(xbc, xbc, xbc, gate, state=state, heads=s.num_heads, groups=s.groups, key_dim=s.state_dim,
                            value_dim=s.head_dim, q_offset=inner + gn, k_offset=inner, v_offset=0, skip=self.skip,
                            cu_seqlens=step.cu_seqlens, state_slots=step.state_slots, num_seqs=step.num_seqs, max_q_len=step.max_q_len)
        return ops.gated_group_norm(y, main, self.norm_w, group=inner // s.norm_groups, eps=s.norm_eps, gate_first=True,
                                    out_dtype=self.dtype, gate_offset=0, out_scale=out_scale)

    def forward(self, x, step, cache):
        return ops.linear(self._features(x, step, cache), self.w_o)

    def forward_residual(self, x, residual, step, cache):
        return ops.linear(self._features(x, step, cache), self.w_o, residual=residual)

    def forward_scaled(self, x, scale, residual, step, cache):
        return ops.linear(self._features(x, step, cache, out_scale=scale), self.w_o, residual=residual)


register_mixer("state_space", StateSpace)
